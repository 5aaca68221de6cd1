// Soft-collision scorer: streams the uint8 bucket codes of every cached key and sums, per
// table, the query's probability mass on that bucket.
//
// Data movement: the scorer table of one (KV head, head tile) — R*L*ht floats, 128 KiB for
// R=256, L=32, ht=4 — is brought into shared memory once per CTA by bulk asynchronous copies
// (cp.async.bulk completing on an mbarrier); the code array is then streamed with 16-byte
// loads, one key (L bytes) per thread, and never re-read: all ht query heads of the KV head
// are scored from one pass.
//
// Shared-memory bandwidth is the limiter (one 16-byte word per key and table), so the
// lookups are arranged to be bank-conflict free for ht = 4: the table is stored
// [bucket][table][head], which puts table l in 16-byte bank group l mod 8, and the 8 lanes
// of a quarter warp walk the tables of each group of 8 in a different order
// (table = j ^ (key index & 7)), so that at every step they hit 8 distinct bank groups whatever
// the bucket values are.  The permutation is applied to the code bytes with two PRMTs per
// 8 bytes.  Consequence: the L terms of a score are added in a lane-dependent order; the
// result differs from the ascending-order sum by fp32 rounding only (~1e-7 relative).
#include "score_body.cuh"

namespace sk {
namespace {

// Shared memory after the table: mbarrier | per-head sample statistics for the filter mode.
constexpr int SC_SAMPLE_WARPS = 16;         // warps whose lanes score one sample key each
constexpr int SC_SAMPLES = 32 * SC_SAMPLE_WARPS;

struct FilterShared {
    uint64_t bar;
    uint32_t skey[4][SC_SAMPLES];          // per head: order keys of the sample scores
    float cut[4];
};

struct FilterArgs {
    int32_t* cnt;        // [rows][chunks_max][SC_WARPS]
    float* cut;          // [rows][chunks_max]
    uint2* cand;         // [rows][chunks_max][SC_WARPS][cap_w]  (score bits, key index)
    // The newest SC_TAIL keys of a row are not filtered: entry t - (T - SC_TAIL) of the row's tail
    // holds key t, whatever its score.  In a real model the keys just before the query score high
    // as a block (rotary position embedding, local context); compacted into their warp's run they
    // would overflow it and send the row to the rescoring path on every step.
    uint2* tail;         // [rows][SC_TAIL]
    int chunks_max, cap_w;
    float keep;          // keys the filter aims to keep per row: 3 * M (the fraction follows the LIVE length)
};

// Per-head cut from the SC_SAMPLES sample scores (one per thread of the first SC_SAMPLE_WARPS warps,
// sv[j]), such that the fraction `frac` of the samples lies at or above it: the r-th largest sample,
// r = frac * SC_SAMPLES, found exactly by one warp per head with a bitwise descent on the order keys
// (the low 8 key bits are left at zero, which can only lower the cut).  Any value would be correct
// (the select kernel proves or repairs the result); a cut above the row's k-th score costs the row a
// full rescoring, and with r around 3 k T^-1 SC_SAMPLES the chance of that is the chance that a third
// of the expected number of samples above the k-th score turns into all of them.
// The cuts are returned in cut[] and, for the select kernel's check, written to cut_out[j * cut_stride].
// Must be called by the whole CTA.
template <int HT>
__device__ __forceinline__ void filter_cuts(FilterShared& fs, const float (&sv)[HT], bool sampling, float frac,
                                            float* __restrict__ cut_out, size_t cut_stride, float (&cut)[HT]) {
    static_assert(HT <= 4 && SC_SAMPLES % 32 == 0, "one selecting warp per head");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (sampling) {
#pragma unroll
        for (int j = 0; j < HT; ++j) {
            const bool fin = sv[j] > -INFINITY && sv[j] < INFINITY;
            fs.skey[j][threadIdx.x] = fin ? order_key(sv[j]) : 0u;     // sampling threads are 0 .. SC_SAMPLES-1
        }
    }
    __syncthreads();
    if (warp < HT) {
        uint32_t k[SC_SAMPLES / 32];
#pragma unroll
        for (int i = 0; i < SC_SAMPLES / 32; ++i) k[i] = fs.skey[warp][lane + 32 * i];
        const int r = max(2, min(SC_SAMPLES / 2, (int)(frac * (float)SC_SAMPLES + 0.5f)));
        // the bits above the highest one in which two usable samples differ are common to all of them
        uint32_t kmx = 0u, kmn = 0xffffffffu;
#pragma unroll
        for (int i = 0; i < SC_SAMPLES / 32; ++i) {
            kmx = max(kmx, k[i]);
            if (k[i] != 0u) kmn = min(kmn, k[i]);
        }
        kmx = __reduce_max_sync(FULL, kmx);
        kmn = __reduce_min_sync(FULL, kmn);
        const int top = kmx > kmn ? 31 - __clz(kmx ^ kmn) : 7;          // first bit to decide
        uint32_t prefix = top < 31 ? (kmx >> (top + 1)) << (top + 1) : 0u;
        if (kmx == 0u) prefix = 0u;
        for (int bit = top; bit >= 8; --bit) {
            const uint32_t cand = prefix | (1u << bit);
            int c = 0;
#pragma unroll
            for (int i = 0; i < SC_SAMPLES / 32; ++i) c += k[i] >= cand;
            c = __reduce_add_sync(FULL, c);
            if (c >= r) prefix = cand;
        }
        if (lane == 0) fs.cut[warp] = prefix != 0u ? order_key_inverse(prefix) : -INFINITY;   // no usable sample: keep everything
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < HT; ++j) cut[j] = fs.cut[j];
    if (threadIdx.x < HT) cut_out[(size_t)threadIdx.x * cut_stride] = fs.cut[threadIdx.x];
}

// L: tables per key (bytes per key), HT: query heads per table word.
// FILTER = false: every score is written to `scores`.
// FILTER = true:  nothing is written for most keys.  Each CTA estimates, per head, a cut from
//   the first 32 keys of each of its warps (the mean of the warps' order statistics) that about
//   `frac` of the keys exceed, and every warp appends the (score, index) pairs >= cut to its own
//   run of the row's candidate buffer — runs are ordered (chunk, warp, index), so the candidates
//   of a row are in ascending index order without atomics.  The select kernel checks that the
//   k-th largest candidate is >= every chunk's cut, which proves the candidate set contains the
//   exact top-k; rows failing the check are rescored there.
template <int L, int HT, bool FILTER>
__global__ void __launch_bounds__(SC_THREADS, 1)
score_kernel(const float* __restrict__ lut, const uint8_t* __restrict__ codes,
             const __half* __restrict__ v_norm, const uint8_t* __restrict__ allowed,
             float* __restrict__ scores, int64_t score_row_stride, int H, int Hkv, int R,
             int64_t T, const int32_t* __restrict__ T_dev, int64_t Tcap, int64_t Tslots,
             int64_t slots_per_cta, int n_groups, int32_t* status, FilterArgs fa) {
    static_assert(L % 16 == 0, "codes are read 16 bytes at a time");
    static_assert(HT <= 4, "at most 4 heads per table word");
    constexpr int NV = L / 16;                 // uint4 per key
    constexpr int L_STRIDE = HT * 4;           // bytes between tables of one bucket
    constexpr int CODE_STRIDE = L * L_STRIDE;  // bytes between buckets
    extern __shared__ __align__(128) char smem_raw[];
    char* lut_s = smem_raw;
    // room for all 256 possible code values, so that no byte value can index past the table
    FilterShared& fs = *reinterpret_cast<FilterShared*>(smem_raw + (size_t)256 * CODE_STRIDE);
    uint64_t* bar = &fs.bar;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rep = H / Hkv;
    const int tiles = rep / HT;
    const uint32_t lut_bytes = (uint32_t)R * CODE_STRIDE;

    pdl_launch_dependents();
    if (threadIdx.x == 0) mbar_init(bar, 1);
    __syncthreads();
    pdl_wait();                                // the table, the live length and the newest codes come from the predecessor

    const int64_t total = (int64_t)n_groups * Tslots;
    int64_t slot = (int64_t)blockIdx.x * slots_per_cta;
    const int64_t slot_end = min(slot + slots_per_cta, total);
    uint32_t phase = 0;
    auto request_table = [&](int g) {          // one thread: bulk copies of group g's table, completing on `bar`
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_expect_tx(bar, lut_bytes);
        const char* src = reinterpret_cast<const char*>(lut) + (size_t)g * lut_bytes;
        for (uint32_t off = 0; off < lut_bytes; off += SC_COPY_CHUNK) {
            const uint32_t n = min((uint32_t)SC_COPY_CHUNK, lut_bytes - off);
            bulk_g2s(lut_s + off, src + off, n, bar);
        }
    };
    // the table of the first segment is requested before the live length has arrived
    bool in_flight = slot < slot_end;
    if (in_flight && threadIdx.x == 0) request_table((int)(slot / Tslots));
    const int Teff = effective_len(T, T_dev);

    while (slot < slot_end) {
        const int g = (int)(slot / Tslots);
        const int64_t t0 = slot - (int64_t)g * Tslots;
        const int64_t seg_end = min((int64_t)(g + 1) * Tslots, slot_end);
        int64_t t1 = seg_end - (int64_t)g * Tslots;
        slot = seg_end;
        if (t1 > Teff) t1 = Teff;

        const int tile = g % tiles;
        const int bk = g / tiles;               // b*Hkv + kvh
        const int b = bk / Hkv, kvh = bk - b * Hkv;
        const int h0 = kvh * rep + tile * HT;
        const size_t row0 = (size_t)b * H + h0;
        const int chunk = (int)((int64_t)blockIdx.x - ((int64_t)g * Tslots) / slots_per_cta);

        if (t0 >= t1) {   // uniform across the CTA: nothing live in this segment
            if (FILTER) {
                if (threadIdx.x < SC_WARPS * HT) {
                    const int j = threadIdx.x / SC_WARPS, w = threadIdx.x % SC_WARPS;
                    fa.cnt[((row0 + j) * fa.chunks_max + chunk) * SC_WARPS + w] = 0;
                }
                if (threadIdx.x < HT) fa.cut[(row0 + threadIdx.x) * fa.chunks_max + chunk] = -INFINITY;
            }
            if (in_flight) {   // its table was requested all the same: let the copy land before the barrier is reused
                const bool landed = mbar_wait(bar, phase);
                phase ^= 1u;
                in_flight = false;
                if (!__syncthreads_and(landed)) {
                    if (threadIdx.x == 0 && status != nullptr) atomicOr(status, SK_DEV_WAIT_TIMEOUT);
                    return;
                }
            }
            continue;
        }

        if (!in_flight) {
            // previous segment's lookups are done before the table is overwritten
            __syncthreads();
            if (threadIdx.x == 0) request_table(g);
        }
        in_flight = false;

        // each warp owns a contiguous run of keys (a multiple of 32 long)
        // (of the LIVE keys of the segment: a partly filled segment still spreads over all warps, so
        // that its sample comes from all warps as soon as it has a thousand keys)
        const int per_warp = (int)(((t1 - t0 + SC_WARPS - 1) / SC_WARPS + 31) / 32 * 32);
        const int ws = (int)t0 + warp * per_warp;
        const int we = min((int)t1, ws + per_warp);
        // table order of a key depends on its index only: table = j ^ (t & 7) inside each group of
        // 8, so that any 8 consecutive keys (a quarter warp) hit 8 distinct bank groups; the lane's
        // keys are 32 apart, hence one permutation per lane and segment
        const int m = (ws + lane) & 7;
        const uint32_t sel_lo = 0x3210u ^ (0x1111u * m);
        const uint32_t sel_hi = 0x7654u ^ (0x1111u * m);
        const uint32_t mL = (uint32_t)m * L_STRIDE;
        const uint4* cg = reinterpret_cast<const uint4*>(codes + (size_t)bk * Tcap * L);
        const __half* vg = v_norm + (size_t)bk * Tcap;

        uint4 cur[NV], nxt[NV];
        __half vcur = __float2half(0.f), vnxt = __float2half(0.f);   // ||v|| travels with the codes
        int t = ws + lane;
        if (FILTER) {
            // the sample: 512 keys spread evenly over the WHOLE row (sampling thread i takes key
            // (i + 1/2) * T / 512, a warp's 32 samples interleaved over the row), the same keys in every
            // CTA of the row.  Every chunk then cuts at the same score, about 3 M keys of the row pass
            // whatever their positions are, and a region of high scores (recent tokens in a real
            // model) does not get a cut of its own above the row's k-th score.
            if (warp < SC_SAMPLE_WARPS) {
                const int ts = (int)(((int64_t)(2 * (lane * SC_SAMPLE_WARPS + warp) + 1) * Teff) / (64 * SC_SAMPLE_WARPS));
#pragma unroll
                for (int i = 0; i < NV; ++i) cur[i] = __ldcg(cg + (size_t)ts * NV + i);
                vcur = __ldcg(vg + ts);
            }
            if (t < we) {                      // the warp's first own key rides behind the sample
#pragma unroll
                for (int i = 0; i < NV; ++i) nxt[i] = __ldcg(cg + (size_t)t * NV + i);
                vnxt = __ldcg(vg + t);
            }
        } else {
            if (t < we) {
#pragma unroll
                for (int i = 0; i < NV; ++i) cur[i] = __ldcg(cg + (size_t)t * NV + i);
                vcur = __ldcg(vg + t);
            }
            if (t + 32 < we) {
#pragma unroll
                for (int i = 0; i < NV; ++i) nxt[i] = __ldcg(cg + (size_t)(t + 32) * NV + i);
                vnxt = __ldcg(vg + t + 32);
            }
        }

        const bool ok = mbar_wait(bar, phase);
        phase ^= 1u;
        if (!__syncthreads_and(ok)) {
            if (threadIdx.x == 0 && status != nullptr) atomicOr(status, SK_DEV_WAIT_TIMEOUT);
            return;
        }

        uint32_t cnt4 = 0;            // four 8-bit run lengths, saturating at 255 (cap_w <= 250)
        const int tail_start = max(Teff - SC_TAIL, 0);
        float cutv[HT];
#pragma unroll
        for (int j = 0; j < HT; ++j) cutv[j] = -INFINITY;
        // this warp's run of head j starts at entry run_index0 + j * run_stride of the candidate buffer
        // (32-bit entry indices: the buffer holds far fewer than 2^31 entries)
        const int run_stride = fa.chunks_max * SC_WARPS * fa.cap_w;
        const int run_index0 = FILTER ? (((int)row0 * fa.chunks_max + chunk) * SC_WARPS + warp) * fa.cap_w : 0;

        if (FILTER) {
            // ---- the row-wide sample: scores, cut
            float sv[HT];
#pragma unroll
            for (int j = 0; j < HT; ++j) sv[j] = 0.f;
            if (warp < SC_SAMPLE_WARPS) {           // warp-uniform
                float acc[HT];
                score_key<L, HT>(cur, lut_s, sel_lo, sel_hi, mL, acc);
                const float vn = __half2float(vcur);
#pragma unroll
                for (int j = 0; j < HT; ++j) sv[j] = acc[j] * vn;
            }
            // a short segment (the newest keys of a partly filled chunk, or the few keys a CTA has on
            // one side of a KV-head boundary) keeps everything when its runs have the room
            if (t1 - t0 <= 1024 && 2 * (t1 - t0) <= slots_per_cta && per_warp <= fa.cap_w) {   // uniform across the CTA
                if (threadIdx.x < HT) fa.cut[(row0 + threadIdx.x) * fa.chunks_max + chunk] = -INFINITY;
            } else {
                // the kept fraction is taken of the live length: the capacity the plan was made for may
                // be several times larger, and a cut for 3M / capacity would drop needed keys
                filter_cuts<HT>(fs, sv, warp < SC_SAMPLE_WARPS, fminf(__fdividef(fa.keep, (float)Teff), 1.0f), fa.cut + row0 * fa.chunks_max + chunk, (size_t)fa.chunks_max, cutv);
            }
            // on to the warp's own keys
#pragma unroll
            for (int i = 0; i < NV; ++i) cur[i] = nxt[i];
            vcur = vnxt;
            if (t + 32 < we) {
#pragma unroll
                for (int i = 0; i < NV; ++i) nxt[i] = __ldcg(cg + (size_t)(t + 32) * NV + i);
                vnxt = __ldcg(vg + t + 32);
            }
        }

        // ---- main loop over this warp's keys, codes double-buffered in registers
        for (; t - lane < we; t += 32) {
            const bool valid = t < we;
            float sv[HT];
            if (valid) {
                float acc[HT];
                score_key<L, HT>(cur, lut_s, sel_lo, sel_hi, mL, acc);
                const float vn = __half2float(vcur);
#pragma unroll
                for (int j = 0; j < HT; ++j) sv[j] = acc[j] * vn;
            }
            if (FILTER) {
                const bool in_tail = valid && t >= tail_start;
                if (in_tail) {
#pragma unroll
                    for (int j = 0; j < HT; ++j)
                        fa.tail[(row0 + j) * SC_TAIL + (t - tail_start)] = make_uint2(__float_as_uint(sv[j]), (uint32_t)t);
                }
#pragma unroll
                for (int j = 0; j < HT; ++j) {
                    const bool hit = valid && !in_tail && sv[j] >= cutv[j];
                    const unsigned bal = __ballot_sync(FULL, hit);
                    if (bal != 0u) {                              // warp-uniform
                        const int have = (int)((cnt4 >> (8 * j)) & 0xffu);
                        const int pos = have + __popc(bal & ((1u << lane) - 1u));
                        if (hit && pos < fa.cap_w)
                            fa.cand[(size_t)(run_index0 + j * run_stride + pos)] =
                                make_uint2(__float_as_uint(sv[j]), (uint32_t)t);
                        cnt4 += (uint32_t)min(__popc(bal), 255 - have) << (8 * j);
                    }
                }
            } else if (valid) {
#pragma unroll
                for (int j = 0; j < HT; ++j) {
                    float sc = sv[j];
                    if (allowed != nullptr && allowed[(row0 + j) * T + t] == 0) sc = -INFINITY;
                    scores[(row0 + j) * score_row_stride + t] = sc;
                }
            }
#pragma unroll
            for (int i = 0; i < NV; ++i) cur[i] = nxt[i];
            vcur = vnxt;
            if (t + 64 < we) {
#pragma unroll
                for (int i = 0; i < NV; ++i) nxt[i] = __ldcg(cg + (size_t)(t + 64) * NV + i);
                vnxt = __ldcg(vg + t + 64);
            }
        }
        if (FILTER && lane == 0) {
#pragma unroll
            for (int j = 0; j < HT; ++j)
                fa.cnt[((row0 + j) * fa.chunks_max + chunk) * SC_WARPS + warp] = (int32_t)((cnt4 >> (8 * j)) & 0xffu);
        }
    }
}

// ------------------------------------------------------------------------------------------
// Packed mode of the filtering scorer (L = 32 tables, 4 query heads per KV-head group).
//
// The fp32 walk above is bound by shared-memory bandwidth (16 bytes per key and table) with the
// integer pipe close behind.  Here the table is the 12-bit fixed-point copy written by the soft
// hash (soft_hash_body.cuh): 8 bytes per (bucket, table) = four 16-bit fields, one per head.  A
// key's sum over 16 tables fits a 16-bit field (16 * 4095 < 65536), so the four heads are summed
// as two packed 32-bit integers per half of the tables - two adds per lookup instead of four, half
// the shared-memory bytes, and no rounding at all: the sums S are exact integers.
//
// What is written per kept key is (S, ||v||) packed into 32 bits, from which scorer and select
// kernel compute the same upper bound  U = (S + K0 + 33) * ||v||  of C * (exact fp32 score); keys
// with U >= the chunk's cut are kept.  The select kernel brackets the k-th exact score with these
// bounds, rescans only the few keys inside the bracket with the fp32 table, and so returns exactly
// the list the fp32 path returns.
//
// Lookups: one LDS.64 per (key, table).  The table lies at a 64 KiB-aligned shared address, one
// 256-byte line per bucket (32 tables x 8 bytes), so a lookup address is
// [8 * table | code | address bits 16..23 | 0] byte by byte and ONE byte permute builds it from
// the register holding the code byte and a per-lane constant.  The 16 lanes of a half warp (one
// shared-memory wavefront of 8-byte accesses) visit, at step p, the tables (p ^ lane) of the
// current half of the tables: 16 distinct bank pairs whatever the codes are.
constexpr int PK_SMEM = 129 * 1024;

__device__ __forceinline__ uint32_t prmt_r(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
template <uint32_t SEL>
__device__ __forceinline__ uint32_t prmt_i(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "n"(SEL));
    return d;
}
// volatile: ordered with the mbarrier wait that guards the table
template <int IMM>
__device__ __forceinline__ void lds64(uint32_t addr, uint32_t& x, uint32_t& y) {
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(x), "=r"(y) : "r"(addr), "n"(IMM));
}
__device__ __forceinline__ void ldg256(const uint8_t* p, uint32_t (&c)[8]) {
    asm volatile("ld.global.cg.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]), "=r"(c[4]), "=r"(c[5]), "=r"(c[6]), "=r"(c[7])
                 : "l"(p));
}

// One half of the tables (16 code bytes in w[0..3]): 16 lookups, packed adds into (a, b).
template <int IMM>
__device__ __forceinline__ void packed_half(const uint32_t* w, bool swap, uint32_t sel_lo, uint32_t sel_hi,
                                            const uint32_t (&X)[6], uint32_t& a, uint32_t& b) {
    // position p of the permuted vector holds the code of table (p ^ m): bit 3 of m swaps the
    // 8-byte halves, bits 0..2 permute inside a half
    const uint32_t h0a = swap ? w[2] : w[0], h0b = swap ? w[3] : w[1];
    const uint32_t h1a = swap ? w[0] : w[2], h1b = swap ? w[1] : w[3];
    uint32_t pv[4];
    pv[0] = prmt_r(h0a, h0b, sel_lo);
    pv[1] = prmt_r(h0a, h0b, sel_hi);
    pv[2] = prmt_r(h1a, h1b, sel_lo);
    pv[3] = prmt_r(h1a, h1b, sel_hi);
    uint32_t x[16], y[16];
#define SK_PK_LOOKUP(P)                                                                             \
    lds64<IMM>(prmt_i<0xF700u | (((P) & 3) << 4) | (4 + (P) % 3)>(pv[(P) >> 2], X[(P) / 3]), x[P], y[P])
    SK_PK_LOOKUP(0); SK_PK_LOOKUP(1); SK_PK_LOOKUP(2); SK_PK_LOOKUP(3);
    SK_PK_LOOKUP(4); SK_PK_LOOKUP(5); SK_PK_LOOKUP(6); SK_PK_LOOKUP(7);
    SK_PK_LOOKUP(8); SK_PK_LOOKUP(9); SK_PK_LOOKUP(10); SK_PK_LOOKUP(11);
    SK_PK_LOOKUP(12); SK_PK_LOOKUP(13); SK_PK_LOOKUP(14); SK_PK_LOOKUP(15);
#undef SK_PK_LOOKUP
    a = 0; b = 0;
#pragma unroll
    for (int p = 0; p < 16; p += 2) {
        a += x[p] + x[p + 1];
        b += y[p] + y[p + 1];
    }
}

// Upper bound, in table units times ||v||, of a key's exact score; computed with exactly these
// operations by the scorer and by the select kernel.
__device__ __forceinline__ float packed_upper(uint32_t S, float K0p, float vn) {
    return __fmul_rn(__fadd_rn(__uint2float_rn(S), K0p), vn);
}

__global__ void __launch_bounds__(SC_THREADS, 1)
score_packed_kernel(const uint8_t* __restrict__ lutq, const float* __restrict__ qpar,
                    const uint8_t* __restrict__ codes, const __half* __restrict__ v_norm, int H, int Hkv, int R,
                    int64_t T, const int32_t* __restrict__ T_dev, int64_t Tcap, int64_t Tslots,
                    int64_t slots_per_cta, int n_groups, int32_t* status, FilterArgs fa) {
    constexpr int L = 32, HT = 4;
    extern __shared__ __align__(1024) char smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t tab = (base + 0xffffu) & ~0xffffu;          // shared address of the table, 64 KiB aligned
    char* lut_s = smem_raw + (tab - base);
    // the statistics block sits in front of the table when the alignment gap has room, else behind it
    FilterShared& fs = *reinterpret_cast<FilterShared*>((tab - base) >= 1024 ? smem_raw : lut_s + 65536);
    uint64_t* bar = &fs.bar;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rep = H / Hkv;
    const int tiles = rep / HT;
    const uint32_t lut_bytes = (uint32_t)R * 256u;

    pdl_launch_dependents();
    if (threadIdx.x == 0) mbar_init(bar, 1);
    __syncthreads();
    pdl_wait();                                // the table, the live length and the newest codes come from the predecessor

    const int64_t total = (int64_t)n_groups * Tslots;
    int64_t slot = (int64_t)blockIdx.x * slots_per_cta;
    const int64_t slot_end = min(slot + slots_per_cta, total);
    uint32_t phase = 0;
    auto request_table = [&](int g) {          // one thread: bulk copies of group g's table, completing on `bar`
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_expect_tx(bar, lut_bytes);
        const char* src = reinterpret_cast<const char*>(lutq) + (size_t)g * 65536;
        for (uint32_t off = 0; off < lut_bytes; off += SC_COPY_CHUNK) {
            const uint32_t n = min((uint32_t)SC_COPY_CHUNK, lut_bytes - off);
            bulk_g2s(lut_s + off, src + off, n, bar);
        }
    };
    bool in_flight = slot < slot_end;
    if (in_flight && threadIdx.x == 0) request_table((int)(slot / Tslots));
    const int Teff = effective_len(T, T_dev);

    while (slot < slot_end) {
        const int g = (int)(slot / Tslots);
        const int64_t t0 = slot - (int64_t)g * Tslots;
        const int64_t seg_end = min((int64_t)(g + 1) * Tslots, slot_end);
        int64_t t1 = seg_end - (int64_t)g * Tslots;
        slot = seg_end;
        if (t1 > Teff) t1 = Teff;

        const int tile = g % tiles;
        const int bk = g / tiles;               // b*Hkv + kvh
        const int b = bk / Hkv, kvh = bk - b * Hkv;
        const int h0 = kvh * rep + tile * HT;
        const size_t row0 = (size_t)b * H + h0;
        const int chunk = (int)((int64_t)blockIdx.x - ((int64_t)g * Tslots) / slots_per_cta);

        if (t0 >= t1) {   // uniform across the CTA: nothing live in this segment
            if (threadIdx.x < SC_WARPS * HT) {
                const int j = threadIdx.x / SC_WARPS, w = threadIdx.x % SC_WARPS;
                fa.cnt[((row0 + j) * fa.chunks_max + chunk) * SC_WARPS + w] = 0;
            }
            if (threadIdx.x < HT) fa.cut[(row0 + threadIdx.x) * fa.chunks_max + chunk] = -INFINITY;
            if (in_flight) {   // its table was requested all the same: let the copy land before the barrier is reused
                const bool landed = mbar_wait(bar, phase);
                phase ^= 1u;
                in_flight = false;
                if (!__syncthreads_and(landed)) {
                    if (threadIdx.x == 0 && status != nullptr) atomicOr(status, SK_DEV_WAIT_TIMEOUT);
                    return;
                }
            }
            continue;
        }

        if (!in_flight) {
            __syncthreads();                    // previous segment's lookups are done before the table is overwritten
            if (threadIdx.x == 0) request_table(g);
        }
        in_flight = false;
        const float K0p = __ldcg(qpar + g) + 33.0f;

        // each warp owns a contiguous run of the segment's live keys (a multiple of 32 long)
        const int per_warp = (int)(((t1 - t0 + SC_WARPS - 1) / SC_WARPS + 31) / 32 * 32);
        const int ws = (int)t0 + warp * per_warp;
        const int we = min((int)t1, ws + per_warp);
        // the lane's keys are 32 apart, so its visiting order (key index & 15) is fixed per segment
        const uint32_t m = (uint32_t)(ws + lane) & 15u;
        const uint32_t sel_lo = 0x3210u ^ (0x1111u * (m & 7u));
        const uint32_t sel_hi = 0x7654u ^ (0x1111u * (m & 7u));
        const bool swap = (m & 8u) != 0u;
        uint32_t X[6];
#pragma unroll
        for (int i = 0; i < 6; ++i) {
            uint32_t v = (tab >> 16) << 24;
#pragma unroll
            for (int c = 0; c < 3; ++c) {
                const uint32_t p = (uint32_t)(3 * i + c);
                if (p < 16u) v |= (8u * (p ^ m)) << (8 * c);
            }
            X[i] = v;
        }
        const uint8_t* cg = codes + (size_t)bk * Tcap * L;
        const __half* vg = v_norm + (size_t)bk * Tcap;

        uint32_t cur[8], nxt[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) cur[i] = nxt[i] = 0u;
        uint16_t vcur = 0, vnxt = 0;                                 // ||v|| (fp16 bits) travels with the codes
        int t = ws + lane;
        {
            // the sample: 512 keys spread evenly over the whole row, the same in every CTA of the row
            // (see score_kernel); the warp's first own key rides behind it
            if (warp < SC_SAMPLE_WARPS) {
                const int ts = (int)(((int64_t)(2 * (lane * SC_SAMPLE_WARPS + warp) + 1) * Teff) / (64 * SC_SAMPLE_WARPS));
                ldg256(cg + (size_t)ts * L, cur);
                vcur = __ldcg(reinterpret_cast<const uint16_t*>(vg) + ts);
            }
            if (t < we) {
                ldg256(cg + (size_t)t * L, nxt);
                vnxt = __ldcg(reinterpret_cast<const uint16_t*>(vg) + t);
            }
        }

        const bool ok = mbar_wait(bar, phase);
        phase ^= 1u;
        if (!__syncthreads_and(ok)) {
            if (threadIdx.x == 0 && status != nullptr) atomicOr(status, SK_DEV_WAIT_TIMEOUT);
            return;
        }

        uint32_t cnt4 = 0;            // four 8-bit run lengths, saturating at 255 (cap_w <= 250)
        const int tail_start = max(Teff - SC_TAIL, 0);
        float cutv[HT];
#pragma unroll
        for (int j = 0; j < HT; ++j) cutv[j] = -INFINITY;
        const int run_stride = fa.chunks_max * SC_WARPS * fa.cap_w;
        const int run_index0 = (((int)row0 * fa.chunks_max + chunk) * SC_WARPS + warp) * fa.cap_w;

        // scores of the key held in cur/vcur: the packed entries and the upper bounds
        auto score_cur = [&](uint32_t (&pk)[HT], float (&sv)[HT]) {
            uint32_t a0, b0, a1, b1;
            packed_half<0>(cur, swap, sel_lo, sel_hi, X, a0, b0);
            packed_half<128>(cur + 4, swap, sel_lo, sel_hi, X, a1, b1);
            const uint32_t S[HT] = {(a0 & 0xffffu) + (a1 & 0xffffu), (a0 >> 16) + (a1 >> 16),
                                    (b0 & 0xffffu) + (b1 & 0xffffu), (b0 >> 16) + (b1 >> 16)};
            const uint32_t vb = (uint32_t)vcur & 0x7fffu;
            const float vn = __half2float(__ushort_as_half((unsigned short)vb));
#pragma unroll
            for (int j = 0; j < HT; ++j) {
                sv[j] = packed_upper(S[j], K0p, vn);
                pk[j] = (S[j] << 15) | vb;
            }
        };
        auto keep = [&](const uint32_t (&pk)[HT], const float (&sv)[HT], bool valid, int tk) {
            const bool in_tail = valid && tk >= tail_start;
            if (in_tail) {                                    // the row's newest keys are kept unfiltered
#pragma unroll
                for (int j = 0; j < HT; ++j)
                    fa.tail[(row0 + j) * SC_TAIL + (tk - tail_start)] = make_uint2(pk[j], (uint32_t)tk);
            }
#pragma unroll
            for (int j = 0; j < HT; ++j) {
                const bool hit = valid && !in_tail && sv[j] >= cutv[j];
                const unsigned bal = __ballot_sync(FULL, hit);
                if (bal != 0u) {                              // warp-uniform
                    const int have = (int)((cnt4 >> (8 * j)) & 0xffu);
                    const int pos = have + __popc(bal & ((1u << lane) - 1u));
                    if (hit && pos < fa.cap_w)
                        fa.cand[(size_t)(run_index0 + j * run_stride + pos)] = make_uint2(pk[j], (uint32_t)tk);
                    cnt4 += (uint32_t)min(__popc(bal), 255 - have) << (8 * j);
                }
            }
        };

        {
            // ---- the row-wide sample: scores, cut
            float sv[HT];
            uint32_t pk[HT];
#pragma unroll
            for (int j = 0; j < HT; ++j) sv[j] = 0.f;
            if (warp < SC_SAMPLE_WARPS) score_cur(pk, sv);          // warp-uniform
            if (t1 - t0 <= 1024 && 2 * (t1 - t0) <= slots_per_cta && per_warp <= fa.cap_w) {   // uniform across the CTA
                if (threadIdx.x < HT) fa.cut[(row0 + threadIdx.x) * fa.chunks_max + chunk] = -INFINITY;
            } else {
                filter_cuts<HT>(fs, sv, warp < SC_SAMPLE_WARPS, fminf(__fdividef(fa.keep, (float)Teff), 1.0f),
                                fa.cut + row0 * fa.chunks_max + chunk, (size_t)fa.chunks_max, cutv);
            }
        }
        // on to the warp's own keys
#pragma unroll
        for (int i = 0; i < 8; ++i) cur[i] = nxt[i];
        vcur = vnxt;
        if (t + 32 < we) {
            ldg256(cg + (size_t)(t + 32) * L, nxt);
            vnxt = __ldcg(reinterpret_cast<const uint16_t*>(vg) + t + 32);
        }
        for (; t - lane < we; t += 32) {
            const bool valid = t < we;
            float sv[HT];
            uint32_t pk[HT];
            score_cur(pk, sv);
            keep(pk, sv, valid, t);
#pragma unroll
            for (int i = 0; i < 8; ++i) cur[i] = nxt[i];
            vcur = vnxt;
            if (t + 64 < we) {
                ldg256(cg + (size_t)(t + 64) * L, nxt);
                vnxt = __ldcg(reinterpret_cast<const uint16_t*>(vg) + t + 64);
            }
        }
        if (lane == 0) {
#pragma unroll
            for (int j = 0; j < HT; ++j)
                fa.cnt[((row0 + j) * fa.chunks_max + chunk) * SC_WARPS + warp] = (int32_t)((cnt4 >> (8 * j)) & 0xffu);
        }
    }
}

// Reference-surface scorer: [B,H,L,T] int16 codes, ascending-table summation.
__global__ void __launch_bounds__(256)
score_compat_kernel(const float* __restrict__ q_probs, const int16_t* __restrict__ key_buckets,
                    const uint8_t* __restrict__ allowed, const float* __restrict__ v_hist,
                    float* __restrict__ out, int L, int R, int64_t T, int use_smem) {
    extern __shared__ float qp_s[];
    const int bh = blockIdx.y;
    const float* qp = q_probs + (size_t)bh * L * R;
    if (use_smem) {
        for (int i = threadIdx.x; i < L * R; i += blockDim.x) qp_s[i] = qp[i];
        __syncthreads();
    }
    const int16_t* kb = key_buckets + (size_t)bh * L * T;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < T;
         t += (int64_t)gridDim.x * blockDim.x) {
        const size_t o = (size_t)bh * T + t;
        if (allowed[o] == 0) {
            out[o] = -INFINITY;
            continue;
        }
        float s = 0.f;
        for (int l = 0; l < L; ++l) {
            const int r = (int)kb[(size_t)l * T + t];
            s += use_smem ? qp_s[l * R + r] : __ldg(qp + (size_t)l * R + r);
        }
        out[o] = s * v_hist[o];
    }
}

template <int L, int HT, bool FILTER>
int score_launch(const float* lut, const uint8_t* codes, const uint16_t* v_norm,
                 const uint8_t* allowed, int B, int H, int Hkv, int R, int64_t T,
                 const int32_t* T_dev, int64_t Tcap, float* scores, int64_t srs, int32_t* status,
                 const ScorePlan& plan, FilterArgs fa, cudaStream_t st) {
    const int rep = H / Hkv;
    const int n_groups = B * Hkv * (rep / HT);
    const size_t smem = (size_t)256 * L * HT * 4 + sizeof(FilterShared);
    auto kern = score_kernel<L, HT, FILTER>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(SK_ERR_CUDA, "score_kernel smem attribute: %s", cudaGetErrorString(e));
    e = launch_chained(kern, dim3((unsigned)plan.grid), dim3(SC_THREADS), smem, st, lut, codes, (const __half*)v_norm, allowed, scores,
                                                        srs, H, Hkv, R, T, T_dev, Tcap, plan.Tslots,
                                                        plan.per_cta, n_groups, status, fa);
    if (e != cudaSuccess) return fail(SK_ERR_CUDA, "score_kernel: %s", cudaGetErrorString(e));
    return check_launch("score_kernel");
}

}  // namespace

bool score_shape_supported(int L, int ht, int R) {
    if (R > 256 || (size_t)256 * L * ht * 4 + sizeof(FilterShared) > 227 * 1024) return false;
    if (L == 32 || L == 16) return ht == 4 || ht == 2 || ht == 1;
    if (L == 64) return ht == 2 || ht == 1;
    return false;
}

int launch_score(const float* lut, const uint8_t* codes, const uint16_t* v_norm,
                 const uint8_t* allowed, int B, int H, int Hkv, int L, int R, int64_t T,
                 const int32_t* T_dev, int64_t Tcap, float* scores, int64_t score_row_stride,
                 int32_t* status, cudaStream_t st) {
    if (T <= 0 || B * H == 0) return SK_OK;
    const int ht = lut_head_tile(H / Hkv);
    if ((size_t)256 * L * ht * 4 + sizeof(FilterShared) > 227 * 1024)
        return fail(SK_ERR_UNSUPPORTED, "sk_score: table of R=%d L=%d does not fit shared memory", R, L);
    const ScorePlan plan = make_score_plan(B * Hkv * ((H / Hkv) / ht), T, 0);
    FilterArgs none{};
#define SK_SCORE_CASE(LL, HT)                                                                    \
    if (L == LL && ht == HT)                                                                     \
        return score_launch<LL, HT, false>(lut, codes, v_norm, allowed, B, H, Hkv, R, T, T_dev,  \
                                           Tcap, scores, score_row_stride, status, plan, none, st)
    SK_SCORE_CASE(32, 4);
    SK_SCORE_CASE(32, 2);
    SK_SCORE_CASE(32, 1);
    SK_SCORE_CASE(16, 4);
    SK_SCORE_CASE(16, 2);
    SK_SCORE_CASE(16, 1);
    SK_SCORE_CASE(64, 2);
    SK_SCORE_CASE(64, 1);
#undef SK_SCORE_CASE
    return fail(SK_ERR_UNSUPPORTED, "sk_score: L=%d with %d heads per KV head not supported", L, H / Hkv);
}

size_t score_select_workspace_bytes(int B, int H, int Hkv, int L, int64_t T, int64_t M) {
    (void)L;
    if (B <= 0 || H <= 0 || Hkv <= 0 || T <= 0) return 256;
    const int ht = lut_head_tile(H / Hkv);
    const ScorePlan plan = make_score_plan(B * Hkv * ((H / Hkv) / ht), T, M);
    return make_fused_layout((int64_t)B * H, plan, T).total;
}

bool packed_filter_applicable(int H, int Hkv, int L, int R) {
    return Hkv > 0 && H % Hkv == 0 && L == 32 && R == 256 && lut_head_tile(H / Hkv) == 4;
}

int launch_score_filter(const float* lut, const uint8_t* codes, const uint16_t* v_norm, int B, int H,
                        int Hkv, int L, int R, int64_t T, const int32_t* T_dev, int64_t Tcap, int64_t M,
                        void* workspace, int32_t* status, cudaStream_t st, const void* lutq, const float* qpar) {
    const int ht = lut_head_tile(H / Hkv);
    const ScorePlan plan = make_score_plan(B * Hkv * ((H / Hkv) / ht), T, M);
    const FusedLayout lay = make_fused_layout((int64_t)B * H, plan, T);
    char* ws = static_cast<char*>(workspace);
    FilterArgs fa;
    fa.cnt = reinterpret_cast<int32_t*>(ws + lay.cnt);
    fa.cut = reinterpret_cast<float*>(ws + lay.cut);
    fa.cand = reinterpret_cast<uint2*>(ws + lay.cand);
    fa.tail = reinterpret_cast<uint2*>(ws + lay.tail);
    fa.chunks_max = plan.chunks_max;
    fa.cap_w = plan.cap_w;
    fa.keep = plan.frac * (float)T;
    if (lutq != nullptr) {
        if (!packed_filter_applicable(H, Hkv, L, R) || qpar == nullptr)
            return fail(SK_ERR_UNSUPPORTED, "packed scorer: needs L=32, R=256 and a multiple of 4 query heads per KV head");
        if (reinterpret_cast<uintptr_t>(codes) % 32 != 0 || reinterpret_cast<uintptr_t>(lutq) % 16 != 0)
            return fail(SK_ERR_MISALIGNED, "packed scorer: codes must be 32-byte aligned, the table 16-byte aligned");
        cudaError_t e = cudaFuncSetAttribute(score_packed_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PK_SMEM);
        if (e != cudaSuccess) return fail(SK_ERR_CUDA, "score_packed_kernel smem attribute: %s", cudaGetErrorString(e));
        const int n_groups = B * Hkv * ((H / Hkv) / 4);
        e = launch_chained(score_packed_kernel, dim3((unsigned)plan.grid), dim3(SC_THREADS), (size_t)PK_SMEM, st,
                           (const uint8_t*)lutq, qpar, codes, (const __half*)v_norm, H, Hkv, R, T, T_dev, Tcap,
                           plan.Tslots, plan.per_cta, n_groups, status, fa);
        if (e != cudaSuccess) return fail(SK_ERR_CUDA, "score_packed_kernel: %s", cudaGetErrorString(e));
        return check_launch("score_packed_kernel");
    }
#define SK_SCORE_CASE(LL, HT)                                                                      \
    if (L == LL && ht == HT)                                                                       \
        return score_launch<LL, HT, true>(lut, codes, v_norm, nullptr, B, H, Hkv, R, T, T_dev, Tcap, \
                                          nullptr, 0, status, plan, fa, st)
    SK_SCORE_CASE(32, 4);
    SK_SCORE_CASE(32, 2);
    SK_SCORE_CASE(32, 1);
#undef SK_SCORE_CASE
    return fail(SK_ERR_UNSUPPORTED, "fused scorer: L=%d with %d heads per KV head not supported", L, H / Hkv);
}

int launch_score_compat(const float* q_probs, const int16_t* key_buckets, const uint8_t* allowed,
                        const float* v_hist, float* out, int B, int H, int L, int R, int64_t T,
                        cudaStream_t st) {
    if (T <= 0 || B * H == 0) return SK_OK;
    const size_t smem = (size_t)L * R * 4;
    const int use_smem = smem <= 160 * 1024;
    if (use_smem && smem > 48 * 1024)
        cudaFuncSetAttribute(score_compat_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    int64_t gx = (T + 255) / 256;
    if (gx > 1024) gx = 1024;
    dim3 grid((unsigned)gx, (unsigned)(B * H));
    score_compat_kernel<<<grid, 256, use_smem ? smem : 0, st>>>(q_probs, key_buckets, allowed, v_hist,
                                                                out, L, R, T, use_smem);
    return check_launch("score_compat_kernel");
}

}  // namespace sk
