// Top-k select + sparse-list assembly, one CTA per (batch, query head) row.
//
// Exact selection on order-preserving uint32 keys with deterministic tie-breaking (among
// equal scores the smallest index wins) and ordered, atomic-free compaction (block prefix
// scans), so the output is a pure function of the scores.
//
// The exact work always happens on chip, on a candidate set held in shared memory (up to
// SEL_CAP entries, kept in index order): a radix select on (key - min), 12 bits per pass, finds
// the k-th key and the number of ties to take, an ordered scan emits the winners.  How the
// candidates get there:
//   * rows with T <= SEL_CAP: the whole row;
//   * longer rows, main path: a 4096-bin value histogram of 8192 strided samples gives a cut
//     that about 2k elements exceed; ONE streaming pass (16-byte loads, 16 elements per thread
//     and scan) then collects every element >= cut.  If the collected set turns out smaller than k or
//     larger than the buffer, the row is redone by
//   * the two-pass path: a 4096-bin histogram (bins linear in the key between the sampled
//     min and max, clamped outside, hence monotone) finds the bin holding the k-th element;
//     a second pass emits everything above that bin and keeps the bin itself as candidates;
//   * rows whose threshold bin overflows the buffer (e.g. all scores equal) fall back to
//     the textbook 4-pass radix select over global memory.
// NaN scores are not ordered; rows containing them get an unspecified (but in-range) list.
#include "common.cuh"

namespace sk {
namespace {

constexpr int SEL_THREADS = 1024;
constexpr int SEL_WARPS = SEL_THREADS / 32;
constexpr int SEL_BINS = 4096;
constexpr int SEL_EPT = 8;                        // consecutive elements per thread (two-pass path)
constexpr int SEL_CHUNK = SEL_THREADS * SEL_EPT;
constexpr int SEL_EPT1 = 16;                      // consecutive elements per thread (one-pass path)
constexpr int SEL_CHUNK1 = SEL_THREADS * SEL_EPT1;
constexpr int SEL_SAMPLES = 8192;

struct SelShared {
    uint32_t hist[SEL_BINS];
    uint32_t cand_key[SEL_CAP];
    int32_t cand_idx[SEL_CAP];
    int scan_buf[2][40];
    uint32_t red_lo[SEL_WARPS], red_hi[SEL_WARPS], red_x[SEL_WARPS];
    int thr_bin, thr_above, thr_inbin;
};

struct Scan {
    int parity = 0;
    // exclusive prefix of v over the block in thread order; total returned through `total`
    __device__ __forceinline__ int excl(int v, int& total, SelShared& s) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        int* buf = s.scan_buf[parity];
        parity ^= 1;
        int inc = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(FULL, inc, o);
            if (lane >= o) inc += n;
        }
        if (lane == 31) buf[warp] = inc;
        __syncthreads();
        if (warp == 0) {
            const int w = buf[lane];
            int winc = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int n = __shfl_up_sync(FULL, winc, o);
                if (lane >= o) winc += n;
            }
            buf[lane] = winc - w;
            if (lane == 31) buf[32] = winc;
        }
        __syncthreads();
        total = buf[32];
        return buf[warp] + inc - v;
    }
};

struct BinMap {
    uint32_t lo;
    int shift;
    __device__ __forceinline__ int operator()(uint32_t key) const {
        if (key < lo) return 0;
        const uint32_t b = ((key - lo) >> shift) + 1u;
        return b > (uint32_t)(SEL_BINS - 1) ? SEL_BINS - 1 : (int)b;
    }
};

__device__ __forceinline__ float key_to_float(uint32_t key) {
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

// Block-wide min / max of one uint32 per thread; every thread gets the result.
__device__ __forceinline__ void block_minmax(SelShared& s, uint32_t& lo, uint32_t& hi) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
        lo = min(lo, __shfl_xor_sync(FULL, lo, o));
        hi = max(hi, __shfl_xor_sync(FULL, hi, o));
    }
    if (lane == 0) {
        s.red_lo[warp] = lo;
        s.red_hi[warp] = hi;
    }
    __syncthreads();
    lo = s.red_lo[lane];
    hi = s.red_hi[lane];
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
        lo = min(lo, __shfl_xor_sync(FULL, lo, o));
        hi = max(hi, __shfl_xor_sync(FULL, hi, o));
    }
    __syncthreads();                                   // red_lo / red_hi may be reused
}

// Same with a second minimum riding along.
__device__ __forceinline__ void block_minmax3(SelShared& s, uint32_t& lo, uint32_t& hi, uint32_t& lo2) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
        lo = min(lo, __shfl_xor_sync(FULL, lo, o));
        hi = max(hi, __shfl_xor_sync(FULL, hi, o));
        lo2 = min(lo2, __shfl_xor_sync(FULL, lo2, o));
    }
    if (lane == 0) {
        s.red_lo[warp] = lo;
        s.red_hi[warp] = hi;
        s.red_x[warp] = lo2;
    }
    __syncthreads();
    lo = s.red_lo[lane];
    hi = s.red_hi[lane];
    lo2 = s.red_x[lane];
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
        lo = min(lo, __shfl_xor_sync(FULL, lo, o));
        hi = max(hi, __shfl_xor_sync(FULL, hi, o));
        lo2 = min(lo2, __shfl_xor_sync(FULL, lo2, o));
    }
    __syncthreads();
}

// Over hist[0..SEL_BINS): the bin b with  #(bins > b) < target <= #(bins >= b)  (target >= 1,
// total count >= target).  All threads take part (4 bins each, descending); result in shared
// memory, valid after the trailing barrier.
__device__ __forceinline__ void find_bin_desc(SelShared& s, Scan& scan, int target) {
    int c[4], local = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        c[j] = (int)s.hist[SEL_BINS - 1 - (4 * threadIdx.x + j)];
        local += c[j];
    }
    int total;
    int before = scan.excl(local, total, s);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if (before < target && before + c[j] >= target) {
            s.thr_bin = SEL_BINS - 1 - (4 * threadIdx.x + j);
            s.thr_above = before;
            s.thr_inbin = c[j];
        }
        before += c[j];
    }
    __syncthreads();
}

// k-th largest (k >= 1) of keys[0..n) in shared memory, n >= k.  Returns the key; `quota` =
// how many elements equal to it belong to the top k.  Radix select on (key - min) with up to
// 12 bits per pass, so score keys that span a few octaves need two passes.
__device__ __forceinline__ uint32_t smem_kth(SelShared& s, Scan& scan, const uint32_t* keys, int n,
                                             uint32_t k, uint32_t& quota) {
    uint32_t kmin = 0xffffffffu, kmax = 0u;
    for (int i = threadIdx.x; i < n; i += SEL_THREADS) {
        const uint32_t key = keys[i];
        kmin = min(kmin, key);
        kmax = max(kmax, key);
    }
    block_minmax(s, kmin, kmax);
    const uint32_t range = kmax - kmin;
    int hi = range == 0 ? 0 : 32 - __clz(range);       // bits [0, hi) of (key - kmin) may be set
    const int n_pass = (hi + 11) / 12;
    const int width = n_pass ? (hi + n_pass - 1) / n_pass : 0;
    uint32_t mask = hi >= 32 ? 0u : ~((1u << hi) - 1u);
    uint32_t prefix = 0;
    uint32_t remaining = k;
    while (hi > 0) {
        const int lo = max(hi - width, 0);
        const uint32_t dmask = (1u << (hi - lo)) - 1u;
        for (int i = threadIdx.x; i < SEL_BINS; i += SEL_THREADS) s.hist[i] = 0;
        __syncthreads();
        for (int base = 0; base < n; base += SEL_THREADS) {
            const int i = base + threadIdx.x;
            uint32_t kp = 0;
            bool active = false;
            if (i < n) {
                kp = keys[i] - kmin;
                active = (kp & mask) == prefix;
            }
            warp_hist_add(s.hist, (kp >> lo) & dmask, active);
        }
        __syncthreads();
        find_bin_desc(s, scan, (int)remaining);
        remaining -= (uint32_t)s.thr_above;
        prefix |= (uint32_t)s.thr_bin << lo;
        mask |= dmask << lo;
        hi = lo;
        __syncthreads();                               // thr_* are rewritten by the next pass
    }
    quota = remaining;
    return kmin + prefix;
}

// N consecutive scores starting at t0 (a multiple of 4); positions >= T read as 0 and are
// masked by the caller.  `vec`: the row base is 16-byte aligned.
template <int N>
__device__ __forceinline__ void load_scores(const float* __restrict__ sc, int t0, int T, bool vec,
                                            float (&f)[N]) {
    if (vec && t0 + N <= T) {
#pragma unroll
        for (int v = 0; v < N / 4; ++v) {
            const float4 a = __ldcg(reinterpret_cast<const float4*>(sc + t0) + v);
            f[4 * v] = a.x; f[4 * v + 1] = a.y; f[4 * v + 2] = a.z; f[4 * v + 3] = a.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < N; ++j) f[j] = (t0 + j < T) ? __ldcg(sc + t0 + j) : 0.f;
    }
}

// Exact top-`need` of the n_cand candidates in shared memory (index order) -> heavy[out_pos..),
// ties at the cut resolved towards the front (= the smallest indices).  Returns the k-th key.
__device__ __forceinline__ uint32_t emit_from_candidates(SelShared& s, Scan& scan, int n_cand, int need,
                                                         int out_pos, int Me, int32_t* __restrict__ heavy) {
    const int tid = threadIdx.x;
    uint32_t quota;
    const uint32_t kth = smem_kth(s, scan, s.cand_key, n_cand, (uint32_t)need, quota);
    int gt_base = 0, eq_base = 0;
    for (int base = 0; base < n_cand; base += SEL_THREADS) {
        const int i = base + tid;
        uint32_t k = 0;
        int idx = 0;
        const bool live = i < n_cand;
        if (live) {
            k = s.cand_key[i];
            idx = s.cand_idx[i];
        }
        const int gt = live && k > kth, eq = live && k == kth;
        int total;
        const int off = scan.excl(gt | (eq << 16), total, s);
        const int gt_before = gt_base + (off & 0xffff);
        const int eq_before = eq_base + (off >> 16);
        const int dst = out_pos + gt_before + min(eq_before, (int)quota);
        if ((gt || (eq && eq_before < (int)quota)) && dst < Me) heavy[dst] = idx;
        gt_base += total & 0xffff;
        eq_base += total >> 16;
    }
    return kth;
}

// Same job as emit_from_candidates with fewer block-wide phases, for the common case of a few
// thousand candidates: one 4096-bin histogram of (key - kmin) finds the bin holding the need-th
// largest key; everything in higher bins is emitted by one ordered scan (consecutive candidates
// per thread), and the handful of candidates inside that bin are ranked against each other
// directly.  hist must be zero on entry.  Returns false (nothing written) if the threshold bin
// holds more than 1024 candidates; the caller then uses the radix path.
__device__ __forceinline__ bool emit_candidates_binned(SelShared& s, Scan& scan, int n, int need, int Me,
                                                       uint32_t kmin, uint32_t kmax,
                                                       int32_t* __restrict__ heavy, uint32_t& kth_out) {
    const int tid = threadIdx.x;
    const uint32_t range = kmax - kmin;
    const int bits = range == 0 ? 0 : 32 - __clz(range);
    const int shift = max(0, bits - 12);
    for (int base = 0; base < n; base += SEL_THREADS) {
        const int i = base + tid;
        const uint32_t k = i < n ? s.cand_key[i] : kmin;
        warp_hist_add(s.hist, (k - kmin) >> shift, i < n);
    }
    __syncthreads();
    find_bin_desc(s, scan, need);
    const int thr = s.thr_bin, above = s.thr_above, inbin = s.thr_inbin;
    if (inbin > 1024) return false;
    __syncthreads();                                   // hist is reused for the tie list below
    uint32_t* tie_key = s.hist;                        // [1024]
    int32_t* tie_idx = reinterpret_cast<int32_t*>(s.hist + 1024);
    const int ept = (n + SEL_THREADS - 1) / SEL_THREADS;
    const int i0 = tid * ept, i1 = min(n, i0 + ept);
    int n_gt = 0, n_eq = 0;
    for (int i = i0; i < i1; ++i) {
        const int b = (int)((s.cand_key[i] - kmin) >> shift);
        n_gt += b > thr;
        n_eq += b == thr;
    }
    int total;
    const int off = scan.excl(n_gt | (n_eq << 16), total, s);
    int g = off & 0xffff, e = off >> 16;
    for (int i = i0; i < i1; ++i) {
        const uint32_t k = s.cand_key[i];
        const int b = (int)((k - kmin) >> shift);
        if (b > thr) {
            if (g < Me) heavy[g] = s.cand_idx[i];
            ++g;
        } else if (b == thr) {
            if (e < 1024) {
                tie_key[e] = k;
                tie_idx[e] = s.cand_idx[i];
            }
            ++e;
        }
    }
    __syncthreads();
    const int want = need - above;                     // 1 <= want <= inbin
    if (tid < inbin) {
        const uint32_t k = tie_key[tid];
        int rank = 0;
        for (int j = 0; j < inbin; ++j) {
            const uint32_t kj = tie_key[j];
            rank += (kj > k) || (kj == k && j < tid);
        }
        if (rank < want && above + rank < Me) heavy[above + rank] = tie_idx[tid];
        if (rank == want - 1) s.red_lo[0] = k;
    }
    __syncthreads();
    kth_out = s.red_lo[0];
    return true;
}

// Top-`Me` (0 < Me) of one row of T scores -> heavy[0..Me).  Exact; see the file header.
__device__ __forceinline__ void select_row(SelShared& s, Scan& scan, const float* __restrict__ sc, int T,
                                           int Me, int32_t* __restrict__ heavy) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool vec = (reinterpret_cast<uintptr_t>(sc) & 15u) == 0;
    if (Me == T) {
        for (int i = tid; i < T; i += SEL_THREADS) heavy[i] = i;
    } else if (Me > 0) {
        int n_cand = 0;        // candidates in shared memory (index order)
        int need = Me;         // how many of them to take
        int out_pos = 0;       // heavy entries already emitted
        bool have_cand = false, global_fallback = false;

        if (T <= SEL_CAP) {
            for (int i = tid; i < T; i += SEL_THREADS) {
                s.cand_key[i] = order_key(sc[i]);
                s.cand_idx[i] = i;
            }
            n_cand = T;
            have_cand = true;
            __syncthreads();
        } else {
            // ---- main path: cut from a sample, then one streaming pass
            const int stride = T / SEL_SAMPLES;                     // >= 2
            const int64_t rs64 = (2 * (int64_t)Me * SEL_SAMPLES + T - 1) / T + 32;
            if (rs64 <= SEL_SAMPLES / 4 && rs64 * stride <= SEL_CAP / 2) {
                // 8 strided samples per thread -> value histogram -> cut with ~r_s samples above
                float fs[8];
                uint32_t flo = 0xffffffffu, fhi = 0u;               // order keys of the finite samples
                // one 32-byte run of 8 consecutive scores per thread, runs spread evenly over the
                // row: 8192 samples for 1024 memory requests
                load_scores<8>(sc, (int)(((int64_t)tid * (T - 8) / SEL_THREADS) & ~3), T, vec, fs);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (fs[j] > -INFINITY && fs[j] < INFINITY) {
                        const uint32_t key = order_key(fs[j]);
                        flo = min(flo, key);
                        fhi = max(fhi, key);
                    }
                }
                for (int i = tid; i < SEL_BINS; i += SEL_THREADS) s.hist[i] = 0;
                block_minmax(s, flo, fhi);
                const float fmin = key_to_float(flo), fmax = key_to_float(fhi);
                float cut = INFINITY;
                if (flo < fhi) {
                    const float scale = (float)(SEL_BINS - 2) / (fmax - fmin);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const uint32_t b = min(__float2uint_rz((fs[j] - fmin) * scale), (uint32_t)(SEL_BINS - 1));
                        warp_hist_add(s.hist, b, true);
                    }
                    __syncthreads();
                    find_bin_desc(s, scan, (int)rs64);
                    if (s.thr_bin >= 1) cut = fmin + (float)s.thr_bin / scale;
                    __syncthreads();
                }
                int base_cnt = 0;
                float cur[SEL_EPT1], nxt[SEL_EPT1];
                load_scores<SEL_EPT1>(sc, tid * SEL_EPT1, T, vec, cur);
                for (int base = 0; base < T && cut < INFINITY; base += SEL_CHUNK1) {
                    const int t0 = base + tid * SEL_EPT1;
                    if (base + SEL_CHUNK1 < T) load_scores<SEL_EPT1>(sc, t0 + SEL_CHUNK1, T, vec, nxt);
                    unsigned hit = 0;
#pragma unroll
                    for (int j = 0; j < SEL_EPT1; ++j)
                        if (cur[j] >= cut && t0 + j < T) hit |= 1u << j;
                    int total;
                    int pos = base_cnt + scan.excl(__popc(hit), total, s);
#pragma unroll
                    for (int j = 0; j < SEL_EPT1; ++j) {
                        if (hit & (1u << j)) {
                            if (pos < SEL_CAP) {
                                s.cand_key[pos] = order_key(cur[j]);
                                s.cand_idx[pos] = t0 + j;
                            }
                            ++pos;
                        }
                    }
                    base_cnt += total;
#pragma unroll
                    for (int j = 0; j < SEL_EPT1; ++j) cur[j] = nxt[j];
                }
                __syncthreads();
                if (base_cnt >= Me && base_cnt <= SEL_CAP) {
                    n_cand = base_cnt;
                    have_cand = true;
                }
            }
            if (!have_cand) {
                // ---- two-pass path: sampled range, histogram, threshold bin
                uint32_t kmin = 0xffffffffu, kmax = 0u;
                const int sstride = T / (SEL_THREADS * 4);
                for (int j = 0; j < 4; ++j) {
                    const float f = sc[(size_t)(tid * 4 + j) * sstride];
                    if (f > -INFINITY && f < INFINITY) {
                        const uint32_t k = order_key(f);
                        kmin = min(kmin, k);
                        kmax = max(kmax, k);
                    }
                }
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) {
                    kmin = min(kmin, __shfl_xor_sync(FULL, kmin, o));
                    kmax = max(kmax, __shfl_xor_sync(FULL, kmax, o));
                }
                if (lane == 0) {
                    s.red_lo[warp] = kmin;
                    s.red_hi[warp] = kmax;
                }
                for (int i = tid; i < SEL_BINS; i += SEL_THREADS) s.hist[i] = 0;
                __syncthreads();
                kmin = s.red_lo[lane];
                kmax = s.red_hi[lane];
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) {
                    kmin = min(kmin, __shfl_xor_sync(FULL, kmin, o));
                    kmax = max(kmax, __shfl_xor_sync(FULL, kmax, o));
                }
                BinMap bin;
                if (kmin > kmax) {  // no finite sample
                    bin.lo = 0;
                    bin.shift = 20;
                } else {
                    const uint32_t range = kmax - kmin;
                    const int bits = 32 - __clz(range | 1u);
                    bin.lo = kmin;
                    bin.shift = max(0, bits - 11);
                }
                // pass 1: histogram; two independent groups per thread keep 4 x 16 B in flight
                for (int base = 0; base < T; base += 2 * SEL_CHUNK) {
                    float fa[SEL_EPT], fb[SEL_EPT];
                    const int ta = base + tid * SEL_EPT, tb = ta + SEL_CHUNK;
                    load_scores<SEL_EPT>(sc, ta, T, vec, fa);
                    load_scores<SEL_EPT>(sc, tb, T, vec, fb);
#pragma unroll
                    for (int j = 0; j < SEL_EPT; ++j)
                        warp_hist_add(s.hist, (uint32_t)bin(order_key(fa[j])), ta + j < T);
#pragma unroll
                    for (int j = 0; j < SEL_EPT; ++j)
                        warp_hist_add(s.hist, (uint32_t)bin(order_key(fb[j])), tb + j < T);
                }
                __syncthreads();
                find_bin_desc(s, scan, Me);
                const int thr = s.thr_bin;
                const int above = s.thr_above;
                const int inbin = s.thr_inbin;
                if (inbin > SEL_CAP) {
                    global_fallback = true;
                } else {
                    // pass 2: emit the sure ones, keep the threshold bin on chip (index order)
                    int sure_base = 0, cand_base = 0;
                    float cur[SEL_EPT], nxt[SEL_EPT];
                    load_scores<SEL_EPT>(sc, tid * SEL_EPT, T, vec, cur);
                    for (int base = 0; base < T; base += SEL_CHUNK) {
                        const int t0 = base + tid * SEL_EPT;
                        if (base + SEL_CHUNK < T) load_scores<SEL_EPT>(sc, t0 + SEL_CHUNK, T, vec, nxt);
                        uint32_t k[SEL_EPT];
                        int cls[SEL_EPT];  // 2 = sure, 1 = candidate
                        int n_sure = 0, n_cnd = 0;
#pragma unroll
                        for (int j = 0; j < SEL_EPT; ++j) {
                            cls[j] = 0;
                            k[j] = order_key(cur[j]);
                            if (t0 + j < T) {
                                const int b = bin(k[j]);
                                cls[j] = b > thr ? 2 : (b == thr ? 1 : 0);
                                n_sure += cls[j] == 2;
                                n_cnd += cls[j] == 1;
                            }
                        }
                        int total;
                        const int off = scan.excl(n_sure | (n_cnd << 16), total, s);
                        int so = sure_base + (off & 0xffff), co = cand_base + (off >> 16);
#pragma unroll
                        for (int j = 0; j < SEL_EPT; ++j) {
                            // bounds hold by construction; the guards keep a row whose scores
                            // change under the kernel from writing outside its buffers
                            if (cls[j] == 2) {
                                if (so < Me) heavy[so] = t0 + j;
                                ++so;
                            } else if (cls[j] == 1) {
                                if (co < SEL_CAP) {
                                    s.cand_key[co] = k[j];
                                    s.cand_idx[co] = t0 + j;
                                }
                                ++co;
                            }
                        }
                        sure_base += total & 0xffff;
                        cand_base += total >> 16;
#pragma unroll
                        for (int j = 0; j < SEL_EPT; ++j) cur[j] = nxt[j];
                    }
                    out_pos = above;
                    need = Me - above;
                    n_cand = inbin;
                    have_cand = true;
                    __syncthreads();
                }
            }
        }

        if (have_cand) {
            emit_from_candidates(s, scan, n_cand, need, out_pos, Me, heavy);
        } else if (global_fallback) {
            // ---- fallback: radix select over the whole row in global memory
            uint32_t prefix = 0, mask = 0, remaining = (uint32_t)Me;
            for (int shift = 24; shift >= 0; shift -= 8) {
                for (int i = tid; i < SEL_BINS; i += SEL_THREADS) s.hist[i] = 0;
                __syncthreads();
                for (int base = 0; base < T; base += SEL_THREADS) {
                    const int t = base + tid;
                    const uint32_t k = t < T ? order_key(sc[t]) : 0u;
                    warp_hist_add_match(s.hist, (k >> shift) & 0xffu, t < T && (k & mask) == prefix);
                }
                __syncthreads();
                find_bin_desc(s, scan, (int)remaining);
                remaining -= (uint32_t)s.thr_above;
                prefix |= (uint32_t)s.thr_bin << shift;
                mask |= 0xffu << shift;
                __syncthreads();
            }
            int gt_base = 0, eq_base = 0;
            for (int base = 0; base < T; base += SEL_CHUNK) {
                const int t0 = base + tid * SEL_EPT;
                int gt[SEL_EPT], eq[SEL_EPT], n_gt = 0, n_eq = 0;
#pragma unroll
                for (int j = 0; j < SEL_EPT; ++j) {
                    gt[j] = eq[j] = 0;
                    if (t0 + j < T) {
                        const uint32_t k = order_key(sc[t0 + j]);
                        gt[j] = k > prefix;
                        eq[j] = k == prefix;
                        n_gt += gt[j];
                        n_eq += eq[j];
                    }
                }
                int total;
                const int off = scan.excl(n_gt | (n_eq << 16), total, s);
                int gt_before = gt_base + (off & 0xffff);
                int eq_before = eq_base + (off >> 16);
#pragma unroll
                for (int j = 0; j < SEL_EPT; ++j) {
                    const int dst = gt_before + min(eq_before, (int)remaining);
                    if ((gt[j] || (eq[j] && eq_before < (int)remaining)) && dst < Me) heavy[dst] = t0 + j;
                    gt_before += gt[j];
                    eq_before += eq[j];
                }
                gt_base += total & 0xffff;
                eq_base += total >> 16;
            }
        }
    }
}

// Structured part of the list ([0..sink) ++ [max(T-window,sink)..T), or [T-1]); returns its length.
__device__ __forceinline__ int write_base(int32_t* __restrict__ out, int T, int sink_in, int window_in) {
    const int tid = threadIdx.x;
    const int sink = max(0, min(sink_in, T));
    const int window = max(0, min(window_in, T));
    const int win_start = max(T - window, sink);
    const int n_win = window > 0 ? T - win_start : 0;
    int nb = sink + n_win;
    for (int i = tid; i < sink; i += SEL_THREADS) out[i] = i;
    for (int i = tid; i < n_win; i += SEL_THREADS) out[sink + i] = win_start + i;
    if (nb == 0) {
        if (tid == 0) out[0] = T - 1;
        nb = 1;
    }
    return nb;
}

// Optional descending-score order of the top-k part, then the -1 masking of the whole list.
__device__ __forceinline__ void finish_row(SelShared& s, const float* __restrict__ sc,
                                           const uint8_t* __restrict__ al, int32_t* __restrict__ out,
                                           int nb, int Me, int sorted) {
    const int tid = threadIdx.x;
    int32_t* heavy = out + nb;
    // ---- optional: order the top-k part by descending score (ties: ascending index)
    if (sorted && Me > 1) {
        uint64_t* keys = reinterpret_cast<uint64_t*>(s.cand_key);  // spans cand_key + cand_idx
        int n2 = 1;
        while (n2 < Me) n2 <<= 1;
        for (int i = tid; i < n2; i += SEL_THREADS) {
            uint64_t v = 0;
            if (i < Me) {
                const int idx = heavy[i];
                v = ((uint64_t)order_key(sc[idx]) << 32) | (uint32_t)(0xffffffffu - (uint32_t)idx);
            }
            keys[i] = v;
        }
        __syncthreads();
        for (int k = 2; k <= n2; k <<= 1) {
            for (int j = k >> 1; j > 0; j >>= 1) {
                for (int i = tid; i < n2; i += SEL_THREADS) {
                    const int p = i ^ j;
                    if (p > i) {
                        const uint64_t a = keys[i], b = keys[p];
                        const bool desc = (i & k) == 0;
                        if (desc ? a < b : a > b) {
                            keys[i] = b;
                            keys[p] = a;
                        }
                    }
                }
                __syncthreads();
            }
        }
        for (int i = tid; i < Me; i += SEL_THREADS)
            heavy[i] = (int32_t)(0xffffffffu - (uint32_t)(keys[i] & 0xffffffffu));
        __syncthreads();
    }

    // ---- entries whose position is masked become -1
    if (al != nullptr) {
        for (int i = tid; i < nb + Me; i += SEL_THREADS) {
            const int idx = out[i];
            if (idx >= 0 && al[idx] == 0) out[i] = -1;
        }
    }
}

__global__ void __launch_bounds__(SEL_THREADS, 1)
select_list_kernel(const float* __restrict__ scores, int64_t score_row_stride,
                   const uint8_t* __restrict__ allowed, int64_t T_host,
                   const int32_t* __restrict__ T_dev, int64_t M, int sink_in, int window_in,
                   int sorted, int32_t* __restrict__ list, int64_t list_row_stride,
                   int32_t* __restrict__ list_len) {
    extern __shared__ __align__(16) char smem_raw[];
    SelShared& s = *reinterpret_cast<SelShared*>(smem_raw);
    const int tid = threadIdx.x;
    const int64_t row = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const float* sc = scores + row * score_row_stride;
    const uint8_t* al = allowed ? allowed + row * T_host : nullptr;
    int32_t* out = list + row * list_row_stride;
    const int T = effective_len(T_host, T_dev);
    Scan scan;
    if (T <= 0) {
        if (tid == 0) list_len[row] = 0;
        return;
    }
    const int nb = write_base(out, T, sink_in, window_in);
    const int Me = (int)(M < (int64_t)T ? M : (int64_t)T);
    if (tid == 0) list_len[row] = nb + Me;
    if (Me > 0) select_row(s, scan, sc, T, Me, out + nb);
    __syncthreads();
    finish_row(s, sc, al, out, nb, Me, sorted);
}


// ------------------------------------------------------------------------------------------
// Candidate mode: the filtering scorer left, per row, runs of (score, index) pairs in
// ascending index order plus the cut each chunk used.  Gather them on chip, select exactly,
// and accept the result only if the k-th key is >= every chunk's cut (then every element of
// the true top-k was kept by its chunk).  Otherwise rescore the row here and select from the
// full row.
// ------------------------------------------------------------------------------------------
struct CandArgs {
    const int32_t* cnt;     // [rows][chunks_max][SC_WARPS]
    const float* cut;       // [rows][chunks_max]
    const uint2* cand;      // [rows][chunks_max][SC_WARPS][cap_w]
    float* scratch;         // [rows][score_stride]
    int32_t* n_fallback;    // statistics: rows that had to be rescored
    int64_t score_stride;
    int chunks_max, cap_w;
    int64_t Tslots, per_cta;
    // for the rescoring path
    const float* lut;
    const uint8_t* codes;
    const __half* v_norm;
    int H, Hkv, L, R, ht;
    int64_t Tcap;
    const float* qpar;      // packed candidates: K0 of every KV-head group
    const float* probs;     // packed candidates: q_probs [rows][32][256] fp32 (rows 32 KiB apart)
    const uint2* tail;      // [rows][SC_TAIL]: the row's newest keys, unfiltered (see FilterArgs::tail)
};

// ------------------------------------------------------------------------------------------
// Packed candidates (written by score_packed_kernel): every entry carries the exact integer sum S
// of the key's 12-bit table entries and ||v||.  With K0 = L * lo * C of the group's table,
//     X = C * sum_l p_l(code_l) - ... lies in [S - 0.1, S + 32.1)            (table construction)
// and the fp32 score the exact scorer computes, e = fl(sum_l p_l) * ||v||, satisfies
//     (S + K0 - 1) * ||v|| * (1 - 2^-21)  <=  C * e  <=  (S + K0 + 33) * ||v|| * (1 + 2^-21)
// (fp32 summation and the two roundings of the bound itself are far inside the slack of 0.9).
// Call the two sides lo_i and up_i.  The candidates are all keys with up_i >= their chunk's cut.
// ------------------------------------------------------------------------------------------
constexpr int BAND_MAX = 1024;                    // keys between the brackets that can be rescored on chip
constexpr int BAND_DIRECT = 256;                  // up to here the band is ranked pair by pair

__device__ __forceinline__ float packed_upper_sel(uint32_t S, float K0p, float vn) {
    return __fmul_rn(__fadd_rn(__uint2float_rn(S), K0p), vn);     // same operations as the scorer
}
__device__ __forceinline__ float packed_lower_sel(uint32_t S, float K0m, float vn) {
    const float v = __fmul_rn(__fadd_rn(__uint2float_rn(S), K0m), vn) * (1.0f - 4.8e-7f);
    return fmaxf(v, 0.f);
}

// Exact fp32 scores of the keys band_t[0..n) of one row (L = 32), the tables added in the very order
// score_kernel adds them for a key (groups of 8 tables ascending, inside a group table u ^ (t & 7)
// at step u), so that the values equal sk_score's bit for bit.  The row's probabilities
// tab_s[l * 256 + bucket] are in shared memory.  A warp takes 8 keys at a time: lane l fetches
// code byte l of each (one 32-byte sector per key) and looks its term up, the terms go through a
// padded tile, four keys at a time, and lanes 0..3 add one key's 32 terms each, in order.
constexpr int XS_KEYS = 8;                        // keys per warp and batch
constexpr int XS_TILE = 4 * 33;                   // floats per warp
constexpr int XS_TAB = 32 * 256;                  // floats of one row's table
static_assert((2 * BAND_MAX + XS_TAB + SEL_WARPS * XS_TILE) * 4 <= SEL_CAP * 4, "band arrays, table and tiles share cand_key");
__device__ __forceinline__ void exact_scores_like_scorer(const float* tab_s, const uint8_t* __restrict__ cg,
                                                         const __half* __restrict__ vg, const int32_t* band_t,
                                                         int n, float* tile_all, uint32_t* band_e) {
    constexpr int L = 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* tile = tile_all + warp * XS_TILE;
    for (int k0 = warp * XS_KEYS; k0 < n; k0 += SEL_WARPS * XS_KEYS) {
        int t[XS_KEYS];
        uint32_t code[XS_KEYS];
#pragma unroll
        for (int kk = 0; kk < XS_KEYS; ++kk) {
            t[kk] = k0 + kk < n ? band_t[k0 + kk] : -1;
            code[kk] = t[kk] >= 0 ? (uint32_t)__ldcg(cg + (size_t)t[kk] * L + lane) : 0u;
        }
        const int mine = k0 + lane;
        const int tm = (lane < XS_KEYS && mine < n) ? band_t[mine] : -1;
        float vn = 0.f;
        if (tm >= 0) vn = __half2float(__ldcg(vg + tm));
#pragma unroll
        for (int half = 0; half < 2; ++half) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) tile[kk * 33 + lane] = tab_s[lane * 256 + code[half * 4 + kk]];
            __syncwarp();
            const int who = lane - 4 * half;               // lanes 0..3 sum the first four keys, 4..7 the others
            if (who >= 0 && who < 4 && tm >= 0) {
                const int m = tm & 7;
                float sum = 0.f;
#pragma unroll
                for (int q = 0; q < 32; ++q) sum += tile[who * 33 + ((q & 24) | ((q & 7) ^ m))];
                band_e[mine] = order_key(sum * vn);
            }
            __syncwarp();
        }
    }
}

// Exact top-Me of a row from its packed candidates (the packed words in cand_key, in index order;
// kmin / kmax = smallest / largest order key of their up_i; hist zero on entry; s_min = smallest S
// of the row's candidates).  Returns false, with nothing usable written, when the result cannot be proved or
// held on chip; the caller then rescans the row.
//
// One histogram of the up_i finds the bin that holds the Me-th largest; its upper edge UB bounds
// C * (k-th exact score) from above.  Every candidate has lo_i >= up_i * (1 - 34 / (s_min + K0 + 33)),
// so LB = (lower edge of that bin) * that factor is below lo_i of the >= Me candidates in the bin
// or above it, hence below C * (k-th exact score).  A key outside the candidate set has
// up < its chunk's cut <= chi, so with chi <= LB it lies strictly below the k-th exact score.
// Candidates with lo_i > UB are in the top Me and are written at once (ascending index); those
// with up_i < LB are out; the few in between are scored exactly (fp32 table, sk_score's summation
// order), ranked by (score descending, index ascending) and the best fill the remaining places.
__device__ __forceinline__ bool emit_packed_candidates(SelShared& s, Scan& scan, int n, int Me, uint32_t kmin,
                                                       uint32_t kmax, uint32_t s_min, uint32_t chi_key, float K0,
                                                       const float* __restrict__ probs_row,
                                                       const uint8_t* __restrict__ cg,
                                                       const __half* __restrict__ vg,
                                                       int32_t* __restrict__ heavy, int32_t* stats) {
    const int tid = threadIdx.x;
    const uint32_t range = kmax - kmin;
    const int bits = range == 0 ? 0 : 32 - __clz(range);
    const int shift = max(0, bits - 12);
    auto vn_of = [](uint32_t x) { return __half2float(__ushort_as_half((unsigned short)(x & 0x7fffu))); };
    for (int base = 0; base < n; base += SEL_THREADS) {
        const int i = base + tid;
        uint32_t k = kmin;
        if (i < n) {
            const uint32_t x = s.cand_key[i];
            k = order_key(packed_upper_sel(x >> 15, K0 + 33.0f, vn_of(x)));
        }
        warp_hist_add(s.hist, (k - kmin) >> shift, i < n);
    }
    // the row's probabilities [L][R] (32 KiB), requested now, stored to shared memory once the
    // classification below has freed cand_key
    float4 tab_r[XS_TAB / 4 / SEL_THREADS];
#pragma unroll
    for (int u = 0; u < XS_TAB / 4 / SEL_THREADS; ++u)
        tab_r[u] = __ldcg(reinterpret_cast<const float4*>(probs_row) + u * SEL_THREADS + tid);
    __syncthreads();
    find_bin_desc(s, scan, Me);
    const uint32_t thr = (uint32_t)s.thr_bin;
    uint64_t ub64 = (uint64_t)kmin + (((uint64_t)thr + 1u) << shift) - 1u;
    if (ub64 > (uint64_t)kmax) ub64 = kmax;
    const float UB = order_key_inverse((uint32_t)ub64);
    const float edge = order_key_inverse(kmin + (thr << shift));
    const float gap = 34.0f / (__uint2float_rz(s_min) + K0 + 33.0f);
    const float LB = fmaxf(edge * (1.0f - gap * 1.0001f) * (1.0f - 1e-5f), 0.f);
    if (!(gap < 0.5f) || order_key(LB) < chi_key) {               // some chunk may have dropped a key of the top Me
        if (tid == 0) atomicAdd(stats + 6, 1);                    // statistics: the bracket reaches below the largest cut
        return false;
    }

    // ---- classes: 1 = in, 2 = between the brackets, 0 = out; two bits per candidate of this thread
    const int ept = (n + SEL_THREADS - 1) / SEL_THREADS;          // <= 16
    const int i0 = tid * ept, i1 = min(n, i0 + ept);
    uint32_t cls_bits = 0;
    int n_sure = 0, n_band = 0;
    for (int i = i0; i < i1; ++i) {
        const uint32_t x = s.cand_key[i];
        const float up = packed_upper_sel(x >> 15, K0 + 33.0f, vn_of(x));
        const float lo = packed_lower_sel(x >> 15, K0 - 1.0f, vn_of(x));
        const uint32_t cls = lo > UB ? 1u : (up >= LB ? 2u : 0u);
        cls_bits |= cls << (2 * (i - i0));
        n_sure += cls == 1u;
        n_band += cls == 2u;
    }
    int total;
    const int off = scan.excl(n_sure | (n_band << 16), total, s);
    const int tot_sure = total & 0xffff, tot_band = total >> 16;
    const int want = Me - tot_sure;
    if (tid == 0) {                                   // statistics: keys rescored, rows ranked by the radix path
        atomicAdd(stats + 1, tot_band);
        if (tot_band > BAND_DIRECT) atomicAdd(stats + 2, 1);
    }
    if (tot_band > BAND_MAX || want < 0 || want > tot_band) {
        if (tid == 0) atomicAdd(stats + (tot_band > BAND_MAX ? 7 : 8), 1);   // bracket too large for the chip / inconsistent counts
        return false;
    }
    // every read of cand_key happened before the scan's barriers: its space now holds the band
    uint32_t* band_e = s.cand_key;                                     // [BAND_MAX] exact order keys
    int32_t* band_t = reinterpret_cast<int32_t*>(s.cand_key + BAND_MAX);   // [BAND_MAX] key index
    float* tab_s = reinterpret_cast<float*>(s.cand_key + 2 * BAND_MAX);    // [L][256] this row's probabilities
#pragma unroll
    for (int u = 0; u < XS_TAB / 4 / SEL_THREADS; ++u)
        reinterpret_cast<float4*>(tab_s)[u * SEL_THREADS + tid] = tab_r[u];
    {
        int spos = off & 0xffff, bpos = off >> 16;
        for (int i = i0; i < i1; ++i) {
            const uint32_t cls = (cls_bits >> (2 * (i - i0))) & 3u;
            if (cls == 1u) {
                if (spos < Me) heavy[spos] = s.cand_idx[i];
                ++spos;
            } else if (cls == 2u) {
                band_t[bpos++] = s.cand_idx[i];
            }
        }
    }
    if (want == 0) return true;                        // uniform
    __syncthreads();
    exact_scores_like_scorer(tab_s, cg, vg, band_t, tot_band, tab_s + XS_TAB, band_e);
    __syncthreads();

    int32_t* out = heavy + tot_sure;                   // `want` places left
    if (tot_band <= BAND_DIRECT) {
        // four threads per key count the keys that precede it (band order = index order)
        const int kb = tid >> 2, part = tid & 3;
        int cnt = 0;
        if (kb < tot_band) {
            // keys before kb in the band (lower index) precede it when they are >=, keys after it when >
            const uint32_t mine = band_e[kb];
            int jj = part;
#pragma unroll 4
            for (; jj < kb; jj += 4) cnt += band_e[jj] >= mine;
            if (jj == kb) jj += 4;                                // kb itself (only the thread with part == kb % 4 meets it)
#pragma unroll 4
            for (; jj < tot_band; jj += 4) cnt += band_e[jj] > mine;
        }
        cnt += __shfl_xor_sync(FULL, cnt, 1);
        cnt += __shfl_xor_sync(FULL, cnt, 2);
        if (kb < tot_band && part == 0 && cnt < want) out[cnt] = band_t[kb];
    } else {
        uint32_t quota;
        const uint32_t kth = smem_kth(s, scan, band_e, tot_band, (uint32_t)want, quota);
        const int ept2 = (tot_band + SEL_THREADS - 1) / SEL_THREADS;
        const int j0 = tid * ept2, j1 = min(tot_band, j0 + ept2);
        int n_gt = 0, n_eq = 0;
        for (int jb = j0; jb < j1; ++jb) {
            n_gt += band_e[jb] > kth;
            n_eq += band_e[jb] == kth;
        }
        int tot2;
        const int off2 = scan.excl(n_gt | (n_eq << 16), tot2, s);
        int gt_before = off2 & 0xffff, eq_before = off2 >> 16;
        for (int jb = j0; jb < j1; ++jb) {
            const uint32_t e = band_e[jb];
            const int dst = gt_before + min(eq_before, (int)quota);
            if ((e > kth || (e == kth && eq_before < (int)quota)) && dst < want) out[dst] = band_t[jb];
            gt_before += e > kth;
            eq_before += e == kth;
        }
    }
    return true;
}

static_assert(SC_TAIL <= SEL_THREADS, "one tail entry per thread in the gather");

// PACKED: the candidates are packed (S, ||v||) words (score_packed_kernel), else fp32 scores.
template <bool PACKED>
__global__ void __launch_bounds__(SEL_THREADS, 1)
select_cand_kernel(CandArgs a, int64_t T_host, const int32_t* __restrict__ T_dev, int64_t M,
                   int sink_in, int window_in, int sorted, int32_t* __restrict__ list,
                   int64_t list_row_stride, int32_t* __restrict__ list_len) {
    extern __shared__ __align__(16) char smem_raw[];
    SelShared& s = *reinterpret_cast<SelShared*>(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t row = blockIdx.x;
    int32_t* out = list + row * list_row_stride;

    // which scorer chunks belong to this row's KV-head group
    const int rep = a.H / a.Hkv, tiles = rep / a.ht;
    const int b = (int)(row / a.H), h = (int)(row - (int64_t)b * a.H);
    const int kvh = h / rep, hj = h - kvh * rep;
    const int g = (b * a.Hkv + kvh) * tiles + hj / a.ht;
    const int64_t first_cta = ((int64_t)g * a.Tslots) / a.per_cta;
    const int64_t last_cta = ((int64_t)(g + 1) * a.Tslots - 1) / a.per_cta;
    const int n_runs = (int)(last_cta - first_cta + 1) * SC_WARPS;      // <= 1024
    const int32_t* cnt = a.cnt + row * a.chunks_max * SC_WARPS;
    constexpr bool packed = PACKED;
    pdl_launch_dependents();
    pdl_wait();                               // the runs, their lengths and the cuts come from the scorer
    const float K0 = packed ? __ldcg(a.qpar + g) : 0.f;
    // one candidate into shared memory: its order key (of the score, or of the packed entry's upper bound)
    uint32_t s_min = 0xffffffffu;                 // packed candidates: smallest integer sum S
    auto put = [&](int i, uint2 e, uint32_t& kmin, uint32_t& kmax) {
        uint32_t k;
        if (packed) {
            s_min = min(s_min, e.x >> 15);
            const float vn = __half2float(__ushort_as_half((unsigned short)(e.x & 0x7fffu)));
            k = order_key(packed_upper_sel(e.x >> 15, K0 + 33.0f, vn));
        } else {
            k = order_key(__uint_as_float(e.x));
        }
        s.cand_key[i] = packed ? e.x : k;
        s.cand_idx[i] = (int32_t)e.y;
        kmin = min(kmin, k);
        kmax = max(kmax, k);
    };
    // run length and chunk cut of this thread: issued before anything waits on the live length
    const int c_run = tid < n_runs ? __ldcg(cnt + tid) : 0;
    const float cut_chunk = tid < n_runs / SC_WARPS ? __ldcg(a.cut + row * a.chunks_max + tid) : -INFINITY;

    const int T = effective_len(T_host, T_dev);
    Scan scan;
    if (T <= 0) {
        if (tid == 0) list_len[row] = 0;
        return;
    }
    const int nb = write_base(out, T, sink_in, window_in);
    const int Me = (int)(M < (int64_t)T ? M : (int64_t)T);
    if (tid == 0) list_len[row] = nb + Me;
    int32_t* heavy = out + nb;
    float* sc = a.scratch + row * a.score_stride;

    bool exact = false;
    if (Me > 0 && Me < T) {
        // ---- run lengths -> offsets (one run per thread), largest cut, overflow flag
        if (tid == 0) {
            s.thr_bin = 0;                             // "some run overflowed"
            s.red_hi[0] = 0u;                          // key of the largest cut
        }
        for (int i = tid; i < SEL_BINS; i += SEL_THREADS) s.hist[i] = 0;
        __syncthreads();
        const int c = c_run;
        if (c > a.cap_w) s.thr_bin = 1;
        if (tid < n_runs / SC_WARPS) atomicMax(&s.red_hi[0], order_key(cut_chunk));
        int total;
        const int off = scan.excl(c, total, s);        // two barriers: the flags above are visible after it
        const bool any_over = s.thr_bin != 0;
        const uint32_t chi = s.red_hi[0];
        // the row's newest keys follow the runs: all of them, in index order (they have the largest indices)
        const int n_tail = min(SC_TAIL, T);
        const int total_runs = total;
        const uint2* tail = a.tail + row * SC_TAIL;
        total += n_tail;
        if (!any_over && total >= Me && total <= SEL_CAP) {
            // ---- gather: G lanes per run (G = the power of two at or above the mean run length, 4 to 32),
            // four runs per lane group in flight, each with its first 3 G entries: all loads of a pass
            // are independent and nothing searches.  Run r's (offset | length << 16) comes from shared
            // memory: the tail of cand_idx while the candidates leave it free, else the histogram bins.
            const bool tail_free = total <= SEL_CAP - 1024;
            int32_t* meta = tail_free ? s.cand_idx + SEL_CAP - 1024 : reinterpret_cast<int32_t*>(s.hist);
            uint32_t kmin = 0xffffffffu, kmax = 0u;
            if (tid < n_runs) meta[tid] = off | (c << 16);
            __syncthreads();
            const uint2* cand = a.cand + row * a.chunks_max * SC_WARPS * a.cap_w;
            const uint2 e_tail = tid < n_tail ? __ldcg(tail + tid) : make_uint2(0u, 0u);   // SC_TAIL <= SEL_THREADS
            int G = 4;
            while (G < 32 && G * n_runs < total_runs) G <<= 1;
            const int rpw = 32 / G, sub = lane / G, li = lane - sub * G;
            const int step_runs = SEL_WARPS * rpw;
            for (int r0 = warp * rpw + sub; r0 < n_runs; r0 += 4 * step_runs) {
                uint2 e[4][3];
                int o[4], n[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int r = r0 + u * step_runs;
                    const int m = r < n_runs ? meta[r] : 0;
                    o[u] = m & 0xffff;
                    n[u] = m >> 16;
#pragma unroll
                    for (int k = 0; k < 3; ++k) {
                        const int i = li + G * k;
                        e[u][k] = make_uint2(0u, 0u);
                        if (i < n[u]) e[u][k] = __ldcg(cand + (size_t)r * a.cap_w + i);
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
#pragma unroll
                    for (int k = 0; k < 3; ++k) {
                        const int i = li + G * k;
                        if (i < n[u]) put(o[u] + i, e[u][k], kmin, kmax);
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {                      // runs longer than 3 G: rare
                    const int r = r0 + u * step_runs;
                    for (int i = li + 3 * G; i < n[u]; i += G)
                        put(o[u] + i, __ldcg(cand + (size_t)r * a.cap_w + i), kmin, kmax);
                }
            }
            if (tid < n_tail) put(total_runs + tid, e_tail, kmin, kmax);
            if (!tail_free) {
                __syncthreads();
                for (int i = tid; i < SEL_BINS; i += SEL_THREADS) s.hist[i] = 0;
            }
            if (packed) block_minmax3(s, kmin, kmax, s_min);
            else block_minmax(s, kmin, kmax);          // also the barrier after the gather
            if (packed) {
                exact = emit_packed_candidates(s, scan, total, Me, kmin, kmax, s_min, chi, K0,
                                               a.probs + (size_t)row * XS_TAB,
                                               a.codes + (size_t)(b * a.Hkv + kvh) * a.Tcap * a.L,
                                               a.v_norm + (size_t)(b * a.Hkv + kvh) * a.Tcap, heavy, a.n_fallback);
            } else {
                uint32_t kth = 0;
                if (!emit_candidates_binned(s, scan, total, Me, Me, kmin, kmax, heavy, kth)) {
                    __syncthreads();
                    kth = emit_from_candidates(s, scan, total, Me, 0, Me, heavy);
                }
                exact = kth >= chi;                    // uniform: kth and chi are block-wide values
            }
        }
        if (!exact) {
            // ---- rescore this row (tables added in the scorer's order), then the full-row select
            if (tid == 0) {
                atomicAdd(a.n_fallback, 1);
                // why: a run overflowed / too few or too many candidates / result not provable on the candidates
                atomicAdd(a.n_fallback + (any_over ? 3 : ((total < Me || total > SEL_CAP) ? 4 : 5)), 1);
            }
            __syncthreads();
            float* tab = reinterpret_cast<float*>(s.cand_key);           // [L][R] of this head
            if (a.probs != nullptr) {
                // packed step: the row's probabilities are the table ([L][R], the very values the fp32
                // scorer table holds), and that table is not written
                const float* pr = a.probs + (size_t)row * a.L * a.R;
                for (int i = tid; i < a.L * a.R; i += SEL_THREADS) tab[i] = __ldcg(pr + i);
            } else {
                const float* lut_g = a.lut + (size_t)g * a.R * a.L * a.ht;
                const int j = hj % a.ht;
                for (int i = tid; i < a.L * a.R; i += SEL_THREADS) {
                    const int l = i / a.R, r = i - l * a.R;
                    tab[i] = __ldcg(lut_g + ((size_t)r * a.L + l) * a.ht + j);
                }
            }
            __syncthreads();
            const uint8_t* cg = a.codes + (size_t)(b * a.Hkv + kvh) * a.Tcap * a.L;
            const __half* vg = a.v_norm + (size_t)(b * a.Hkv + kvh) * a.Tcap;
            for (int t = tid; t < T; t += SEL_THREADS) {
                const uint4* cp = reinterpret_cast<const uint4*>(cg + (size_t)t * a.L);
                const int m = t & 7;                   // the scorer's table order for this key
                float sum = 0.f;
                for (int v = 0; v < a.L / 16; ++v) {
                    const uint4 w4 = __ldcg(cp + v);
                    const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                    for (int q = 0; q < 16; ++q) {
                        const int tb = (q & 8) | ((q & 7) ^ m);
                        sum += tab[(v * 16 + tb) * a.R + ((w[tb >> 2] >> (8 * (tb & 3))) & 0xffu)];
                    }
                }
                sc[t] = sum * __half2float(__ldcg(vg + t));
            }
            __syncthreads();
            select_row(s, scan, sc, T, Me, heavy);
        }
    } else if (Me == T) {
        for (int i = tid; i < T; i += SEL_THREADS) heavy[i] = i;
    }
    __syncthreads();
    finish_row(s, sc, nullptr, out, nb, Me, 0);
}

}  // namespace

int launch_select_list(const float* scores, int64_t score_row_stride, const uint8_t* allowed,
                       int64_t rows, int64_t T, const int32_t* T_dev, int64_t M, int sink,
                       int window, int sorted, int32_t* list, int64_t list_row_stride,
                       int32_t* list_len, int32_t* status, cudaStream_t st) {
    (void)status;
    if (rows <= 0) return SK_OK;
    if (T > 0x7fffffff) return fail(SK_ERR_UNSUPPORTED, "sk_select_list: T too large");
    if (sorted && (M < T ? M : T) > SEL_CAP)
        return fail(SK_ERR_UNSUPPORTED, "sk_select_list: sorted output supports top-k <= %d", SEL_CAP);
    const size_t smem = sizeof(SelShared);
    cudaError_t e = cudaFuncSetAttribute(select_list_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return fail(SK_ERR_CUDA, "select_list_kernel smem attribute: %s", cudaGetErrorString(e));
    // not chained to its predecessor: this kernel reads the score matrix through the read-only cache
    select_list_kernel<<<(unsigned)rows, SEL_THREADS, smem, st>>>(
        scores, score_row_stride, allowed, T, T_dev, M, sink, window, sorted, list, list_row_stride,
        list_len);
    return check_launch("select_list_kernel");
}

int launch_select_candidates(const float* lut, const uint8_t* codes, const uint16_t* v_norm, int B, int H,
                             int Hkv, int L, int R, int64_t T, const int32_t* T_dev, int64_t Tcap, int64_t M,
                             int sink, int window, int sorted, int32_t* list, int64_t list_row_stride,
                             int32_t* list_len, void* workspace, int32_t* status, cudaStream_t st,
                             const float* qpar, const float* probs) {
    (void)status;
    if (sorted) return fail(SK_ERR_UNSUPPORTED, "fused score+select: sorted output not supported");
    const int ht = lut_head_tile(H / Hkv);
    const ScorePlan plan = make_score_plan(B * Hkv * ((H / Hkv) / ht), T, M);
    const int64_t rows = (int64_t)B * H;
    const FusedLayout lay = make_fused_layout(rows, plan, T);
    char* ws = static_cast<char*>(workspace);
    CandArgs a;
    a.cnt = reinterpret_cast<const int32_t*>(ws + lay.cnt);
    a.cut = reinterpret_cast<const float*>(ws + lay.cut);
    a.cand = reinterpret_cast<const uint2*>(ws + lay.cand);
    a.scratch = reinterpret_cast<float*>(ws + lay.scores);
    a.n_fallback = reinterpret_cast<int32_t*>(ws + lay.stats);
    a.score_stride = lay.score_stride;
    a.chunks_max = plan.chunks_max;
    a.cap_w = plan.cap_w;
    a.Tslots = plan.Tslots;
    a.per_cta = plan.per_cta;
    a.lut = lut;
    a.codes = codes;
    a.v_norm = reinterpret_cast<const __half*>(v_norm);
    a.H = H; a.Hkv = Hkv; a.L = L; a.R = R; a.ht = ht;
    a.Tcap = Tcap;
    a.qpar = qpar;
    a.probs = probs;
    a.tail = reinterpret_cast<const uint2*>(ws + lay.tail);
    if ((size_t)L * R * 4 > sizeof(uint32_t) * SEL_CAP)
        return fail(SK_ERR_UNSUPPORTED, "fused score+select: L*R too large for the rescoring table");
    const size_t smem = sizeof(SelShared);
    auto kern = qpar != nullptr ? select_cand_kernel<true> : select_cand_kernel<false>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(SK_ERR_CUDA, "select_cand_kernel smem attribute: %s", cudaGetErrorString(e));
    e = launch_chained(kern, dim3((unsigned)rows), dim3(SEL_THREADS), smem, st, a, T, T_dev, M, sink,
                       window, sorted, list, list_row_stride, list_len);
    if (e != cudaSuccess) return fail(SK_ERR_CUDA, "select_cand_kernel: %s", cudaGetErrorString(e));
    return check_launch("select_cand_kernel");
}

}  // namespace sk
