// Scorer and exact top-k in ONE launch: a thread-block cluster per (KV head, head tile).
//
// The CL CTAs of a cluster split the keys of their KV head evenly; each scores its slice for the
// four query heads of the tile (same table walk and summation order as score_kernel, so the
// scores are bit-identical) and keeps the order-preserving keys of ALL its scores in shared
// memory.  The k-th largest score of each head is then found by a radix select whose histograms
// are combined through distributed shared memory.  All traffic between CTAs is remote STORES
// followed by a cluster barrier, so no CTA ever waits on the latency of a remote load:
//
//   1. every CTA pushes its min / max key to all peers          -> bins = (key - min) >> shift
//   2. every CTA histograms its keys (2048 bins) and pushes slice r of the histogram to CTA r;
//      CTA r sums the CL copies and pushes the totals to all peers; every CTA then scans the
//      full cluster-wide histogram locally                       -> threshold bin b*, keys in
//      higher bins are selected
//   3. the keys of bin b* ("boundary") are few: every CTA pushes its counts, then its boundary
//      (key, index) pairs, to all peers and ranks them by (score descending, index ascending)
//                                                                -> cut-off pair, offsets
//      (more than CS_BCAP boundary keys: refine bin b* by the next 11 key bits first; no bits
//      left means the boundary keys are all equal, and the lowest indices win)
//   4. every CTA writes its selected keys, in ascending index order, at its offset in the list.
//
// The result is the exact top-k with ties going to the lowest index, in ascending index order:
// the same list the two-kernel paths produce.  No score matrix, no candidate buffer, no second
// launch.  Every CTA reaches every cluster barrier on every path (a timed-out table copy only
// sets the status flag), and the only spin is the bounded wait on the table copy.
#include <cooperative_groups.h>

#include "score_body.cuh"

namespace cg = cooperative_groups;

namespace sk {
namespace {

constexpr int CS_THREADS = 1024;
constexpr int CS_WARPS = CS_THREADS / 32;
constexpr int CS_MAX_CL = 16;
constexpr int CS_ITERS_MAX = 5;               // keys per thread
constexpr int CS_KEYS_MAX = CS_ITERS_MAX * CS_THREADS;   // key slots per CTA
constexpr int CS_NB = 2048;                  // bins per radix level
constexpr int CS_NBP = CS_NB + CS_MAX_CL;    // room for the padding of the last slice
constexpr int CS_BITS = 11;
constexpr int CS_BCAP = 256;                 // boundary keys that are ranked pairwise (per head, cluster-wide)
constexpr int CS_SEG = CS_BCAP / CS_MAX_CL;  // boundary pairs per CTA that travel with the counts
constexpr int CS_LUT_BYTES = 256 * 32 * 16;  // R=256 buckets x L=32 tables x 4 heads x fp32
constexpr int CS_HT = 4;

// The table region is dead once the keys are scored; the select phase lays this over it.
struct ClusterScratch {
    uint32_t hist[CS_HT][CS_NBP];            // this CTA's histogram of the current level
    uint32_t parts[CS_HT * CS_NBP];          // [src CTA][head][bin of my slice]: pushed by the peers
    uint32_t tot[CS_HT][CS_NBP];             // cluster-wide histogram: pushed by the slice owners
    uint32_t bkey[CS_HT][CS_BCAP];           // this CTA's boundary keys ...
    int32_t bidx[CS_HT][CS_BCAP];            // ... and their key indices
    uint32_t seg_key[CS_HT][CS_MAX_CL][CS_SEG];   // first boundary pairs of every CTA: pushed by their owners
    int32_t seg_idx[CS_HT][CS_MAX_CL][CS_SEG];
    uint32_t gkey[CS_HT][CS_BCAP];           // all boundary pairs of the cluster, CTA by CTA
    int32_t gidx[CS_HT][CS_BCAP];
};
static_assert(sizeof(ClusterScratch) <= CS_LUT_BYTES, "select scratch must fit in the table region");

struct ClusterShared {
    uint64_t bar;
    uint32_t red_lo[CS_HT][CS_WARPS], red_hi[CS_HT][CS_WARPS];
    uint32_t mm[CS_MAX_CL][CS_HT][2];        // pushed by every CTA: its min, max
    uint32_t cnt[CS_MAX_CL][CS_HT][2];       // pushed by every CTA: keys above the boundary bin, keys in it
    uint32_t kmin[CS_HT];
    int shift[CS_HT];                        // bins of the current level = ((key - kmin) >> shift) & mask
    uint32_t mask[CS_HT];
    int pshift[CS_HT];                       // boundary keys: (key - kmin) >> pshift == prefix
    uint32_t prefix[CS_HT];
    int done[CS_HT];                         // boundary bin small enough (or no key bits left)
    int need[CS_HT];                         // keys still to take from the boundary bin
    int nbt[CS_HT];                          // boundary keys in the whole cluster
    int more[4];                             // per level: some head needs another level
    int round2;                              // a CTA has more boundary pairs than a segment takes
    uint32_t scan[CS_HT][8];                 // per-warp sums of the locate scan
    uint32_t n_above[CS_HT], n_bound[CS_HT]; // local counts
    int goff[CS_HT][CS_MAX_CL + 1];          // boundary keys of the CTAs before r (exclusive prefix)
    int sel_by_cta[CS_HT][CS_MAX_CL];        // pairwise mode: selected boundary keys per CTA
    uint32_t cut_key[CS_HT];                 // pairwise mode: last selected (key, index) pair
    int32_t cut_idx[CS_HT];
    int take[CS_HT];                         // tie mode: boundary keys this CTA takes (lowest indices)
    int out_off[CS_HT];                      // where this CTA's selected keys start in the list
    int32_t warp_sel[CS_HT][CS_WARPS];       // selected keys per warp
    int32_t warp_bnd[CS_HT][CS_WARPS];       // boundary keys per warp (tie mode)
};

struct ClusterArgs {
    const float* lut;
    const uint8_t* codes;
    const __half* v_norm;
    int H, Hkv;
    int64_t T, Tcap, M;
    const int32_t* T_dev;
    int sink, window;
    int32_t* list;
    int64_t list_row_stride;
    int32_t* list_len;
    int32_t* status;
};

template <typename T>
__device__ __forceinline__ T* remote(cg::cluster_group& cluster, T* p, int r) {
    return cluster.map_shared_rank(p, r);
}

__global__ void __launch_bounds__(CS_THREADS, 1)
score_select_cluster_kernel(ClusterArgs a) {
    constexpr int L = 32;
    constexpr int NV = L / 16;
    extern __shared__ __align__(128) char smem_raw[];
    char* lut_s = smem_raw;
    ClusterScratch& cs = *reinterpret_cast<ClusterScratch*>(smem_raw);
    uint32_t* keyS = reinterpret_cast<uint32_t*>(smem_raw + CS_LUT_BYTES);       // [4][CS_KEYS_MAX]
    ClusterShared& s = *reinterpret_cast<ClusterShared*>(smem_raw + CS_LUT_BYTES + CS_HT * CS_KEYS_MAX * 4);

    cg::cluster_group cluster = cg::this_cluster();
    const int CL = (int)cluster.num_blocks();
    const int rank = (int)cluster.block_rank();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const unsigned lt_mask = (1u << lane) - 1u;
    const int g = blockIdx.x / CL;
    const int rep = a.H / a.Hkv, tiles = rep / CS_HT;
    const int tile = g % tiles, bk = g / tiles;
    const int b = bk / a.Hkv, kvh = bk - b * a.Hkv;
    const size_t row0 = (size_t)b * a.H + kvh * rep + tile * CS_HT;

    pdl_launch_dependents();
    pdl_wait();                               // the table, the live length and the newest codes come from the predecessor
    const int T = effective_len(a.T, a.T_dev);
    if (T <= 0) {   // uniform over the grid
        if (rank == 0 && tid < CS_HT) a.list_len[row0 + tid] = 0;
        return;
    }
    const int Me = (int)(a.M < (int64_t)T ? a.M : (int64_t)T);
    const int sink = max(0, min(a.sink, T));
    const int window = max(0, min(a.window, T));
    const int win_start = max(T - window, sink);
    const int n_win = window > 0 ? T - win_start : 0;
    const int nb = sink + n_win == 0 ? 1 : sink + n_win;

    // ---- structured part and lengths: CTA r writes the rows j with j % CL == r
    for (int j = rank; j < CS_HT; j += CL) {
        int32_t* out = a.list + (row0 + j) * a.list_row_stride;
        for (int i = tid; i < sink; i += CS_THREADS) out[i] = i;
        for (int i = tid; i < n_win; i += CS_THREADS) out[sink + i] = win_start + i;
        if (sink + n_win == 0 && tid == 0) out[0] = T - 1;
        if (tid == 0) a.list_len[row0 + j] = nb + Me;
    }
    if (Me <= 0) return;   // uniform

    // ---- this CTA's keys [t_lo, t_lo + n_local); warp w owns kpw consecutive ones, lane l the keys
    // w*kpw + 32*k + l, so that (warp, k, lane) order is ascending key order
    const int per_cta = (T + CL - 1) / CL;
    const int t_lo = rank * per_cta;
    const int n_local = max(0, min(per_cta, T - t_lo));
    const int kpw = (per_cta + CS_WARPS - 1) / CS_WARPS;          // <= 32 * CS_ITERS_MAX (checked on the host)
    const int iters = (kpw + 31) / 32;
    const int w_lo = warp * kpw;

    if (Me == T) {   // uniform: everything is selected, ascending
        for (int j = 0; j < CS_HT; ++j) {
            int32_t* heavy = a.list + (row0 + j) * a.list_row_stride + nb;
            for (int i = tid; i < n_local; i += CS_THREADS) heavy[t_lo + i] = t_lo + i;
        }
        return;
    }

    // ---- score: table to shared memory, keys streamed 16 bytes at a time
    uint64_t* bar = &s.bar;
    if (tid == 0) mbar_init(bar, 1);
    __syncthreads();
    if (tid == 0) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_expect_tx(bar, (uint32_t)CS_LUT_BYTES);
        const char* src = reinterpret_cast<const char*>(a.lut) + (size_t)g * CS_LUT_BYTES;
        for (uint32_t off = 0; off < (uint32_t)CS_LUT_BYTES; off += SC_COPY_CHUNK)
            bulk_g2s(lut_s + off, src + off, SC_COPY_CHUNK, bar);
    }
    // table order of a key: table = j ^ (key index & 7) inside each group of 8, as in score_kernel;
    // a lane's keys are 32 apart, so one permutation per lane
    const int m = (t_lo + w_lo + lane) & 7;
    const uint32_t sel_lo = 0x3210u ^ (0x1111u * m);
    const uint32_t sel_hi = 0x7654u ^ (0x1111u * m);
    const uint32_t mL = (uint32_t)m * 16u;
    const uint4* cgp = reinterpret_cast<const uint4*>(a.codes + (size_t)bk * a.Tcap * L);
    const __half* vg = a.v_norm + (size_t)bk * a.Tcap;
    // key of (k, lane): local index w_lo + 32k + lane, live if inside the warp's and the CTA's range
    auto local_of = [&](int k) { return w_lo + 32 * k + lane; };
    auto live = [&](int k) { return 32 * k + lane < kpw && w_lo + 32 * k + lane < n_local; };

    uint4 cur[NV], nxt[NV];
    float vcur = 0.f, vnxt = 0.f;
    if (live(0)) {
#pragma unroll
        for (int i = 0; i < NV; ++i) cur[i] = __ldcg(cgp + (size_t)(t_lo + local_of(0)) * NV + i);
        vcur = __half2float(__ldcg(vg + t_lo + local_of(0)));
    }
    if (live(1)) {
#pragma unroll
        for (int i = 0; i < NV; ++i) nxt[i] = __ldcg(cgp + (size_t)(t_lo + local_of(1)) * NV + i);
        vnxt = __half2float(__ldcg(vg + t_lo + local_of(1)));
    }
    const bool ok = mbar_wait(bar, 0);
    if (!__syncthreads_and(ok)) {
        // keep going (the cluster barriers below need every CTA); the caller sees the flag
        if (tid == 0 && a.status != nullptr) atomicOr(a.status, SK_DEV_WAIT_TIMEOUT);
    }
    uint32_t lo[CS_HT], hi[CS_HT];
#pragma unroll
    for (int j = 0; j < CS_HT; ++j) {
        lo[j] = 0xffffffffu;
        hi[j] = 0u;
    }
    for (int k = 0; k < iters; ++k) {
        if (live(k)) {
            float acc[CS_HT];
            score_key<L, CS_HT>(cur, lut_s, sel_lo, sel_hi, mL, acc);
#pragma unroll
            for (int j = 0; j < CS_HT; ++j) {
                const uint32_t key = order_key(acc[j] * vcur);
                keyS[j * CS_KEYS_MAX + warp * 32 * iters + 32 * k + lane] = key;
                lo[j] = min(lo[j], key);
                hi[j] = max(hi[j], key);
            }
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) cur[i] = nxt[i];
        vcur = vnxt;
        if (live(k + 2)) {
#pragma unroll
            for (int i = 0; i < NV; ++i) nxt[i] = __ldcg(cgp + (size_t)(t_lo + local_of(k + 2)) * NV + i);
            vnxt = __half2float(__ldcg(vg + t_lo + local_of(k + 2)));
        }
    }
    // shared-memory slot of (k, lane): conflict free, 32 * iters slots per warp
    const uint32_t* myk = keyS + warp * 32 * iters + lane;
    auto key_of = [&](int j, int k) { return myk[j * CS_KEYS_MAX + 32 * k]; };

    // ---- 1. cluster-wide min / max per head
#pragma unroll
    for (int j = 0; j < CS_HT; ++j) {
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
            lo[j] = min(lo[j], __shfl_xor_sync(FULL, lo[j], o));
            hi[j] = max(hi[j], __shfl_xor_sync(FULL, hi[j], o));
        }
        if (lane == 0) {
            s.red_lo[j][warp] = lo[j];
            s.red_hi[j][warp] = hi[j];
        }
    }
    __syncthreads();                          // also: every lookup of the table is done
    if (warp < CS_HT) {
        uint32_t l2 = s.red_lo[warp][lane], h2 = s.red_hi[warp][lane];
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
            l2 = min(l2, __shfl_xor_sync(FULL, l2, o));
            h2 = max(h2, __shfl_xor_sync(FULL, h2, o));
        }
        if (lane < CL) {                      // lane r pushes to CTA r
            uint32_t* dst = remote(cluster, &s.mm[rank][warp][0], lane);
            dst[0] = l2;
            dst[1] = h2;
        }
    }
    // the select scratch overlays the table: clear the first level's histogram and the counters
    for (int i = tid; i < CS_HT * CS_NBP; i += CS_THREADS) (&cs.hist[0][0])[i] = 0u;
    cluster.sync();
    if (warp < CS_HT) {
        uint32_t l2 = 0xffffffffu, h2 = 0u;
        if (lane < CL) {
            l2 = s.mm[lane][warp][0];
            h2 = s.mm[lane][warp][1];
        }
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
            l2 = min(l2, __shfl_xor_sync(FULL, l2, o));
            h2 = max(h2, __shfl_xor_sync(FULL, h2, o));
        }
        if (lane == 0) {
            const uint32_t range = h2 - l2;   // the cluster holds T >= 1 keys, so h2 >= l2
            const int bits = 32 - __clz(range);
            s.kmin[warp] = l2;
            s.shift[warp] = max(bits - CS_BITS, 0);
            s.mask[warp] = (uint32_t)CS_NB - 1u;
            s.pshift[warp] = 0;
            s.prefix[warp] = 0u;
            s.done[warp] = 0;
            s.need[warp] = Me;
            s.nbt[warp] = T;
            s.n_above[warp] = 0u;
            s.n_bound[warp] = 0u;
            s.more[warp] = 0;
            s.round2 = 0;
        }
        if (lane < CS_MAX_CL) s.sel_by_cta[warp][lane] = 0;
    }
    __syncthreads();

    // ---- 2. radix levels: local histogram -> slices to their owners -> totals to everybody -> scan
    const int S = (CS_NB + CL - 1) / CL;      // bins per slice; CL * S <= CS_NBP
    for (int level = 0; level < 3; ++level) {
#pragma unroll
        for (int j = 0; j < CS_HT; ++j) {
            if (level > 0 && s.done[j]) continue;                  // uniform
            const uint32_t kmin = s.kmin[j], prefix = s.prefix[j], mask = s.mask[j];
            const int shift = s.shift[j], pshift = s.pshift[j];
            uint32_t bin[CS_ITERS_MAX];
            bool member[CS_ITERS_MAX];
            uint32_t first = 0xffffffffu;
            int n_mem = 0;
#pragma unroll
            for (int k = 0; k < CS_ITERS_MAX; ++k) {
                const bool valid = k < iters && live(k);
                const uint32_t d = valid ? key_of(j, k) - kmin : 0u;
                member[k] = valid && (level == 0 || (d >> pshift) == prefix);
                bin[k] = (d >> shift) & mask;
                if (member[k]) {
                    first = min(first, bin[k]);
                    ++n_mem;
                }
            }
            // all keys of the warp in one bin (equal scores): one add instead of a serialised pile-up
            const uint32_t wfirst = __reduce_min_sync(FULL, first);
            bool same = true;
#pragma unroll
            for (int k = 0; k < CS_ITERS_MAX; ++k) same = same && (!member[k] || bin[k] == wfirst);
            if (__all_sync(FULL, same)) {
                const int n = __reduce_add_sync(FULL, n_mem);
                if (lane == 0 && n > 0) atomicAdd(&cs.hist[j][wfirst], (uint32_t)n);
            } else {
#pragma unroll
                for (int k = 0; k < CS_ITERS_MAX; ++k)
                    if (member[k]) atomicAdd(&cs.hist[j][bin[k]], 1u);
            }
        }
        __syncthreads();
        // slice r of my histogram -> CTA r (one (head, bin) item per thread and pass; no divisions inside)
        for (int item = tid; item < CS_HT * S; item += CS_THREADS) {
            const int j = item / S, bl = item - j * S;
            uint32_t* dst = &cs.parts[(rank * CS_HT + j) * S + bl];
            const uint32_t* src = &cs.hist[j][bl];
            for (int r = 0; r < CL; ++r) *remote(cluster, dst, r) = src[r * S];
        }
        cluster.sync();
        for (int item = tid; item < CS_HT * S; item += CS_THREADS) {
            const int j = item / S, bl = item - j * S;
            uint32_t v = 0;
            const uint32_t* src = &cs.parts[j * S + bl];
            for (int r = 0; r < CL; ++r) v += src[r * CS_HT * S];
            uint32_t* dst = &cs.tot[j][rank * S + bl];
            for (int r = 0; r < CL; ++r) *remote(cluster, dst, r) = v;
        }
        for (int i = tid; i < CS_HT * CS_NBP; i += CS_THREADS) (&cs.hist[0][0])[i] = 0u;   // for the next level
        cluster.sync();
        {
            // 256 threads per head scan the cluster-wide histogram from the top bin down, 8 bins each
            const int j = tid >> 8, th = tid & 255, w8 = warp & 7;
            const uint32_t need = (uint32_t)s.need[j];
            const bool skip = level > 0 && s.done[j];
            uint32_t c[8], local = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                c[i] = skip ? 0u : cs.tot[j][CS_NB - 1 - (8 * th + i)];
                local += c[i];
            }
            uint32_t inc = local;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t n = __shfl_up_sync(FULL, inc, o);
                if (lane >= o) inc += n;
            }
            if (lane == 31) s.scan[j][w8] = inc;
            __syncthreads();
            uint32_t before = inc - local;
            for (int w = 0; w < w8; ++w) before += s.scan[j][w];
            if (!skip) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (before < need && need <= before + c[i]) {
                        // exactly one thread of the head gets here
                        const int shift = s.shift[j];
                        const uint32_t bin = (uint32_t)(CS_NB - 1 - (8 * th + i));
                        s.prefix[j] = level == 0 ? bin : ((s.prefix[j] << (s.pshift[j] - shift)) | bin);
                        s.pshift[j] = shift;
                        s.need[j] = (int)(need - before);
                        s.nbt[j] = (int)c[i];
                        const bool done = c[i] <= (uint32_t)CS_BCAP || shift == 0;
                        s.done[j] = done ? 1 : 0;
                        if (!done) {
                            const int nshift = max(shift - CS_BITS, 0);
                            s.shift[j] = nshift;
                            s.mask[j] = (1u << (shift - nshift)) - 1u;
                            s.more[level] = 1;
                        }
                    }
                    before += c[i];
                }
            }
        }
        __syncthreads();
        if (!s.more[level]) break;            // same value in every CTA of the cluster
    }

    // ---- 3. classify: keys above the boundary bin are in; boundary keys are listed (or, when they
    // are all equal, only counted).  Counts and the first CS_SEG boundary pairs go to every peer.
#pragma unroll
    for (int j = 0; j < CS_HT; ++j) {
        const uint32_t kmin = s.kmin[j], prefix = s.prefix[j];
        const int pshift = s.pshift[j];
        const bool pairwise = s.nbt[j] <= CS_BCAP;                 // uniform
        int n_ab = 0;
#pragma unroll
        for (int k = 0; k < CS_ITERS_MAX; ++k) {
            const bool valid = k < iters && live(k);
            const uint32_t key = valid ? key_of(j, k) : 0u;
            const uint32_t d = (key - kmin) >> pshift;
            n_ab += (valid && d > prefix) ? 1 : 0;
            const bool bnd = valid && d == prefix;
            if (pairwise) {
                if (bnd) {                                         // a handful per cluster
                    const uint32_t pos = atomicAdd(&s.n_bound[j], 1u);
                    if (pos < (uint32_t)CS_BCAP) {                 // always true: the cluster has <= CS_BCAP of them
                        cs.bkey[j][pos] = key;
                        cs.bidx[j][pos] = t_lo + local_of(k);
                    }
                }
            } else {
                const unsigned bb = __ballot_sync(FULL, bnd);
                if (lane == 0 && bb != 0u) atomicAdd(&s.n_bound[j], (uint32_t)__popc(bb));
            }
        }
        n_ab = __reduce_add_sync(FULL, n_ab);
        if (lane == 0 && n_ab != 0) atomicAdd(&s.n_above[j], (uint32_t)n_ab);
    }
    __syncthreads();
    if (tid < CS_HT * CL) {
        const int j = tid / CL, r = tid - j * CL;
        uint32_t* dst = remote(cluster, &s.cnt[rank][j][0], r);
        dst[0] = s.n_above[j];
        dst[1] = s.n_bound[j];
    }
    {
        const int j = tid >> 8, th = tid & 255;
        const int e = th / CL, r = th - e * CL;
        if (s.nbt[j] <= CS_BCAP && e < min((int)s.n_bound[j], CS_SEG)) {
            *remote(cluster, &cs.seg_key[j][rank][e], r) = cs.bkey[j][e];
            *remote(cluster, &cs.seg_idx[j][rank][e], r) = cs.bidx[j][e];
        }
    }
    cluster.sync();
    if (tid < CS_HT) {
        int acc = 0;
        bool over = false;
        for (int r = 0; r < CL; ++r) {
            s.goff[tid][r] = acc;
            acc += (int)s.cnt[r][tid][1];
            over = over || (int)s.cnt[r][tid][1] > CS_SEG;
        }
        s.goff[tid][CL] = acc;
        if (over && s.nbt[tid] <= CS_BCAP) s.round2 = 1;           // same outcome in every CTA
    }
    __syncthreads();
    if (s.round2) {
        // some CTA holds more boundary pairs than a segment takes: everybody sends all of its pairs,
        // at its offset in the cluster-wide list
#pragma unroll
        for (int j = 0; j < CS_HT; ++j) {
            if (s.nbt[j] > CS_BCAP) continue;                      // tie mode: nothing to exchange
            const int mine = min((int)s.n_bound[j], CS_BCAP), off = s.goff[j][rank];
            for (int i = tid; i < mine * CL; i += CS_THREADS) {
                const int r = i / mine, e = i - r * mine;
                if (off + e < CS_BCAP) {
                    *remote(cluster, &cs.gkey[j][off + e], r) = cs.bkey[j][e];
                    *remote(cluster, &cs.gidx[j][off + e], r) = cs.bidx[j][e];
                }
            }
        }
        cluster.sync();                       // last remote access
    } else {
        // the segments hold everything: compact them into one list per head (no remote access after
        // the barrier above, so CTAs may run ahead and exit from here on)
        const int j = tid >> 8, th = tid & 255;
        if (s.nbt[j] <= CS_BCAP && th < min(s.goff[j][CL], CS_BCAP)) {
            int r = 0;
            for (int q = 1; q < CL; ++q) r += (s.goff[j][q] <= th) ? 1 : 0;
            cs.gkey[j][th] = cs.seg_key[j][r][th - s.goff[j][r]];
            cs.gidx[j][th] = cs.seg_idx[j][r][th - s.goff[j][r]];
        }
        __syncthreads();
    }
    {
        const int j = tid >> 8, th = tid & 255;
        const bool pairwise = s.nbt[j] <= CS_BCAP;
        const int need = s.need[j];
        const int nbt = min(s.goff[j][CL], CS_BCAP);
        if (pairwise) {
            for (int e = th; e < nbt; e += 256) {
                const uint32_t ke = cs.gkey[j][e];
                const int32_t ie = cs.gidx[j][e];
                int rk = 0;
                for (int f = 0; f < nbt; ++f) {
                    const uint32_t kf = cs.gkey[j][f];
                    rk += (kf > ke || (kf == ke && cs.gidx[j][f] < ie)) ? 1 : 0;
                }
                if (rk < need) {
                    int r = 0;
                    for (int q = 1; q < CL; ++q) r += (s.goff[j][q] <= e) ? 1 : 0;
                    atomicAdd(&s.sel_by_cta[j][r], 1);
                }
                if (rk == need - 1) {
                    s.cut_key[j] = ke;
                    s.cut_idx[j] = ie;
                }
            }
        }
        __syncthreads();
        if (th == 0) {
            int off = 0;
            for (int r = 0; r < rank; ++r) {
                const int nbc = s.goff[j][r + 1] - s.goff[j][r];
                const int selb = pairwise ? s.sel_by_cta[j][r] : max(0, min(need - s.goff[j][r], nbc));
                off += (int)s.cnt[r][j][0] + selb;
            }
            s.out_off[j] = off;
            const int mine = s.goff[j][rank + 1] - s.goff[j][rank];
            s.take[j] = pairwise ? 0 : max(0, min(need - s.goff[j][rank], mine));
        }
    }
    __syncthreads();

    // ---- 4. emit this CTA's selected keys in ascending index order
    unsigned sel_mask[CS_HT][CS_ITERS_MAX];
    if (s.nbt[0] > CS_BCAP || s.nbt[1] > CS_BCAP || s.nbt[2] > CS_BCAP || s.nbt[3] > CS_BCAP) {
        // tie mode somewhere: boundary keys are taken in index order, so their per-warp counts come first
#pragma unroll
        for (int j = 0; j < CS_HT; ++j) {
            int n = 0;
            for (int k = 0; k < iters; ++k) {
                const bool valid = live(k);
                const uint32_t d = valid ? (key_of(j, k) - s.kmin[j]) >> s.pshift[j] : 0u;
                n += __popc(__ballot_sync(FULL, valid && d == s.prefix[j]));
            }
            if (lane == 0) s.warp_bnd[j][warp] = n;
        }
        __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < CS_HT; ++j) {
        const uint32_t kmin = s.kmin[j], prefix = s.prefix[j];
        const int pshift = s.pshift[j];
        const bool pairwise = s.nbt[j] <= CS_BCAP;
        const uint32_t cut_key = s.cut_key[j];
        const int32_t cut_idx = s.cut_idx[j];
        int bnd_before = 0;
        if (!pairwise) {
            int v = lane < warp ? s.warp_bnd[j][lane] : 0;
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
            bnd_before = v;
        }
        const int take = s.take[j];
        int n_sel = 0;
#pragma unroll
        for (int k = 0; k < CS_ITERS_MAX; ++k) {
            sel_mask[j][k] = 0u;
            if (k < iters) {
                const bool valid = live(k);
                const uint32_t key = valid ? key_of(j, k) : 0u;
                const uint32_t d = (key - kmin) >> pshift;
                bool sel = valid && d > prefix;
                const bool bnd = valid && d == prefix;
                if (pairwise) {
                    sel = sel || (bnd && (key > cut_key || (key == cut_key && t_lo + local_of(k) <= cut_idx)));
                } else {
                    const unsigned bb = __ballot_sync(FULL, bnd);
                    sel = sel || (bnd && bnd_before + __popc(bb & lt_mask) < take);
                    bnd_before += __popc(bb);
                }
                sel_mask[j][k] = __ballot_sync(FULL, sel);
                n_sel += __popc(sel_mask[j][k]);
            }
        }
        if (lane == 0) s.warp_sel[j][warp] = n_sel;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < CS_HT; ++j) {
        int before = lane < warp ? s.warp_sel[j][lane] : 0;
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) before += __shfl_xor_sync(FULL, before, o);
        int32_t* heavy = a.list + (row0 + j) * a.list_row_stride + nb + s.out_off[j] + before;
#pragma unroll
        for (int k = 0; k < CS_ITERS_MAX; ++k) {
            const unsigned mk = sel_mask[j][k];
            if (k < iters && mk != 0u) {                           // warp-uniform
                if ((mk >> lane) & 1u) heavy[__popc(mk & lt_mask)] = t_lo + local_of(k);
                heavy += __popc(mk);
            }
        }
    }
}

}  // namespace

namespace {

constexpr size_t CS_SMEM = CS_LUT_BYTES + (size_t)CS_HT * CS_KEYS_MAX * 4 + sizeof(ClusterShared);

void cluster_config(cudaLaunchConfig_t& cfg, cudaLaunchAttribute& attr, int cl, int n_clusters, cudaStream_t st) {
    cfg = cudaLaunchConfig_t{};
    cfg.gridDim = dim3((unsigned)(n_clusters * cl), 1, 1);
    cfg.blockDim = dim3(CS_THREADS, 1, 1);
    cfg.dynamicSmemBytes = CS_SMEM;
    cfg.stream = st;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = (unsigned)cl;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
}

// Clusters of `cl` CTAs that can be resident at once on the current device (0: configuration not
// available).  Asked once per device and cluster size.
int cluster_capacity(int cl) {
    static int cached[64][CS_MAX_CL + 1];
    static bool known[64][CS_MAX_CL + 1];
    int dev = 0;
    if (cl < 1 || cl > CS_MAX_CL || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (known[dev][cl]) return cached[dev][cl];
    int n = 0;
    cudaError_t e = cudaFuncSetAttribute(score_select_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)CS_SMEM);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(score_select_cluster_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e == cudaSuccess) {
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attr;
        cluster_config(cfg, attr, cl, 1, nullptr);
        e = cudaOccupancyMaxActiveClusters(&n, score_select_cluster_kernel, &cfg);
    }
    if (e != cudaSuccess) {
        (void)cudaGetLastError();   // not an error of the caller: the path is simply not offered
        n = 0;
    }
    cached[dev][cl] = n;
    known[dev][cl] = true;
    return n;
}

}  // namespace

// Cluster size the one-launch scorer + select would use for this shape on the current device, or 0
// when the shape is outside it: L = 32, R = 256, four query heads per table word, every cluster
// resident at once, and at most CS_ITERS_MAX keys per thread.  Among the sizes that qualify the one
// that puts the most CTAs to work wins (ties: the larger cluster).
int score_select_cluster_size(int B, int H, int Hkv, int L, int R, int64_t T, int64_t M) {
    if (B <= 0 || H <= 0 || Hkv <= 0 || H % Hkv || L != 32 || R != 256 || T <= 0 || M < 0) return 0;
    if (T > 0x7fffffff) return 0;
    const int rep = H / Hkv;
    if (lut_head_tile(rep) != CS_HT) return 0;
    const int64_t n_groups = (int64_t)B * Hkv * (rep / CS_HT);
    int best = 0;
    for (int cl = CS_MAX_CL; cl >= 2; --cl) {
        const int64_t per_cta = (T + cl - 1) / cl;
        const int64_t kpw = (per_cta + CS_WARPS - 1) / CS_WARPS;
        if (kpw > 32 * CS_ITERS_MAX) break;           // smaller clusters only get more keys per CTA
        if (n_groups <= cluster_capacity(cl) && best == 0) best = cl;
    }
    return best;
}

int launch_score_select_cluster(const float* lut, const uint8_t* codes, const uint16_t* v_norm, int B, int H,
                                int Hkv, int L, int R, int64_t T, const int32_t* T_dev, int64_t Tcap, int64_t M,
                                int sink, int window, int32_t* list, int64_t list_row_stride, int32_t* list_len,
                                int32_t* status, cudaStream_t st) {
    const int cl = score_select_cluster_size(B, H, Hkv, L, R, T, M);
    if (cl == 0) return fail(SK_ERR_UNSUPPORTED, "one-launch scorer + select: shape or device outside its range");
    ClusterArgs a;
    a.lut = lut;
    a.codes = codes;
    a.v_norm = reinterpret_cast<const __half*>(v_norm);
    a.H = H;
    a.Hkv = Hkv;
    a.T = T;
    a.Tcap = Tcap;
    a.M = M;
    a.T_dev = T_dev;
    a.sink = sink;
    a.window = window;
    a.list = list;
    a.list_row_stride = list_row_stride;
    a.list_len = list_len;
    a.status = status;
    const int n_groups = B * Hkv * ((H / Hkv) / CS_HT);
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr;
    cluster_config(cfg, attr, cl, n_groups, st);
    cudaError_t e = cudaLaunchKernelEx(&cfg, score_select_cluster_kernel, a);
    if (e != cudaSuccess)
        return fail(SK_ERR_CUDA, "score_select_cluster_kernel (clusters of %d): %s", cl, cudaGetErrorString(e));
    return check_launch("score_select_cluster_kernel");
}

}  // namespace sk
