// Top-k select + sparse-list assembly, one CTA per (batch, query head) row.
//
// Exact radix select on order-preserving uint32 keys with deterministic tie-breaking (among
// equal scores the smallest index wins) and ordered, atomic-free compaction (warp ballots +
// block prefix scans), so the output is a pure function of the scores.
//
// Rows that fit the shared-memory candidate buffer are selected entirely on chip.  Longer
// rows take two streaming passes: a 4096-bin histogram over a range found by sampling
// (bins are linear in the key between the sampled min and max, clamped outside, which keeps
// the map monotone), then one pass that emits every element above the threshold bin and
// collects the threshold bin's elements as on-chip candidates.  A row whose threshold bin
// overflows the buffer (e.g. all scores equal) falls back to the textbook 4-pass radix
// select over global memory.
#include "common.cuh"

namespace sk {
namespace {

constexpr int SEL_THREADS = 1024;
constexpr int SEL_WARPS = SEL_THREADS / 32;
constexpr int SEL_CAP = 16384;
constexpr int SEL_BINS = 4096;
constexpr int SEL_CHUNK = SEL_THREADS * 4;

struct SelShared {
    uint32_t hist[SEL_BINS];
    uint32_t cand_key[SEL_CAP];
    int32_t cand_idx[SEL_CAP];
    int scan_buf[2][40];
    uint32_t red_lo[SEL_WARPS], red_hi[SEL_WARPS];
    int thr_bin, thr_above, thr_inbin;
    uint32_t digit, digit_above;
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

// One 8-bit radix step over `count(d)` = hist[d]: finds the digit d with
// #(digit > d) < remaining <= #(digit >= d).  Executed by warp 0; results in shared memory.
__device__ __forceinline__ void find_digit(SelShared& s, uint32_t remaining) {
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        uint32_t c[8];
        uint32_t local = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            c[j] = s.hist[255 - (8 * lane + j)];
            local += c[j];
        }
        uint32_t inc = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t n = __shfl_up_sync(FULL, inc, o);
            if (lane >= o) inc += n;
        }
        uint32_t before = inc - local;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (before < remaining && before + c[j] >= remaining) {
                s.digit = 255 - (8 * lane + j);
                s.digit_above = before;
            }
            before += c[j];
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
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t row = blockIdx.x;
    const float* sc = scores + row * score_row_stride;
    const uint8_t* al = allowed ? allowed + row * T_host : nullptr;
    int32_t* out = list + row * list_row_stride;
    const int T = effective_len(T_host, T_dev);
    Scan scan;

    if (T <= 0) {
        if (tid == 0) list_len[row] = 0;
        return;
    }
    // ---- structured part: sink prefix and local window
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
    const int Me = (int)(M < (int64_t)T ? M : (int64_t)T);
    if (tid == 0) list_len[row] = nb + Me;
    int32_t* heavy = out + nb;

    if (Me == T) {
        for (int i = tid; i < T; i += SEL_THREADS) heavy[i] = i;
    } else if (Me > 0) {
        int n_cand = 0;        // candidates in shared memory
        int need = Me;         // how many of them to take
        int out_pos = 0;       // heavy entries already emitted
        bool global_fallback = false;

        if (T <= SEL_CAP) {
            for (int i = tid; i < T; i += SEL_THREADS) {
                s.cand_key[i] = order_key(sc[i]);
                s.cand_idx[i] = i;
            }
            n_cand = T;
            __syncthreads();
        } else {
            // ---- sampled range
            uint32_t kmin = 0xffffffffu, kmax = 0u;
            const int stride = T / SEL_CHUNK;
            for (int j = 0; j < 4; ++j) {
                const int t = (tid * 4 + j) * stride;
                const float f = sc[t];
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
            // ---- pass 1: histogram
            for (int t = tid; t < T; t += SEL_THREADS) atomicAdd(&s.hist[bin(order_key(sc[t]))], 1u);
            __syncthreads();
            {
                int c[4], local = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    c[j] = (int)s.hist[SEL_BINS - 1 - (4 * tid + j)];
                    local += c[j];
                }
                int total;
                int before = scan.excl(local, total, s);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (before < Me && before + c[j] >= Me) {
                        s.thr_bin = SEL_BINS - 1 - (4 * tid + j);
                        s.thr_above = before;
                        s.thr_inbin = c[j];
                    }
                    before += c[j];
                }
            }
            __syncthreads();
            const int thr = s.thr_bin;
            const int above = s.thr_above;
            const int inbin = s.thr_inbin;
            if (inbin > SEL_CAP) {
                global_fallback = true;
            } else {
                // ---- pass 2: emit the sure ones, keep the threshold bin on chip (index order)
                int sure_base = 0, cand_base = 0;
                for (int base = 0; base < T; base += SEL_CHUNK) {
                    const int t0 = base + tid * 4;
                    uint32_t k[4];
                    int cls[4];  // 2 = sure, 1 = candidate
                    int n_sure = 0, n_cnd = 0;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        cls[j] = 0;
                        if (t0 + j < T) {
                            k[j] = order_key(sc[t0 + j]);
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
                    for (int j = 0; j < 4; ++j) {
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
                }
                out_pos = above;
                need = Me - above;
                n_cand = inbin;
                __syncthreads();
            }
        }

        if (!global_fallback) {
            // ---- exact select among the on-chip candidates: 4 x 8-bit radix from the top
            uint32_t prefix = 0, mask = 0, remaining = (uint32_t)need;
            for (int shift = 24; shift >= 0; shift -= 8) {
                for (int i = tid; i < 256; i += SEL_THREADS) s.hist[i] = 0;
                __syncthreads();
                for (int i = tid; i < n_cand; i += SEL_THREADS) {
                    const uint32_t k = s.cand_key[i];
                    if ((k & mask) == prefix) atomicAdd(&s.hist[(k >> shift) & 0xffu], 1u);
                }
                __syncthreads();
                find_digit(s, remaining);
                __syncthreads();
                remaining -= s.digit_above;
                prefix |= s.digit << shift;
                mask |= 0xffu << shift;
            }
            // prefix = k-th key, remaining = how many equal to it are taken (lowest index first)
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
                const int gt = live && k > prefix, eq = live && k == prefix;
                int total;
                const int off = scan.excl(gt | (eq << 16), total, s);
                const int gt_before = gt_base + (off & 0xffff);
                const int eq_before = eq_base + (off >> 16);
                const int eq_taken_before = min(eq_before, (int)remaining);
                const int dst = out_pos + gt_before + eq_taken_before;
                if ((gt || (eq && eq_before < (int)remaining)) && dst < Me) heavy[dst] = idx;
                gt_base += total & 0xffff;
                eq_base += total >> 16;
            }
        } else {
            // ---- fallback: radix select over the whole row in global memory
            uint32_t prefix = 0, mask = 0, remaining = (uint32_t)Me;
            for (int shift = 24; shift >= 0; shift -= 8) {
                for (int i = tid; i < 256; i += SEL_THREADS) s.hist[i] = 0;
                __syncthreads();
                for (int t = tid; t < T; t += SEL_THREADS) {
                    const uint32_t k = order_key(sc[t]);
                    if ((k & mask) == prefix) atomicAdd(&s.hist[(k >> shift) & 0xffu], 1u);
                }
                __syncthreads();
                find_digit(s, remaining);
                __syncthreads();
                remaining -= s.digit_above;
                prefix |= s.digit << shift;
                mask |= 0xffu << shift;
            }
            int gt_base = 0, eq_base = 0;
            for (int base = 0; base < T; base += SEL_CHUNK) {
                const int t0 = base + tid * 4;
                int gt[4], eq[4], n_gt = 0, n_eq = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
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
                for (int j = 0; j < 4; ++j) {
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
    __syncthreads();

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
    select_list_kernel<<<(unsigned)rows, SEL_THREADS, smem, st>>>(
        scores, score_row_stride, allowed, T, T_dev, M, sink, window, sorted, list, list_row_stride,
        list_len);
    return check_launch("select_list_kernel");
}

}  // namespace sk
