// Row-parallel projection of a decode step fused with the sum over the tensor-parallel ranks:
//
//     out[b, :] = res[b, :] + sum_r  x_r[b, :] . W_r[:, :]^T          (b < B <= 8 new tokens)
//
// where rank r holds the activation slice x_r [B, K] and the weight shard W_r [N, K] (the
// input-column block of `wo` / `w2` that GPT-FAST/tp.py:130,122 gives it).  The reference runs the
// GEMM and then a separate NCCL all-reduce (tp.py:117-118,139-140); for messages of 8-128 KiB that
// collective is pure latency (about 20 us per call, twice per layer).  Here ONE kernel does both:
//
//   1. a CTA owns 32 (64 for wide models) output columns: it streams its rows of W_r once (16-byte
//      loads, several in flight per lane) with x_r staged in shared memory.  The products run on
//      the tensor cores as 16 x 8 x 16 tiles - 16 weight rows against the (up to) 8 tokens of the
//      batch, which is exactly the B operand's width - so a 16-byte piece of W costs one load and
//      a quarter of an mma instead of 8 B fused multiply-adds and as many conversions; each warp
//      takes a contiguous part of K and the warps' tiles are added in warp order.  (K not a
//      multiple of 32: a scalar loop, rows side by side per warp.)
//   2. it PUSHES its partial sums straight into every rank's receive buffer over NVLink as 8-byte
//      words {value (fp32), call number}: such a store arrives whole, so the word validates itself
//      and no fence, flag or second hop is needed (the "low latency" protocol of collective
//      libraries);
//   3. it polls its own receive buffer until the words of all `world` ranks for the columns it
//      owns carry this call's number - the CTAs with the same index on the other ranks are their
//      only producers - and adds the values in rank order (every rank gets the same bits), plus
//      the residual, and writes `out`.
//
// No CTA waits for a CTA of its own grid, the grid never exceeds the number of SMs (all CTAs are
// resident), and every wait is bounded: when it runs out the kernel sets SK_DEV_WAIT_TIMEOUT and
// carries on with whatever has arrived, so a missing peer costs a wrong value, never a hang.
//
// Buffers: every rank allocates the same peer-mapped block of receive slots (host side: torch's
// symmetric memory; `peer_base[r]` is rank r's block as this GPU addresses it).  The slots are
// double-buffered by call parity: a rank can be at most one call ahead of a peer (it needs that
// peer's words of the current call to finish it), so call n+2 never overwrites words a peer still
// reads for call n, and a word left by call n-2 never carries call n's number.  The per-CTA call
// counter lives in this GPU's own memory, so a CUDA graph can replay the call.
#include "common.cuh"

namespace sk {
namespace {

constexpr int GA_THREADS = 256;
constexpr int GA_WARPS = GA_THREADS / 32;
constexpr int GA_MAX_COLS = 64;                // output columns per CTA: 32, or 64 when 32 would need more CTAs than SMs
constexpr int GA_MAXB = 8;
constexpr int GA_MAX_WORLD = 8;
constexpr uint32_t GA_WAIT_LIMIT = 1u << 21;   // polls (with a short sleep each) before giving up: ~0.1 s

// one 8-byte word {value, call number}: written and read whole
__device__ __forceinline__ void st_word(uint2* p, float v, uint32_t epoch) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(epoch) : "memory");
}
__device__ __forceinline__ uint2 ld_word(const uint2* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void unpack8(const uint4& w, const __nv_bfloat16*, float (&f)[8]) {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(u[i] << 16);
        f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ void unpack8(const uint4& w, const __half*, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&w);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = __half22float2(h[i]);
        f[2 * i] = v.x;
        f[2 * i + 1] = v.y;
    }
}

// D (16 x 8, fp32) += A (16 x 16, row-major) * B (16 x 8, column-major)
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1, const __nv_bfloat16*) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1, const __half*) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename T, int GA_COLS>
__global__ void __launch_bounds__(GA_THREADS, 1)
gemv_allreduce_kernel(const T* __restrict__ x, const T* __restrict__ W, int64_t w_row_stride,
                      const T* __restrict__ res, T* __restrict__ out, int B, int N, int K,
                      void* const* __restrict__ peer_base, int world, int rank,
                      int max_batch, int n_pad, uint32_t* __restrict__ counters, int32_t* status) {
    extern __shared__ __align__(16) char ga_smem[];
    const int KS = K + 8;                                 // row stride of x_s: 16 bytes of padding spread the rows over the banks
    T* x_s = reinterpret_cast<T*>(ga_smem);                                           // [B][KS]
    // [GA_MAX_WORLD][GA_MAXB][GA_COLS] partial values; the warps' tiles of step 1 sit behind its first [GA_MAXB][GA_MAX_COLS]
    float* y_s = reinterpret_cast<float*>(ga_smem + (((size_t)B * KS * sizeof(T) + 15) & ~(size_t)15));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int blk = blockIdx.x, n0 = blk * GA_COLS;
    const uint32_t epoch = counters[blk] + 1u;            // this call's number for this CTA, the same on every rank
    const int slot = (int)(epoch & 1u);

    // ---- 1. activations to shared memory, then this CTA's rows of W
    for (int i = tid; i < B * (K / 8); i += GA_THREADS) {
        const int b = i / (K / 8), c = i - b * (K / 8);
        reinterpret_cast<uint4*>(x_s + (size_t)b * KS)[c] = reinterpret_cast<const uint4*>(x)[i];
    }
    __syncthreads();
    constexpr int RPW = GA_COLS / GA_WARPS;               // rows per warp, walked side by side
    if ((K & 31) == 0) {
        // Tensor-core tiles.  Lane (g, t) = (lane / 4, lane % 4) loads 16 bytes = elements
        // k0 + 8 t .. k0 + 8 t + 7 of weight rows g and g + 8 of each 16-row tile and of token g's
        // activations; the four lanes of a row cover 32 consecutive k.  A dot product does not care in
        // which order k is walked, so the 16 k of one mma are taken to be the lanes' register pairs
        // (elements 8 t + {0,1} and 8 t + {2,3} for the first mma of a block, + {4,5} and {6,7} for the
        // second), the same for A and B: no shuffles, no shared-memory staging of W.
        constexpr int TILES = GA_COLS / 16;
        const int g = lane >> 2, t = lane & 3;
        const int n_kb = K >> 5;                          // blocks of 32 k
        const int kb0 = (int)(((int64_t)warp * n_kb) / GA_WARPS), kb1 = (int)(((int64_t)(warp + 1) * n_kb) / GA_WARPS);
        float acc[TILES][4];
#pragma unroll
        for (int rt = 0; rt < TILES; ++rt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[rt][i] = 0.f;
        const T* wrow[TILES][2];
#pragma unroll
        for (int rt = 0; rt < TILES; ++rt) {
            // rows past the end repeat the last one; their results are never stored
            wrow[rt][0] = W + (size_t)min(n0 + rt * 16 + g, N - 1) * w_row_stride + 8 * t;
            wrow[rt][1] = W + (size_t)min(n0 + rt * 16 + g + 8, N - 1) * w_row_stride + 8 * t;
        }
        const T* xrow = x_s + (size_t)min(g, B - 1) * KS + 8 * t;
        const bool token = g < B;
        // (unrolled: 32 independent loads per lane, 128 KiB per CTA, are issued before the first is
        // consumed - the rows are streamed once and only the bytes in flight hide the memory latency)
#pragma unroll (16 / TILES)
        for (int kb = kb0; kb < kb1; ++kb) {
            const int k0 = kb << 5;
            uint4 wa[TILES], wb[TILES];
#pragma unroll
            for (int rt = 0; rt < TILES; ++rt) {          // 2 TILES independent 16-byte loads in flight
                wa[rt] = __ldg(reinterpret_cast<const uint4*>(wrow[rt][0] + k0));
                wb[rt] = __ldg(reinterpret_cast<const uint4*>(wrow[rt][1] + k0));
            }
            uint4 xv = *reinterpret_cast<const uint4*>(xrow + k0);
            if (!token) xv = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int rt = 0; rt < TILES; ++rt) {
                mma16816(acc[rt], wa[rt].x, wb[rt].x, wa[rt].y, wb[rt].y, xv.x, xv.y, (const T*)nullptr);
                mma16816(acc[rt], wa[rt].z, wb[rt].z, wa[rt].w, wb[rt].w, xv.z, xv.w, (const T*)nullptr);
            }
        }
        // acc[rt] = {(row g, token 2t), (row g, token 2t+1), (row g+8, token 2t), (row g+8, token 2t+1)}
        // of this warp's part of K: the warps' parts meet in shared memory and are added in warp order
        float* red_s = y_s + GA_MAXB * GA_MAX_COLS;       // [GA_WARPS][GA_MAXB][GA_COLS], inside the y_s block
#pragma unroll
        for (int rt = 0; rt < TILES; ++rt) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int b = 2 * t + (i & 1), col = rt * 16 + g + ((i >> 1) << 3);
                red_s[(warp * GA_MAXB + b) * GA_COLS + col] = acc[rt][i];
            }
        }
        __syncthreads();
        for (int idx = tid; idx < B * GA_COLS; idx += GA_THREADS) {
            const int b = idx / GA_COLS, col = idx - b * GA_COLS;
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < GA_WARPS; ++w) v += red_s[(w * GA_MAXB + b) * GA_COLS + col];
            y_s[b * GA_COLS + col] = v;
        }
    } else {
        const int nw = n0 + warp * RPW;
        float acc[RPW][GA_MAXB];
#pragma unroll
        for (int rr = 0; rr < RPW; ++rr)
#pragma unroll
            for (int b = 0; b < GA_MAXB; ++b) acc[rr][b] = 0.f;
        // (unrolled: several iterations' loads are issued before the first is consumed - the rows are
        // streamed once and only the bytes in flight hide the memory latency)
#pragma unroll 4
        for (int c = lane; c < K / 8; c += 32) {
            uint4 wv[RPW];
#pragma unroll
            for (int rr = 0; rr < RPW; ++rr) {            // RPW independent 16-byte loads in flight
                const int n = min(nw + rr, N - 1);        // rows past the end repeat the last one; never stored
                wv[rr] = __ldg(reinterpret_cast<const uint4*>(W + (size_t)n * w_row_stride) + c);
            }
#pragma unroll
            for (int b = 0; b < GA_MAXB; ++b) {
                if (b < B) {
                    float xf[8];
                    unpack8(*reinterpret_cast<const uint4*>(x_s + (size_t)b * KS + c * 8), (const T*)nullptr, xf);
#pragma unroll
                    for (int rr = 0; rr < RPW; ++rr) {
                        float wf[8];
                        unpack8(wv[rr], (const T*)nullptr, wf);
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[rr][b] = fmaf(wf[i], xf[i], acc[rr][b]);
                    }
                }
            }
        }
#pragma unroll
        for (int rr = 0; rr < RPW; ++rr) {
#pragma unroll
            for (int b = 0; b < GA_MAXB; ++b) {
                if (b < B) {
                    float v = acc[rr][b];
#pragma unroll
                    for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
                    if (lane == 0) y_s[b * GA_COLS + warp * RPW + rr] = v;
                }
            }
        }
    }
    __syncthreads();

    // ---- 2. push the partial rows to every rank (this one included)
    // receive layout of a rank: [slot][source rank][batch row][n_pad] words
    for (int idx = warp; idx < world * B; idx += GA_WARPS) {
        const int r = idx / B, b = idx - r * B;
        uint2* dst = reinterpret_cast<uint2*>(peer_base[r]) +
                     (((size_t)slot * world + rank) * max_batch + b) * n_pad + n0;
#pragma unroll
        for (int l = lane; l < GA_COLS; l += 32)
            if (n0 + l < N) st_word(dst + l, y_s[b * GA_COLS + l], epoch);
    }

    // ---- 3. collect this CTA's columns from every rank: a thread polls one word at a time
    const uint2* mine = reinterpret_cast<const uint2*>(peer_base[rank]);
    float* part_s = y_s;                                  // reused: [world][B][GA_COLS] partial values
    __syncthreads();                                      // y_s has been read by the pushing warps
    bool late = false;
    for (int idx = tid; idx < world * B * GA_COLS; idx += GA_THREADS) {
        const int l = idx % GA_COLS, rb = idx / GA_COLS;  // rb = r * B + b
        const int r = rb / B, b = rb - r * B;
        float v = 0.f;
        if (n0 + l < N) {
            const uint2* src = mine + (((size_t)slot * world + r) * max_batch + b) * n_pad + n0 + l;
            uint2 w = ld_word(src);
            uint32_t it = 0;
            while (w.y != epoch) {
                if (++it >= GA_WAIT_LIMIT) {
                    late = true;
                    break;
                }
                __nanosleep(20);
                w = ld_word(src);
            }
            v = __uint_as_float(w.x);
        }
        part_s[idx] = v;
    }
    if (late && status != nullptr) atomicOr(status, SK_DEV_WAIT_TIMEOUT);
    __syncthreads();
    for (int idx = tid; idx < B * GA_COLS; idx += GA_THREADS) {
        const int b = idx / GA_COLS, l = idx - b * GA_COLS;
        const int n = n0 + l;
        if (n < N) {
            float s = res != nullptr ? to_f32(res[(size_t)b * N + n]) : 0.f;
            for (int r = 0; r < world; ++r) s += part_s[(r * B + b) * GA_COLS + l];
            out[(size_t)b * N + n] = from_f32<T>(s);
        }
    }
    if (tid == 0) counters[blk] = epoch;
}

}  // namespace

// Columns per CTA: as few as keep the grid within the SMs (every CTA must be resident); 0 = too wide.
static int gemv_allreduce_cols(int N) {
    for (int cols = 32; cols <= GA_MAX_COLS; cols *= 2)
        if ((N + cols - 1) / cols <= sm_count()) return cols;
    return 0;
}
size_t gemv_allreduce_buffer_bytes(int world, int max_batch, int N) {
    const int n_pad = (N + GA_MAX_COLS - 1) / GA_MAX_COLS * GA_MAX_COLS;
    return sk_up256((size_t)2 * world * max_batch * n_pad * sizeof(uint2));
}

int launch_gemv_allreduce(const void* x, const void* W, int64_t w_row_stride, const void* res, void* out, int dtype,
                          int B, int N, int K, void* const* peer_base, int world, int rank, int max_batch,
                          uint32_t* counters, int32_t* status, cudaStream_t st) {
    const int cols = gemv_allreduce_cols(N);
    if (cols == 0)
        return fail(SK_ERR_UNSUPPORTED, "sk_gemv_allreduce: %d output columns need more than %d CTAs of %d columns "
                                        "(every CTA must be resident)", N, sm_count(), GA_MAX_COLS);
    const int n_pad = (N + GA_MAX_COLS - 1) / GA_MAX_COLS * GA_MAX_COLS;
    const int grid = (N + cols - 1) / cols;
    if (B < 1 || B > GA_MAXB || B > max_batch)
        return fail(SK_ERR_UNSUPPORTED, "sk_gemv_allreduce: batch %d outside 1..%d (buffer holds %d)", B, GA_MAXB, max_batch);
    if (world < 1 || world > GA_MAX_WORLD || rank < 0 || rank >= world)
        return fail(SK_ERR_INVALID_ARGUMENT, "sk_gemv_allreduce: world %d / rank %d", world, rank);
    if (K % 8 != 0 || w_row_stride % 8 != 0)
        return fail(SK_ERR_MISALIGNED, "sk_gemv_allreduce: K and the weight row stride must be multiples of 8 elements");
    const size_t smem = (((size_t)B * (K + 8) * 2 + 15) & ~(size_t)15) +
                        (size_t)(GA_MAX_WORLD + 1) * GA_MAXB * GA_MAX_COLS * sizeof(float);   // + the warps' tiles of step 1
    if (smem > 200 * 1024)
        return fail(SK_ERR_UNSUPPORTED, "sk_gemv_allreduce: %d x %d activations do not fit shared memory", B, K);
#define SK_GA_LAUNCH(T)                                                                                     \
    do {                                                                                                    \
        auto kern = cols == 32 ? gemv_allreduce_kernel<T, 32> : gemv_allreduce_kernel<T, 64>;               \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) return fail(SK_ERR_CUDA, "gemv_allreduce_kernel smem attribute: %s", cudaGetErrorString(e)); \
        kern<<<grid, GA_THREADS, smem, st>>>((const T*)x, (const T*)W, w_row_stride, (const T*)res, (T*)out, B, N, K, \
                                             peer_base, world, rank, max_batch, n_pad, counters, status); \
        return check_launch("gemv_allreduce_kernel");                                                       \
    } while (0)
    if (dtype == SK_BF16) SK_GA_LAUNCH(__nv_bfloat16);
    if (dtype == SK_F16) SK_GA_LAUNCH(__half);
#undef SK_GA_LAUNCH
    return fail(SK_ERR_UNSUPPORTED, "sk_gemv_allreduce: bf16 or fp16 only");
}

}  // namespace sk
