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
//      loads, several rows in flight per warp), with x_r
//      staged in shared memory, and reduces the products per warp;
//   2. it PUSHES its 32 x B partial sums (fp32) straight into every rank's receive buffer over
//      NVLink (peer stores, 128-byte rows), fences, and raises a flag in every rank's flag array;
//   3. it waits until the CTAs with the same index on all ranks have raised theirs - those are the
//      only producers of the 32 columns it owns - and adds the `world` partial rows, in rank order
//      (every rank gets the same bits), plus the residual, and writes `out`.
//
// No CTA waits for a CTA of its own grid, the grid never exceeds the number of SMs (all CTAs are
// resident), and every wait is bounded: when it runs out the kernel sets SK_DEV_WAIT_TIMEOUT and
// carries on with whatever has arrived, so a missing peer costs a wrong value, never a hang.
//
// Buffers: every rank allocates the same peer-mapped block [receive slots | flags] (host side:
// torch's symmetric memory; `peer_base[r]` is rank r's block as this GPU addresses it).  Receive
// slots are double-buffered by call parity: a rank can be at most one call ahead of a peer (it
// needs that peer's flag of the current call to finish it), so call n+2 never overwrites data a
// peer still reads for call n.  Flags hold call numbers and only grow; the per-CTA call counter
// lives in this GPU's own memory, so a CUDA graph can replay the call.
#include "common.cuh"

namespace sk {
namespace {

constexpr int GA_THREADS = 256;
constexpr int GA_WARPS = GA_THREADS / 32;
constexpr int GA_MAX_COLS = 64;                // output columns per CTA: 32, or 64 when 32 would need more CTAs than SMs
constexpr int GA_MAXB = 8;
constexpr int GA_MAX_WORLD = 8;
constexpr uint32_t GA_WAIT_LIMIT = 1u << 21;   // polls (with a short sleep each) before giving up: ~0.1 s

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float ld_volatile_f32(const float* p) {
    float v;
    asm volatile("ld.volatile.global.f32 %0, [%1];" : "=f"(v) : "l"(p));
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

template <typename T, int GA_COLS>
__global__ void __launch_bounds__(GA_THREADS, 1)
gemv_allreduce_kernel(const T* __restrict__ x, const T* __restrict__ W, int64_t w_row_stride,
                      const T* __restrict__ res, T* __restrict__ out, int B, int N, int K,
                      void* const* __restrict__ peer_base, int world, int rank, size_t flag_off,
                      int max_batch, int n_pad, uint32_t* __restrict__ counters, int32_t* status) {
    extern __shared__ __align__(16) char ga_smem[];
    T* x_s = reinterpret_cast<T*>(ga_smem);                                           // [B][K]
    float* y_s = reinterpret_cast<float*>(ga_smem + (((size_t)B * K * sizeof(T) + 15) & ~(size_t)15));   // [GA_MAXB][GA_COLS]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int blk = blockIdx.x, n0 = blk * GA_COLS;
    const uint32_t epoch = counters[blk] + 1u;            // this call's number for this CTA, the same on every rank
    const int slot = (int)(epoch & 1u);

    // ---- 1. activations to shared memory, then this CTA's rows of W
    for (int i = tid; i < B * K / 8; i += GA_THREADS)
        reinterpret_cast<uint4*>(x_s)[i] = reinterpret_cast<const uint4*>(x)[i];
    __syncthreads();
    constexpr int RPW = GA_COLS / GA_WARPS;               // rows per warp, walked side by side
    {
        const int nw = n0 + warp * RPW;
        float acc[RPW][GA_MAXB];
#pragma unroll
        for (int rr = 0; rr < RPW; ++rr)
#pragma unroll
            for (int b = 0; b < GA_MAXB; ++b) acc[rr][b] = 0.f;
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
                    unpack8(*reinterpret_cast<const uint4*>(x_s + (size_t)b * K + c * 8), (const T*)nullptr, xf);
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

    // ---- 2. push the partial rows to every rank (this one included), then raise the flags
    // receive layout of a rank: [slot][source rank][batch row][n_pad] fp32
    for (int idx = warp; idx < world * B; idx += GA_WARPS) {
        const int r = idx / B, b = idx - r * B;
        float* dst = reinterpret_cast<float*>(peer_base[r]) +
                     (((size_t)slot * world + rank) * max_batch + b) * n_pad + n0;
#pragma unroll
        for (int l = lane; l < GA_COLS; l += 32)
            if (n0 + l < N) dst[l] = y_s[b * GA_COLS + l];
    }
    __threadfence_system();
    __syncthreads();
    if (tid < world) {
        uint32_t* flag = reinterpret_cast<uint32_t*>(reinterpret_cast<char*>(peer_base[tid]) + flag_off) +
                         (size_t)blk * GA_MAX_WORLD + rank;
        st_release_sys(flag, epoch);
    }

    // ---- 3. wait for the same CTA of every rank, add the rows in rank order
    if (tid < world) {
        const uint32_t* flag = reinterpret_cast<const uint32_t*>(reinterpret_cast<const char*>(peer_base[rank]) + flag_off) +
                               (size_t)blk * GA_MAX_WORLD + tid;
        uint32_t it = 0;
        while ((int32_t)(ld_acquire_sys(flag) - epoch) < 0) {
            if (++it >= GA_WAIT_LIMIT) {
                if (status != nullptr) atomicOr(status, SK_DEV_WAIT_TIMEOUT);
                break;
            }
            __nanosleep(40);
        }
    }
    __syncthreads();
    const float* mine = reinterpret_cast<const float*>(peer_base[rank]);
    for (int idx = tid; idx < B * GA_COLS; idx += GA_THREADS) {
        const int b = idx / GA_COLS, l = idx - b * GA_COLS;
        const int n = n0 + l;
        if (n < N) {
            float s = res != nullptr ? to_f32(res[(size_t)b * N + n]) : 0.f;
            for (int r = 0; r < world; ++r)
                s += ld_volatile_f32(mine + (((size_t)slot * world + r) * max_batch + b) * n_pad + n);
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
size_t gemv_allreduce_flag_offset(int world, int max_batch, int n_pad) {
    return sk_up256((size_t)2 * world * max_batch * n_pad * sizeof(float));
}
size_t gemv_allreduce_buffer_bytes(int world, int max_batch, int N) {
    const int n_pad = (N + GA_MAX_COLS - 1) / GA_MAX_COLS * GA_MAX_COLS;
    const int grid = n_pad / 32;                                  // room for the finer split
    return gemv_allreduce_flag_offset(world, max_batch, n_pad) + sk_up256((size_t)grid * GA_MAX_WORLD * sizeof(uint32_t));
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
    const size_t smem = (((size_t)B * K * 2 + 15) & ~(size_t)15) + (size_t)GA_MAXB * GA_MAX_COLS * sizeof(float);
    if (smem > 200 * 1024)
        return fail(SK_ERR_UNSUPPORTED, "sk_gemv_allreduce: %d x %d activations do not fit shared memory", B, K);
    const size_t flag_off = gemv_allreduce_flag_offset(world, max_batch, n_pad);
#define SK_GA_LAUNCH(T)                                                                                     \
    do {                                                                                                    \
        auto kern = cols == 32 ? gemv_allreduce_kernel<T, 32> : gemv_allreduce_kernel<T, 64>;               \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) return fail(SK_ERR_CUDA, "gemv_allreduce_kernel smem attribute: %s", cudaGetErrorString(e)); \
        kern<<<grid, GA_THREADS, smem, st>>>((const T*)x, (const T*)W, w_row_stride, (const T*)res, (T*)out, B, N, K, \
                                             peer_base, world, rank, flag_off, max_batch, n_pad, counters, status); \
        return check_launch("gemv_allreduce_kernel");                                                       \
    } while (0)
    if (dtype == SK_BF16) SK_GA_LAUNCH(__nv_bfloat16);
    if (dtype == SK_F16) SK_GA_LAUNCH(__half);
#undef SK_GA_LAUNCH
    return fail(SK_ERR_UNSUPPORTED, "sk_gemv_allreduce: bf16 or fp16 only");
}

}  // namespace sk
