// Query soft hash: per (query head, table) a softmax over the R buckets, written both in
// the reference's [B,H,L,R] layout and as the scorer's lookup table.
//
// Scorer table layout: lut[g][r][l][j], g = (b*Hkv + kvh)*tiles + tile, j < ht query heads of
// that KV head.  One lookup (bucket r of table l) then yields the probabilities of all ht
// heads in one 4*ht-byte shared-memory word.
#include "common.cuh"

namespace sk {

int lut_head_tile(int rep) {
    if (rep % 4 == 0) return 4;
    if (rep % 2 == 0) return 2;
    return 1;
}

namespace {

constexpr int SH_THREADS = 256;
constexpr int SH_WARPS = SH_THREADS / 32;
constexpr int SH_TL = 8;  // tables per CTA

__device__ __forceinline__ float warp_sum_f(float x) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) x += __shfl_xor_sync(FULL, x, o);
    return x;
}
__device__ __forceinline__ float warp_max_f(float x) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) x = fmaxf(x, __shfl_xor_sync(FULL, x, o));
    return x;
}

// stage[r][lt][j] (R * tl * ht floats) -> lut rows; every warp store covers one contiguous
// run of tl*ht floats.
__device__ __forceinline__ void write_lut_tile(const float* stage, float* lut_g, int R, int L, int l0,
                                               int tl, int ht) {
    const int seg = tl * ht;
    for (int i = threadIdx.x; i < R * seg; i += blockDim.x) {
        const int r = i / seg, w = i - r * seg;
        lut_g[((size_t)r * L + l0) * ht + w] = stage[i];
    }
}

template <typename QT, typename PT>
__global__ void __launch_bounds__(SH_THREADS)
soft_hash_kernel(const QT* __restrict__ q, const PT* __restrict__ planes,
                 const float* __restrict__ protos_T, float inv_temperature, int H, int Hkv, int D,
                 int L, int P, int R, int ht, float* __restrict__ q_probs, float* __restrict__ lut) {
    extern __shared__ float smem[];
    const int rep = H / Hkv;
    const int tiles = rep / ht;
    const int g = blockIdx.y;                 // (b*Hkv + kvh)*tiles + tile
    const int tile = g % tiles;
    const int bk = g / tiles;                 // b*Hkv + kvh
    const int b = bk / Hkv, kvh = bk % Hkv;
    const int h0 = kvh * rep + tile * ht;     // first query head of this tile
    const int l0 = blockIdx.x * SH_TL;
    const int tl = min(SH_TL, L - l0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    float* q_s = smem;                        // [ht][D]
    float* t_s = q_s + ht * D;                // [ht][SH_TL][P]
    float* pr_s = t_s + ht * SH_TL * P;       // [P][R]
    float* stage = pr_s + P * R;              // [R][tl][ht]

    for (int i = threadIdx.x; i < ht * D; i += SH_THREADS) {
        const int j = i / D, d = i - j * D;
        q_s[i] = to_f32(q[((size_t)b * H + h0 + j) * D + d]);
    }
    for (int i = threadIdx.x; i < P * R; i += SH_THREADS) pr_s[i] = protos_T[i];
    __syncthreads();

    const float inv_sqrt_d = 1.0f / fmaxf(sqrtf((float)D), 1e-6f);
    // projections: one warp per (head, table, plane)
    for (int i = warp; i < ht * tl * P; i += SH_WARPS) {
        const int p = i % P;
        const int lt = (i / P) % tl;
        const int j = i / (P * tl);
        const PT* pl = planes + ((size_t)(l0 + lt) * P + p) * D;
        float s = 0.f;
        for (int d = lane; d < D; d += 32) s = fmaf(q_s[j * D + d], to_f32(pl[d]), s);
        s = warp_sum_f(s);
        if (lane == 0) t_s[(j * SH_TL + lt) * P + p] = tanhf(s) * inv_sqrt_d;
    }
    __syncthreads();

    // softmax rows: one warp per (head, table)
    for (int i = warp; i < ht * tl; i += SH_WARPS) {
        const int lt = i % tl, j = i / tl;
        const float* t = t_s + (j * SH_TL + lt) * P;
        float mx = -INFINITY;
        for (int r = lane; r < R; r += 32) {
            float lg = 0.f;
            for (int p = 0; p < P; ++p) lg = fmaf(t[p], pr_s[p * R + r], lg);
            mx = fmaxf(mx, lg * inv_temperature);
        }
        mx = warp_max_f(mx);
        float se = 0.f;
        for (int r = lane; r < R; r += 32) {
            float lg = 0.f;
            for (int p = 0; p < P; ++p) lg = fmaf(t[p], pr_s[p * R + r], lg);
            se += expf(lg * inv_temperature - mx);
        }
        se = warp_sum_f(se);
        float* qp_row = q_probs ? q_probs + (((size_t)b * H + h0 + j) * L + l0 + lt) * R : nullptr;
        for (int r = lane; r < R; r += 32) {
            float lg = 0.f;
            for (int p = 0; p < P; ++p) lg = fmaf(t[p], pr_s[p * R + r], lg);
            const float pr = expf(lg * inv_temperature - mx) / se;
            if (qp_row) qp_row[r] = pr;
            stage[((size_t)r * tl + lt) * ht + j] = pr;
        }
    }
    if (lut == nullptr) return;
    __syncthreads();
    write_lut_tile(stage, lut + (size_t)g * R * L * ht, R, L, l0, tl, ht);
}

template <typename T>
__global__ void __launch_bounds__(SH_THREADS)
lut_from_probs_kernel(const T* __restrict__ q_probs, int H, int Hkv, int L, int R, int ht,
                      float* __restrict__ lut) {
    extern __shared__ float smem[];
    const int rep = H / Hkv;
    const int tiles = rep / ht;
    const int g = blockIdx.y;
    const int tile = g % tiles;
    const int bk = g / tiles;
    const int b = bk / Hkv, kvh = bk % Hkv;
    const int h0 = kvh * rep + tile * ht;
    const int l0 = blockIdx.x * SH_TL;
    const int tl = min(SH_TL, L - l0);
    float* stage = smem;  // [R][tl][ht]
    for (int i = threadIdx.x; i < ht * tl * R; i += SH_THREADS) {
        const int r = i % R;
        const int lt = (i / R) % tl;
        const int j = i / (R * tl);
        stage[((size_t)r * tl + lt) * ht + j] =
            to_f32(q_probs[(((size_t)b * H + h0 + j) * L + l0 + lt) * R + r]);
    }
    __syncthreads();
    write_lut_tile(stage, lut + (size_t)g * R * L * ht, R, L, l0, tl, ht);
}

}  // namespace

int launch_soft_hash(const void* q, int q_dtype, const void* planes, int plane_dtype,
                     const float* protos_T, float temperature, int B, int H, int Hkv, int D, int L,
                     int P, int R, float* q_probs, float* lut, cudaStream_t st) {
    const int rep = H / Hkv;
    const int ht = lut_head_tile(rep);
    const int tiles = rep / ht;
    dim3 grid((L + SH_TL - 1) / SH_TL, B * Hkv * tiles);
    size_t smem = sizeof(float) * ((size_t)ht * D + (size_t)ht * SH_TL * P + (size_t)P * R +
                                   (size_t)R * SH_TL * ht);
    if (smem > 200 * 1024) return fail(SK_ERR_UNSUPPORTED, "sk_soft_hash: P*R too large (%d*%d)", P, R);
    const float inv_t = 1.0f / temperature;
#define SK_SH_LAUNCH(QT, PT)                                                                      \
    do {                                                                                          \
        auto kern = soft_hash_kernel<QT, PT>;                                                     \
        if (smem > 48 * 1024)                                                                     \
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
        kern<<<grid, SH_THREADS, smem, st>>>((const QT*)q, (const PT*)planes, protos_T, inv_t, H, \
                                             Hkv, D, L, P, R, ht, q_probs, lut);                  \
    } while (0)
    if (q_dtype == SK_F32 && plane_dtype == SK_F32) SK_SH_LAUNCH(float, float);
    else if (q_dtype == SK_BF16 && plane_dtype == SK_BF16) SK_SH_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (q_dtype == SK_F16 && plane_dtype == SK_F16) SK_SH_LAUNCH(__half, __half);
    else if (q_dtype == SK_BF16 && plane_dtype == SK_F32) SK_SH_LAUNCH(__nv_bfloat16, float);
    else if (q_dtype == SK_F16 && plane_dtype == SK_F32) SK_SH_LAUNCH(__half, float);
    else return fail(SK_ERR_UNSUPPORTED, "sk_soft_hash: unsupported q/plane dtype pair (%d,%d)", q_dtype, plane_dtype);
#undef SK_SH_LAUNCH
    return check_launch("soft_hash_kernel");
}

int launch_lut_from_probs(const void* q_probs, int dtype, int B, int H, int Hkv, int L, int R,
                          float* lut, cudaStream_t st) {
    const int rep = H / Hkv;
    const int ht = lut_head_tile(rep);
    const int tiles = rep / ht;
    dim3 grid((L + SH_TL - 1) / SH_TL, B * Hkv * tiles);
    size_t smem = sizeof(float) * (size_t)R * SH_TL * ht;
    if (smem > 200 * 1024) return fail(SK_ERR_UNSUPPORTED, "sk_lut_from_probs: R too large (%d)", R);
#define SK_LP_LAUNCH(T)                                                                          \
    do {                                                                                         \
        auto kern = lut_from_probs_kernel<T>;                                                    \
        if (smem > 48 * 1024)                                                                    \
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        kern<<<grid, SH_THREADS, smem, st>>>((const T*)q_probs, H, Hkv, L, R, ht, lut);          \
    } while (0)
    if (dtype == SK_F32) SK_LP_LAUNCH(float);
    else if (dtype == SK_BF16) SK_LP_LAUNCH(__nv_bfloat16);
    else if (dtype == SK_F16) SK_LP_LAUNCH(__half);
    else return fail(SK_ERR_UNSUPPORTED, "sk_lut_from_probs: unsupported dtype %d", dtype);
#undef SK_LP_LAUNCH
    return check_launch("lut_from_probs_kernel");
}

}  // namespace sk
