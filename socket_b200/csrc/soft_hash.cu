// Query soft hash: per (query head, table) a softmax over the R buckets, written both in
// the reference's [B,H,L,R] layout and as the scorer's lookup table.
//
// Scorer table layout: lut[g][r][l][j], g = (b*Hkv + kvh)*tiles + tile, j < ht query heads of
// that KV head.  One lookup (bucket r of table l) then yields the probabilities of all ht
// heads in one 4*ht-byte shared-memory word.
#include "soft_hash_body.cuh"

namespace sk {

int lut_head_tile(int rep) {
    if (rep % 4 == 0) return 4;
    if (rep % 2 == 0) return 2;
    return 1;
}

namespace {

constexpr int LP_TL = 8;  // tables per CTA in the layout-only kernel

template <typename QT, typename PT>
__global__ void __launch_bounds__(SH_THREADS)
soft_hash_kernel(const QT* __restrict__ q, const PT* __restrict__ planes,
                 const float* __restrict__ protos_T, float inv_temperature, int H, int Hkv, int D,
                 int L, int P, int R, int ht, float* __restrict__ q_probs, float* __restrict__ lut,
                 uint2* __restrict__ lutq, float* __restrict__ qpar) {
    extern __shared__ __align__(16) float sh_smem[];
    soft_hash_body<QT, PT>(q, planes, protos_T, inv_temperature, H, Hkv, D, L, P, R, ht, blockIdx.y,
                           blockIdx.x * (SH_WARPS / ht), q_probs, lut, sh_smem, lutq, qpar);
}

template <typename T>
__global__ void __launch_bounds__(SH_THREADS)
lut_from_probs_kernel(const T* __restrict__ q_probs, int H, int Hkv, int L, int R, int ht,
                      float* __restrict__ lut) {
    extern __shared__ __align__(16) float lp_smem[];
    const int rep = H / Hkv;
    const int tiles = rep / ht;
    const int g = blockIdx.y;
    const int tile = g % tiles;
    const int bk = g / tiles;
    const int b = bk / Hkv, kvh = bk % Hkv;
    const int h0 = kvh * rep + tile * ht;
    const int l0 = blockIdx.x * LP_TL;
    const int tl = min(LP_TL, L - l0);
    float* stage = lp_smem;  // [R][tl][ht]
    for (int i = threadIdx.x; i < ht * tl * R; i += SH_THREADS) {
        const int r = i % R;
        const int lt = (i / R) % tl;
        const int j = i / (R * tl);
        stage[((size_t)r * tl + lt) * ht + j] =
            to_f32(q_probs[(((size_t)b * H + h0 + j) * L + l0 + lt) * R + r]);
    }
    __syncthreads();
    float* lut_g = lut + (size_t)g * R * L * ht;
    const int seg = tl * ht;
    for (int i = threadIdx.x; i < R * seg; i += SH_THREADS) {
        const int r = i / seg, w = i - r * seg;
        lut_g[((size_t)r * L + l0) * ht + w] = stage[i];
    }
}

}  // namespace

int launch_soft_hash(const void* q, int q_dtype, const void* planes, int plane_dtype,
                     const float* protos_T, float temperature, int B, int H, int Hkv, int D, int L,
                     int P, int R, float* q_probs, float* lut, cudaStream_t st, void* lutq, float* qpar) {
    const int rep = H / Hkv;
    const int ht = lut_head_tile(rep);
    const int tiles = rep / ht;
    const int tpc = SH_WARPS / ht;
    if (P > 16) return fail(SK_ERR_UNSUPPORTED, "sk_soft_hash: P=%d > 16", P);
    dim3 grid((L + tpc - 1) / tpc, B * Hkv * tiles);
    const size_t smem = soft_hash_smem_bytes(P, R, ht);
    if (smem > 200 * 1024) return fail(SK_ERR_UNSUPPORTED, "sk_soft_hash: P*R too large (%d*%d)", P, R);
    const float inv_t = 1.0f / temperature;
#define SK_SH_LAUNCH(QT, PT)                                                                      \
    do {                                                                                          \
        auto kern = soft_hash_kernel<QT, PT>;                                                     \
        if (smem > 48 * 1024)                                                                     \
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
        kern<<<grid, SH_THREADS, smem, st>>>((const QT*)q, (const PT*)planes, protos_T, inv_t, H, \
                                             Hkv, D, L, P, R, ht, q_probs, lut,                   \
                                             (uint2*)lutq, qpar);                                 \
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
    dim3 grid((L + LP_TL - 1) / LP_TL, B * Hkv * tiles);
    size_t smem = sizeof(float) * (size_t)R * LP_TL * ht;
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
