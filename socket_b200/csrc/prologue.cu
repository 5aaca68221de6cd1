// Decode-step prologue: the KV-cache append of the new token (hash K, copy K/V, ||v||) and the
// query soft hash are independent of each other, so one launch runs both — the first CTAs of
// the grid do the append, the rest the soft hash — instead of two dependent launches.
#include "hash_body.cuh"
#include "soft_hash_body.cuh"

namespace sk {
namespace {

static_assert(HASH_THREADS == SH_THREADS, "both roles share one block size");

template <typename T, typename PT>
__global__ void __launch_bounds__(SH_THREADS, 2)
decode_prologue_kernel(const T* __restrict__ q, const T* __restrict__ k_new, const T* __restrict__ v_new,
                       const int64_t* __restrict__ input_pos, const PT* __restrict__ planes,
                       const float* __restrict__ protos_T, float inv_temperature, T* __restrict__ k_cache,
                       T* __restrict__ v_cache, uint8_t* __restrict__ codes, __half* __restrict__ v_norm,
                       int32_t* prefill_len, int32_t* status, float* __restrict__ lut, int B, int H,
                       int Hkv, int64_t Tcap, int L, int P, int R, int ht, int append_gx, int append_gy,
                       int sh_gx, uint2* __restrict__ lutq, float* __restrict__ qpar,
                       float* __restrict__ q_probs) {
    extern __shared__ __align__(16) float pro_smem[];
    pdl_launch_dependents();
    const int n_append = append_gx * append_gy;
    if ((int)blockIdx.x < n_append) {
        const int bx = blockIdx.x % append_gx, by = blockIdx.x / append_gx;
        kv_append_body<T, PT, 4>(k_new, v_new, input_pos, planes, k_cache, v_cache, codes, v_norm,
                                 prefill_len, status, B, 1, Hkv, Tcap, L, P, (int64_t)bx * HASH_ROWS,
                                 by * HASH_WARPS);
    } else {
        const int i = blockIdx.x - n_append;
        const int bx = i % sh_gx, g = i / sh_gx;
        soft_hash_body<T, PT>(q, planes, protos_T, inv_temperature, H, Hkv, 128, L, P, R, ht, g,
                              bx * (SH_WARPS / ht), q_probs, lut, pro_smem, lutq, qpar);
    }
}

}  // namespace

// Returns SK_ERR_UNSUPPORTED (without recording an error) when the fused form does not apply;
// the caller then uses the two separate launches.
int launch_decode_prologue(const void* q, const void* k_new, const void* v_new, int dtype,
                           const int64_t* input_pos, const void* planes, int plane_dtype,
                           const float* protos_T, float temperature, void* k_cache, void* v_cache,
                           uint8_t* codes, uint16_t* v_norm, int32_t* prefill_len, int32_t* status,
                           float* lut, int B, int H, int Hkv, int D, int64_t Tcap, int L, int P, int R,
                           cudaStream_t st, bool* launched, void* lutq, float* qpar, float* q_probs) {
    *launched = false;
    if (D != 128 || P > 16) return SK_OK;
    const int rep = H / Hkv;
    const int ht = lut_head_tile(rep);
    const int tiles = rep / ht;
    const int tpc = SH_WARPS / ht;
    const int append_gx = (B * Hkv + HASH_ROWS - 1) / HASH_ROWS;
    const int append_gy = (L + HASH_WARPS - 1) / HASH_WARPS;
    // (taking several table groups per CTA to fit the grid into one wave was tried: slower)
    const int sh_gx = (L + tpc - 1) / tpc;
    const int n_tiles = B * Hkv * tiles;
    const int sh_total = sh_gx * n_tiles;
    const size_t smem = soft_hash_smem_bytes(P, R, ht);
    if (smem > 200 * 1024) return SK_OK;
    const float inv_t = 1.0f / temperature;
    const unsigned grid = (unsigned)(append_gx * append_gy + sh_total);
#define SK_PRO_LAUNCH(T, PT)                                                                         \
    do {                                                                                             \
        auto kern = decode_prologue_kernel<T, PT>;                                                   \
        if (smem > 48 * 1024)                                                                        \
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
        kern<<<grid, SH_THREADS, smem, st>>>((const T*)q, (const T*)k_new, (const T*)v_new, input_pos, \
                                             (const PT*)planes, protos_T, inv_t, (T*)k_cache,        \
                                             (T*)v_cache, codes, (__half*)v_norm, prefill_len, status, \
                                             lut, B, H, Hkv, Tcap, L, P, R, ht, append_gx, append_gy, \
                                             sh_gx, (uint2*)lutq, qpar, q_probs);                    \
        *launched = true;                                                                            \
    } while (0)
    if (dtype == SK_F32 && plane_dtype == SK_F32) SK_PRO_LAUNCH(float, float);
    else if (dtype == SK_BF16 && plane_dtype == SK_BF16) SK_PRO_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (dtype == SK_F16 && plane_dtype == SK_F16) SK_PRO_LAUNCH(__half, __half);
    else if (dtype == SK_BF16 && plane_dtype == SK_F32) SK_PRO_LAUNCH(__nv_bfloat16, float);
    else if (dtype == SK_F16 && plane_dtype == SK_F32) SK_PRO_LAUNCH(__half, float);
    else return SK_OK;
#undef SK_PRO_LAUNCH
    return check_launch("decode_prologue_kernel");
}

}  // namespace sk
