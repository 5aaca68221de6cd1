// Decode-step front end: split the fused QKV projection of one new token into q / k / v and rotate
// the pairs of q and k by the position's rotary angles - one launch in place of the slice, cast,
// multiply, stack and cast kernels the tensor-level formulation takes per layer and token.
//
// Arithmetic follows the reference's apply_rotary_emb (GPT-FAST/model.py:626-637) operation by
// operation: pairs of consecutive elements, everything in fp32, products rounded before the
// add / subtract (no fused multiply-add), result cast to the activation type.
#include "common.cuh"

namespace sk {
namespace {

template <typename T, typename FT>
__global__ void __launch_bounds__(64)
rope_split_kernel(const T* __restrict__ qkv, const FT* __restrict__ freqs_cis, const int64_t* __restrict__ input_pos,
                  int H, int Hkv, int D, int64_t n_pos, T* __restrict__ q_out, T* __restrict__ k_out,
                  T* __restrict__ v_out, int32_t* status) {
    const int b = blockIdx.y, head = blockIdx.x;          // head over [q heads | k heads | v heads]
    const int n_heads = H + 2 * Hkv;
    const T* src = qkv + ((size_t)b * n_heads + head) * D;
    T* dst;
    bool rotate = true;
    if (head < H) dst = q_out + ((size_t)b * H + head) * D;
    else if (head < H + Hkv) dst = k_out + ((size_t)b * Hkv + (head - H)) * D;
    else {
        dst = v_out + ((size_t)b * Hkv + (head - H - Hkv)) * D;
        rotate = false;
    }
    const int64_t pos = input_pos[0];
    if (pos < 0 || pos >= n_pos) {                      // outside the table: flagged, nothing written
        if (threadIdx.x == 0 && status != nullptr) atomicOr(status, SK_DEV_POS_OUT_OF_RANGE);
        return;
    }
    for (int i = threadIdx.x; i < D / 2; i += blockDim.x) {
        const float x0 = to_f32(src[2 * i]), x1 = to_f32(src[2 * i + 1]);
        float y0 = x0, y1 = x1;
        if (rotate) {
            const float c = to_f32(freqs_cis[(pos * (D / 2) + i) * 2]);
            const float s = to_f32(freqs_cis[(pos * (D / 2) + i) * 2 + 1]);
            y0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
            y1 = __fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, s));
        }
        dst[2 * i] = from_f32<T>(y0);
        dst[2 * i + 1] = from_f32<T>(y1);
    }
}

}  // namespace

int launch_rope_split(const void* qkv, int dtype, const void* freqs_cis, int freq_dtype, const int64_t* input_pos,
                      int B, int H, int Hkv, int D, int64_t n_pos, void* q_out, void* k_out, void* v_out,
                      int32_t* status, cudaStream_t st) {
    dim3 grid((unsigned)(H + 2 * Hkv), (unsigned)B);
#define SK_ROPE_LAUNCH(T, FT)                                                                              \
    do {                                                                                                   \
        rope_split_kernel<T, FT><<<grid, 64, 0, st>>>((const T*)qkv, (const FT*)freqs_cis, input_pos, H, Hkv, D, \
                                                      n_pos, (T*)q_out, (T*)k_out, (T*)v_out, status);     \
        return check_launch("rope_split_kernel");                                                          \
    } while (0)
    if (dtype == SK_BF16 && freq_dtype == SK_BF16) SK_ROPE_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    if (dtype == SK_BF16 && freq_dtype == SK_F32) SK_ROPE_LAUNCH(__nv_bfloat16, float);
    if (dtype == SK_F16 && freq_dtype == SK_BF16) SK_ROPE_LAUNCH(__half, __nv_bfloat16);
    if (dtype == SK_F16 && freq_dtype == SK_F32) SK_ROPE_LAUNCH(__half, float);
    if (dtype == SK_F32 && freq_dtype == SK_BF16) SK_ROPE_LAUNCH(float, __nv_bfloat16);
    if (dtype == SK_F32 && freq_dtype == SK_F32) SK_ROPE_LAUNCH(float, float);
#undef SK_ROPE_LAUNCH
    return fail(SK_ERR_UNSUPPORTED, "sk_rope_split: unsupported dtype pair (%d,%d)", dtype, freq_dtype);
}

}  // namespace sk
