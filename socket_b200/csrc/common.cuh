// Shared device helpers and host-side launcher declarations (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/socket_b200.h"

namespace sk {

constexpr unsigned FULL = 0xffffffffu;

// ---------------------------------------------------------------- host error plumbing
int fail(int status, const char* fmt, ...);       // records a thread-local message
int check_launch(const char* what);               // cudaGetLastError -> SK_ERR_CUDA

// ---------------------------------------------------------------- element access
template <int DT> struct Elem;
template <> struct Elem<SK_F32> { using type = float; };
template <> struct Elem<SK_BF16> { using type = __nv_bfloat16; };
template <> struct Elem<SK_F16> { using type = __half; };

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) {
    return __float2bfloat16_rn(x);
}
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

// Order-preserving map float -> uint32 (larger float <=> larger key); -0 folds onto +0.
__device__ __forceinline__ uint32_t order_key(float f) {
    uint32_t u = __float_as_uint(f);
    if (u == 0x80000000u) u = 0u;
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ int effective_len(int64_t T, const int32_t* T_dev) {
    int64_t t = T;
    if (T_dev != nullptr) {
        int64_t d = (int64_t)(*T_dev);
        t = d < t ? d : t;
    }
    return t < 0 ? 0 : (int)t;
}

// ---------------------------------------------------------------- launchers (one per .cu)
int launch_hash_keys(const void* keys, int key_dtype, int64_t key_row_stride, const void* planes,
                     int plane_dtype, int64_t N, int D, int L, int P, void* codes, int code_bytes,
                     int64_t code_row_stride, cudaStream_t st);
int launch_kv_append(const void* k_new, const void* v_new, int kv_dtype, const int64_t* input_pos,
                     const void* planes, int plane_dtype, void* k_cache, void* v_cache,
                     uint8_t* codes, uint16_t* v_norm, int32_t* prefill_len, int32_t* status,
                     int B, int S, int Hkv, int D, int64_t Tcap, int L, int P, cudaStream_t st);
int launch_soft_hash(const void* q, int q_dtype, const void* planes, int plane_dtype,
                     const float* protos_T, float temperature, int B, int H, int Hkv, int D, int L,
                     int P, int R, float* q_probs, float* lut, cudaStream_t st);
int launch_lut_from_probs(const void* q_probs, int dtype, int B, int H, int Hkv, int L, int R,
                          float* lut, cudaStream_t st);
int launch_score(const float* lut, const uint8_t* codes, const uint16_t* v_norm,
                 const uint8_t* allowed, int B, int H, int Hkv, int L, int R, int64_t T,
                 const int32_t* T_dev, int64_t Tcap, float* scores, int64_t score_row_stride,
                 int32_t* status, cudaStream_t st);
int launch_score_compat(const float* q_probs, const int16_t* key_buckets, const uint8_t* allowed,
                        const float* v_hist, float* out, int B, int H, int L, int R, int64_t T,
                        cudaStream_t st);
int launch_select_list(const float* scores, int64_t score_row_stride, const uint8_t* allowed,
                       int64_t rows, int64_t T, const int32_t* T_dev, int64_t M, int sink,
                       int window, int sorted, int32_t* list, int64_t list_row_stride,
                       int32_t* list_len, int32_t* status, cudaStream_t st);
size_t sparse_decode_workspace_bytes(int B, int H, int D, int64_t max_list_len);
int launch_sparse_decode(const void* q, int q_dtype, const void* k_cache, const void* v_cache,
                         int kv_dtype, int64_t kv_batch_stride, int64_t kv_head_stride,
                         int64_t kv_row_stride, const int32_t* list, int64_t list_row_stride,
                         const int32_t* list_len, int64_t max_list_len, void* out, int B, int H,
                         int Hkv, int D, int64_t T, const int32_t* T_dev, void* workspace,
                         size_t workspace_bytes, int32_t* status, cudaStream_t st);

int lut_head_tile(int rep);
int launch_decode_prologue(const void* q, const void* k_new, const void* v_new, int dtype,
                           const int64_t* input_pos, const void* planes, int plane_dtype,
                           const float* protos_T, float temperature, void* k_cache, void* v_cache,
                           uint8_t* codes, uint16_t* v_norm, int32_t* prefill_len, int32_t* status,
                           float* lut, int B, int H, int Hkv, int D, int64_t Tcap, int L, int P, int R,
                           cudaStream_t st, bool* launched);

}  // namespace sk
