// Key hashing (sign-random-projection codes) and the KV-cache append.
//
// Exactness: every projection is accumulated in fp64.  For 16-bit inputs each product is
// exact in fp64 and so is the 128-term sum for any realistic dynamic range, hence the sign
// (the hash bit) is the sign of the true dot product and does not depend on the order of
// summation.
#include "hash_body.cuh"

namespace sk {
namespace {

// grid (row groups, table groups): a CTA hashes HASH_ROWS rows against HASH_WARPS tables.
template <typename KT, typename PT, int EPL>
__global__ void __launch_bounds__(HASH_THREADS)
hash_keys_kernel(const KT* __restrict__ keys, int64_t key_row_stride, const PT* __restrict__ planes,
                 int64_t N, int L, int P, void* codes, int code_bytes, int64_t code_row_stride) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int l = blockIdx.y * HASH_WARPS + warp;
    for (int64_t n0 = (int64_t)blockIdx.x * HASH_ROWS; n0 < N; n0 += (int64_t)gridDim.x * HASH_ROWS) {
        double kd[HASH_ROWS][EPL];
        void* code_ptr[HASH_ROWS];
#pragma unroll
        for (int r = 0; r < HASH_ROWS; ++r) {
            const int64_t n = n0 + r;
            if (n < N) {
                load_row_f64<KT, EPL>(keys + n * key_row_stride, lane, kd[r]);
                code_ptr[r] = static_cast<char*>(codes) + n * code_row_stride * code_bytes;
            } else {
#pragma unroll
                for (int i = 0; i < EPL; ++i) kd[r][i] = 0.0;
                code_ptr[r] = nullptr;
            }
        }
        if (l < L) hash_table_rows<PT, EPL>(kd, code_ptr, planes, l, P, code_bytes, lane);
    }
}

template <typename KT, typename PT, int EPL>
__global__ void __launch_bounds__(HASH_THREADS)
kv_append_kernel(const KT* __restrict__ k_new, const KT* __restrict__ v_new,
                 const int64_t* __restrict__ input_pos, const PT* __restrict__ planes,
                 KT* __restrict__ k_cache, KT* __restrict__ v_cache, uint8_t* __restrict__ codes,
                 __half* __restrict__ v_norm, int32_t* prefill_len, int32_t* status, int B, int S,
                 int Hkv, int64_t Tcap, int L, int P) {
    kv_append_body<KT, PT, EPL>(k_new, v_new, input_pos, planes, k_cache, v_cache, codes, v_norm,
                                prefill_len, status, B, S, Hkv, Tcap, L, P,
                                (int64_t)blockIdx.x * HASH_ROWS, blockIdx.y * HASH_WARPS);
}

// Bulk cache write without hashing (the tensor-core path hashes separately): one warp per new
// (b, s, kvh) row of 128 bf16; lanes 0-15 move the key, lanes 16-31 the value (16 bytes each)
// and accumulate ||v||^2 in fp64, so v_norm is the same number the fused append stores.
__global__ void __launch_bounds__(256)
kv_copy_kernel(const uint4* __restrict__ k_new, const uint4* __restrict__ v_new,
               const int64_t* __restrict__ input_pos, uint4* __restrict__ k_cache,
               uint4* __restrict__ v_cache, __half* __restrict__ v_norm, int32_t* prefill_len,
               int32_t* status, int64_t N, int S, int Hkv, int64_t Tcap) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    bool bad = false;
    int32_t max_len = 0;
    for (int64_t n = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); n < N; n += warps) {
        const int kvh = (int)(n % Hkv);
        const int s = (int)((n / Hkv) % S);
        const int64_t b = n / ((int64_t)Hkv * S);
        const int64_t pos = __ldg(input_pos + s);
        if (pos < 0 || pos >= Tcap) {
            bad = true;
            continue;
        }
        const int64_t row = (b * Hkv + kvh) * Tcap + pos;
        if (pos + 1 > max_len) max_len = (int32_t)(pos + 1);
        if (lane < 16) {
            k_cache[row * 16 + lane] = __ldg(k_new + n * 16 + lane);
        } else {
            const uint4 x = __ldg(v_new + n * 16 + (lane - 16));
            v_cache[row * 16 + (lane - 16)] = x;
            const uint32_t w[4] = {x.x, x.y, x.z, x.w};
            double ss = 0.0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const double lo = (double)__uint_as_float(w[i] << 16);
                const double hi = (double)__uint_as_float(w[i] & 0xffff0000u);
                ss = fma(lo, lo, ss);
                ss = fma(hi, hi, ss);
            }
#pragma unroll
            for (int o = 8; o >= 1; o >>= 1) ss += __shfl_xor_sync(0xffff0000u, ss, o);
            if (lane == 16) v_norm[row] = __float2half_rn((float)sqrt(ss));
        }
    }
    if (lane == 0) {
        if (bad && status != nullptr) atomicOr(status, SK_DEV_POS_OUT_OF_RANGE);
        if (max_len > 0) atomicMax(prefill_len, max_len);
    }
}

template <typename KT, typename PT>
int hash_keys_dispatch(const void* keys, int64_t krs, const void* planes, int64_t N, int D, int L,
                       int P, void* codes, int cb, int64_t crs, cudaStream_t st) {
    int64_t groups = (N + HASH_ROWS - 1) / HASH_ROWS;
    dim3 grid((unsigned)(groups < sm_count() * 8 ? groups : sm_count() * 8), (unsigned)((L + HASH_WARPS - 1) / HASH_WARPS));
    if (D == 128)
        hash_keys_kernel<KT, PT, 4><<<grid, HASH_THREADS, 0, st>>>(
            (const KT*)keys, krs, (const PT*)planes, N, L, P, codes, cb, crs);
    else if (D == 64)
        hash_keys_kernel<KT, PT, 2><<<grid, HASH_THREADS, 0, st>>>(
            (const KT*)keys, krs, (const PT*)planes, N, L, P, codes, cb, crs);
    else
        return fail(SK_ERR_UNSUPPORTED, "sk_hash_keys: head_dim %d not supported (64 or 128)", D);
    return check_launch("hash_keys_kernel");
}

template <typename KT, typename PT>
int kv_append_dispatch(const void* k_new, const void* v_new, const int64_t* pos, const void* planes,
                       void* kc, void* vc, uint8_t* codes, uint16_t* vn, int32_t* plen,
                       int32_t* status, int B, int S, int Hkv, int D, int64_t Tcap, int L, int P,
                       cudaStream_t st) {
    const int64_t N = (int64_t)B * S * Hkv;
    const int64_t gx = (N + HASH_ROWS - 1) / HASH_ROWS;
    if (gx > 0x7fffffff) return fail(SK_ERR_UNSUPPORTED, "sk_kv_append: too many rows");
    dim3 grid((unsigned)gx, (unsigned)((L + HASH_WARPS - 1) / HASH_WARPS));
    if (D == 128)
        kv_append_kernel<KT, PT, 4><<<grid, HASH_THREADS, 0, st>>>(
            (const KT*)k_new, (const KT*)v_new, pos, (const PT*)planes, (KT*)kc, (KT*)vc, codes,
            (__half*)vn, plen, status, B, S, Hkv, Tcap, L, P);
    else
        return fail(SK_ERR_UNSUPPORTED, "sk_kv_append: head_dim %d not supported (128)", D);
    return check_launch("kv_append_kernel");
}

}  // namespace

#define SK_DISPATCH_KP(kdt, pdt, CALL)                                                       \
    do {                                                                                     \
        if (kdt == SK_F32 && pdt == SK_F32) { using KT = float; using PT = float; CALL; }    \
        else if (kdt == SK_BF16 && pdt == SK_BF16) { using KT = __nv_bfloat16; using PT = __nv_bfloat16; CALL; } \
        else if (kdt == SK_F16 && pdt == SK_F16) { using KT = __half; using PT = __half; CALL; } \
        else if (kdt == SK_BF16 && pdt == SK_F32) { using KT = __nv_bfloat16; using PT = float; CALL; } \
        else if (kdt == SK_F16 && pdt == SK_F32) { using KT = __half; using PT = float; CALL; } \
        else return fail(SK_ERR_UNSUPPORTED, "unsupported key/plane dtype pair (%d,%d)", kdt, pdt); \
    } while (0)

int launch_hash_keys(const void* keys, int key_dtype, int64_t key_row_stride, const void* planes,
                     int plane_dtype, int64_t N, int D, int L, int P, void* codes, int code_bytes,
                     int64_t code_row_stride, cudaStream_t st) {
    if (N == 0) return SK_OK;
    SK_DISPATCH_KP(key_dtype, plane_dtype,
                   return (hash_keys_dispatch<KT, PT>(keys, key_row_stride, planes, N, D, L, P, codes,
                                                      code_bytes, code_row_stride, st)));
}

int launch_kv_append(const void* k_new, const void* v_new, int kv_dtype, const int64_t* input_pos,
                     const void* planes, int plane_dtype, void* k_cache, void* v_cache,
                     uint8_t* codes, uint16_t* v_norm, int32_t* prefill_len, int32_t* status,
                     int B, int S, int Hkv, int D, int64_t Tcap, int L, int P, cudaStream_t st) {
    if ((int64_t)B * S * Hkv == 0) return SK_OK;
    SK_DISPATCH_KP(kv_dtype, plane_dtype,
                   return (kv_append_dispatch<KT, PT>(k_new, v_new, input_pos, planes, k_cache, v_cache,
                                                      codes, v_norm, prefill_len, status, B, S, Hkv,
                                                      D, Tcap, L, P, st)));
}

// K/V copy, ||v|| and prefill_len of S new tokens without hashing (the codes are written by the
// tensor-core hashing path): the append kernel with zero tables.
int launch_kv_copy(const void* k_new, const void* v_new, int kv_dtype, const int64_t* input_pos, void* k_cache,
                   void* v_cache, uint16_t* v_norm, int32_t* prefill_len, int32_t* status, int B, int S,
                   int Hkv, int D, int64_t Tcap, cudaStream_t st) {
    const int64_t N = (int64_t)B * S * Hkv;
    if (N == 0) return SK_OK;
    if (kv_dtype != SK_BF16 || D != 128) return fail(SK_ERR_UNSUPPORTED, "kv copy: bf16 and head_dim 128 only");
    if ((((uintptr_t)k_new | (uintptr_t)v_new | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) != 0)
        return fail(SK_ERR_MISALIGNED, "kv copy: K/V pointers must be 16-byte aligned");
    int64_t gx = (N + 7) / 8;
    if (gx > sm_count() * 16) gx = sm_count() * 16;
    kv_copy_kernel<<<(unsigned)gx, 256, 0, st>>>((const uint4*)k_new, (const uint4*)v_new, input_pos, (uint4*)k_cache,
                                                 (uint4*)v_cache, (__half*)v_norm, prefill_len, status, N, S, Hkv,
                                                 Tcap);
    return check_launch("kv_copy_kernel");
}

}  // namespace sk
