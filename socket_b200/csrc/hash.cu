// Key hashing (sign-random-projection codes) and the fused KV-cache append.
//
// Exactness: every projection is accumulated in fp64.  For 16-bit inputs each product is
// exact in fp64 and so is the 128-term sum for any realistic dynamic range, hence the sign
// (the hash bit) is the sign of the true dot product and does not depend on the order of
// summation.  This kernel serves the decode-time append (a handful of rows) and is the
// reference path for bulk hashing.
#include "common.cuh"

namespace sk {
namespace {

constexpr int HASH_THREADS = 256;
constexpr int HASH_WARPS = HASH_THREADS / 32;
constexpr int HASH_ROWS = 4;  // rows hashed together by one CTA

template <typename T, int EPL>
__device__ __forceinline__ void load_row(const T* row, int lane, double (&dst)[EPL]) {
#pragma unroll
    for (int i = 0; i < EPL; ++i) dst[i] = (double)to_f32(row[lane * EPL + i]);
}

// Sum of 32 per-lane values for each of 32 slots; lane j ends up with the total of slot j.
__device__ __forceinline__ double transpose_reduce32(double (&v)[32], int lane) {
#pragma unroll
    for (int step = 16; step >= 1; step >>= 1) {
        const bool upper = (lane & step) != 0;
#pragma unroll
        for (int i = 0; i < step; ++i) {
            const double send = upper ? v[i] : v[i + step];
            const double keep = upper ? v[i + step] : v[i];
            v[i] = keep + __shfl_xor_sync(FULL, send, step);
        }
    }
    return v[0];
}

__device__ __forceinline__ double warp_sum(double x) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) x += __shfl_xor_sync(FULL, x, o);
    return x;
}

struct RowSet {
    const void* key[HASH_ROWS];   // nullptr = row absent
    void* code[HASH_ROWS];        // where this row's L codes go
};

// Hash up to HASH_ROWS rows against all L tables.  Warps split the tables.
template <typename KT, typename PT, int EPL>
__device__ __forceinline__ void hash_row_set(const RowSet& rs, const PT* __restrict__ planes, int L,
                                             int P, int code_bytes, int warp, int lane) {
    constexpr int D = EPL * 32;
    double kd[HASH_ROWS][EPL];
#pragma unroll
    for (int r = 0; r < HASH_ROWS; ++r) {
        if (rs.key[r] != nullptr) {
            load_row<KT, EPL>(static_cast<const KT*>(rs.key[r]), lane, kd[r]);
        } else {
#pragma unroll
            for (int i = 0; i < EPL; ++i) kd[r][i] = 0.0;
        }
    }
    for (int l = warp; l < L; l += HASH_WARPS) {
        const PT* pl = planes + (size_t)l * P * D;
        if (P == 8) {
            // slot j = r*8 + (7-p): after the ballot, byte r of the mask is row r's code
            double v[32];
#pragma unroll
            for (int p = 0; p < 8; ++p) {
                double pd[EPL];
                load_row<PT, EPL>(pl + (size_t)p * D, lane, pd);
#pragma unroll
                for (int r = 0; r < HASH_ROWS; ++r) {
                    double s = 0.0;
#pragma unroll
                    for (int i = 0; i < EPL; ++i) s = fma(kd[r][i], pd[i], s);
                    v[r * 8 + (7 - p)] = s;
                }
            }
            const double tot = transpose_reduce32(v, lane);
            const unsigned bits = __ballot_sync(FULL, tot >= 0.0);
            if (lane < HASH_ROWS && rs.code[lane] != nullptr) {
                const unsigned code = (bits >> (8 * lane)) & 0xffu;
                if (code_bytes == 1) static_cast<uint8_t*>(rs.code[lane])[l] = (uint8_t)code;
                else static_cast<int16_t*>(rs.code[lane])[l] = (int16_t)code;
            }
        } else {
            unsigned code[HASH_ROWS];
#pragma unroll
            for (int r = 0; r < HASH_ROWS; ++r) code[r] = 0;
            for (int p = 0; p < P; ++p) {
                double pd[EPL];
                load_row<PT, EPL>(pl + (size_t)p * D, lane, pd);
#pragma unroll
                for (int r = 0; r < HASH_ROWS; ++r) {
                    double s = 0.0;
#pragma unroll
                    for (int i = 0; i < EPL; ++i) s = fma(kd[r][i], pd[i], s);
                    s = warp_sum(s);
                    code[r] = code[r] * 2u + (s >= 0.0 ? 1u : 0u);
                }
            }
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < HASH_ROWS; ++r) {
                    if (rs.code[r] == nullptr) continue;
                    if (code_bytes == 1) static_cast<uint8_t*>(rs.code[r])[l] = (uint8_t)code[r];
                    else static_cast<int16_t*>(rs.code[r])[l] = (int16_t)code[r];
                }
            }
        }
    }
}

template <typename KT, typename PT, int EPL>
__global__ void __launch_bounds__(HASH_THREADS)
hash_keys_kernel(const KT* __restrict__ keys, int64_t key_row_stride, const PT* __restrict__ planes,
                 int64_t N, int L, int P, void* codes, int code_bytes, int64_t code_row_stride) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int64_t n0 = (int64_t)blockIdx.x * HASH_ROWS; n0 < N; n0 += (int64_t)gridDim.x * HASH_ROWS) {
        RowSet rs;
#pragma unroll
        for (int r = 0; r < HASH_ROWS; ++r) {
            const int64_t n = n0 + r;
            const bool ok = n < N;
            rs.key[r] = ok ? keys + n * key_row_stride : nullptr;
            rs.code[r] = ok ? static_cast<char*>(codes) + n * code_row_stride * code_bytes : nullptr;
        }
        hash_row_set<KT, PT, EPL>(rs, planes, L, P, code_bytes, warp, lane);
    }
}

// One CTA per HASH_ROWS new (b, s, kvh) rows: hash K, copy K and V into the cache, store
// ||v|| as fp16, advance prefill_len.
template <typename KT, typename PT, int EPL>
__global__ void __launch_bounds__(HASH_THREADS)
kv_append_kernel(const KT* __restrict__ k_new, const KT* __restrict__ v_new,
                 const int64_t* __restrict__ input_pos, const PT* __restrict__ planes,
                 KT* __restrict__ k_cache, KT* __restrict__ v_cache, uint8_t* __restrict__ codes,
                 __half* __restrict__ v_norm, int32_t* prefill_len, int32_t* status, int B, int S,
                 int Hkv, int64_t Tcap, int L, int P) {
    constexpr int D = EPL * 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t N = (int64_t)B * S * Hkv;
    const int64_t n0 = (int64_t)blockIdx.x * HASH_ROWS;
    RowSet rs;
    int64_t cache_row[HASH_ROWS];
#pragma unroll
    for (int r = 0; r < HASH_ROWS; ++r) {
        const int64_t n = n0 + r;
        rs.key[r] = nullptr;
        rs.code[r] = nullptr;
        cache_row[r] = -1;
        if (n < N) {
            const int kvh = (int)(n % Hkv);
            const int s = (int)((n / Hkv) % S);
            const int b = (int)(n / ((int64_t)Hkv * S));
            const int64_t pos = input_pos[s];
            if (pos < 0 || pos >= Tcap) {
                if (status != nullptr && threadIdx.x == 0) atomicOr(status, SK_DEV_POS_OUT_OF_RANGE);
            } else {
                cache_row[r] = ((int64_t)b * Hkv + kvh) * Tcap + pos;
                rs.key[r] = k_new + n * D;
                rs.code[r] = codes + cache_row[r] * L;
                if (threadIdx.x == 0 && kvh == 0 && b == 0) atomicMax(prefill_len, (int32_t)(pos + 1));
            }
        }
    }
    hash_row_set<KT, PT, EPL>(rs, planes, L, P, 1, warp, lane);
    if (warp < HASH_ROWS && cache_row[warp] >= 0) {
        const int64_t n = n0 + warp;
        const KT* ks = k_new + n * D;
        const KT* vs = v_new + n * D;
        KT* kd = k_cache + cache_row[warp] * D;
        KT* vd = v_cache + cache_row[warp] * D;
        double ss = 0.0;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const int d = lane * EPL + i;
            kd[d] = ks[d];
            const KT x = vs[d];
            vd[d] = x;
            const double xf = (double)to_f32(x);
            ss = fma(xf, xf, ss);
        }
        ss = warp_sum(ss);
        if (lane == 0) v_norm[cache_row[warp]] = __float2half_rn((float)sqrt(ss));
    }
}

template <typename KT, typename PT>
int hash_keys_dispatch(const void* keys, int64_t krs, const void* planes, int64_t N, int D, int L,
                       int P, void* codes, int cb, int64_t crs, cudaStream_t st) {
    int64_t groups = (N + HASH_ROWS - 1) / HASH_ROWS;
    int grid = (int)(groups < 148 * 8 ? groups : 148 * 8);
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
    const int64_t grid = (N + HASH_ROWS - 1) / HASH_ROWS;
    if (grid > 0x7fffffff) return fail(SK_ERR_UNSUPPORTED, "sk_kv_append: too many rows");
    if (D == 128)
        kv_append_kernel<KT, PT, 4><<<(int)grid, HASH_THREADS, 0, st>>>(
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

}  // namespace sk
