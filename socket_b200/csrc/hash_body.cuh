// Device code shared by the hashing kernels: exact (fp64) sign-random-projection codes of up
// to four rows at a time, and the write of one new token into the KV cache.
#pragma once
#include "common.cuh"

namespace sk {

constexpr int HASH_THREADS = 256;
constexpr int HASH_WARPS = HASH_THREADS / 32;
constexpr int HASH_ROWS = 4;  // rows hashed together by one CTA

template <typename T, int EPL>
__device__ __forceinline__ void load_row_f64(const T* row, int lane, double (&dst)[EPL]) {
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

__device__ __forceinline__ double warp_sum_f64(double x) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) x += __shfl_xor_sync(FULL, x, o);
    return x;
}

__device__ __forceinline__ void store_code(void* base, int code_bytes, int l, unsigned code) {
    if (code_bytes == 1) static_cast<uint8_t*>(base)[l] = (uint8_t)code;
    else static_cast<int16_t*>(base)[l] = (int16_t)code;
}

// The 8 planes of table `l`, EPL elements per lane each.
template <typename PT, int EPL>
__device__ __forceinline__ void load_planes8(const PT* __restrict__ planes, int l, int lane,
                                             double (&pd)[8][EPL]) {
    constexpr int D = EPL * 32;
    const PT* pl = planes + (size_t)l * 8 * D;
#pragma unroll
    for (int p = 0; p < 8; ++p) load_row_f64<PT, EPL>(pl + (size_t)p * D, lane, pd[p]);
}

// One warp, P == 8: codes of one table for HASH_ROWS rows; keys and planes are in registers.
// code_ptr[r] == nullptr marks an absent row.
template <int EPL>
__device__ __forceinline__ void hash_rows_planes8(const double (&kd)[HASH_ROWS][EPL],
                                                  const double (&pd)[8][EPL],
                                                  void* const (&code_ptr)[HASH_ROWS], int l,
                                                  int code_bytes, int lane) {
    // slot j = r*8 + (7-p): after the ballot, byte r of the mask is row r's code
    double v[32];
#pragma unroll
    for (int p = 0; p < 8; ++p) {
#pragma unroll
        for (int r = 0; r < HASH_ROWS; ++r) {
            double s = 0.0;
#pragma unroll
            for (int i = 0; i < EPL; ++i) s = fma(kd[r][i], pd[p][i], s);
            v[r * 8 + (7 - p)] = s;
        }
    }
    const double tot = transpose_reduce32(v, lane);
    const unsigned bits = __ballot_sync(FULL, tot >= 0.0);
#pragma unroll
    for (int r = 0; r < HASH_ROWS; ++r)
        if (lane == r && code_ptr[r] != nullptr) store_code(code_ptr[r], code_bytes, l, (bits >> (8 * r)) & 0xffu);
}

// One warp, any P <= 15: plane by plane.
template <typename PT, int EPL>
__device__ __forceinline__ void hash_rows_generic(const double (&kd)[HASH_ROWS][EPL],
                                                  void* const (&code_ptr)[HASH_ROWS],
                                                  const PT* __restrict__ planes, int l, int P,
                                                  int code_bytes, int lane) {
    constexpr int D = EPL * 32;
    const PT* pl = planes + (size_t)l * P * D;
    unsigned code[HASH_ROWS];
#pragma unroll
    for (int r = 0; r < HASH_ROWS; ++r) code[r] = 0;
    for (int p = 0; p < P; ++p) {
        double pd[EPL];
        load_row_f64<PT, EPL>(pl + (size_t)p * D, lane, pd);
#pragma unroll
        for (int r = 0; r < HASH_ROWS; ++r) {
            double s = 0.0;
#pragma unroll
            for (int i = 0; i < EPL; ++i) s = fma(kd[r][i], pd[i], s);
            s = warp_sum_f64(s);
            code[r] = code[r] * 2u + (s >= 0.0 ? 1u : 0u);
        }
    }
#pragma unroll
    for (int r = 0; r < HASH_ROWS; ++r)
        if (lane == 0 && code_ptr[r] != nullptr) store_code(code_ptr[r], code_bytes, l, code[r]);
}

// One warp: codes of table `l` for HASH_ROWS rows whose elements are already in registers.
template <typename PT, int EPL>
__device__ __forceinline__ void hash_table_rows(const double (&kd)[HASH_ROWS][EPL],
                                                void* const (&code_ptr)[HASH_ROWS],
                                                const PT* __restrict__ planes, int l, int P,
                                                int code_bytes, int lane) {
    if (P == 8) {
        double pd[8][EPL];
        load_planes8<PT, EPL>(planes, l, lane, pd);
        hash_rows_planes8<EPL>(kd, pd, code_ptr, l, code_bytes, lane);
    } else {
        hash_rows_generic<PT, EPL>(kd, code_ptr, planes, l, P, code_bytes, lane);
    }
}

// KV-cache append of HASH_ROWS new (b, s, kvh) rows starting at row `n0`: this CTA hashes
// them against tables [l0, l0 + HASH_WARPS) (one table per warp); the CTA with l0 == 0 also
// copies K and V, stores ||v|| as fp16 and advances prefill_len.
template <typename KT, typename PT, int EPL>
__device__ __forceinline__ void kv_append_body(
    const KT* __restrict__ k_new, const KT* __restrict__ v_new, const int64_t* __restrict__ input_pos,
    const PT* __restrict__ planes, KT* __restrict__ k_cache, KT* __restrict__ v_cache,
    uint8_t* __restrict__ codes, __half* __restrict__ v_norm, int32_t* prefill_len, int32_t* status,
    int B, int S, int Hkv, int64_t Tcap, int L, int P, int64_t n0, int l0) {
    constexpr int D = EPL * 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t N = (int64_t)B * S * Hkv;
    const int l = l0 + warp;
    // Every global load is issued before the first one is consumed, so the append costs one memory
    // round trip: the new K rows and this warp's V row (their addresses do not depend on
    // input_pos), the positions, and the planes.
    const bool fast = (P == 8) && (l < L);
    const bool mover = l0 == 0 && warp < HASH_ROWS && n0 + warp < N;      // warp r moves row r
    KT kraw[HASH_ROWS][EPL], vraw[EPL];
    int64_t posv[HASH_ROWS];
#pragma unroll
    for (int r = 0; r < HASH_ROWS; ++r) {
        const int64_t n = n0 + r;
        posv[r] = -1;
#pragma unroll
        for (int i = 0; i < EPL; ++i) kraw[r][i] = from_f32<KT>(0.f);
        if (n < N) {
#pragma unroll
            for (int i = 0; i < EPL; ++i) kraw[r][i] = k_new[n * D + lane * EPL + i];
            posv[r] = input_pos[(int)((n / Hkv) % S)];
        }
    }
#pragma unroll
    for (int i = 0; i < EPL; ++i) vraw[i] = mover ? v_new[(n0 + warp) * D + lane * EPL + i] : from_f32<KT>(0.f);
    double pd[8][EPL];
    if (fast) load_planes8<PT, EPL>(planes, l, lane, pd);

    double kd[HASH_ROWS][EPL];
    void* code_ptr[HASH_ROWS];
    int64_t cache_row[HASH_ROWS];
#pragma unroll
    for (int r = 0; r < HASH_ROWS; ++r) {
        const int64_t n = n0 + r;
        code_ptr[r] = nullptr;
        cache_row[r] = -1;
#pragma unroll
        for (int i = 0; i < EPL; ++i) kd[r][i] = 0.0;
        if (n < N) {
            const int kvh = (int)(n % Hkv);
            const int b = (int)(n / ((int64_t)Hkv * S));
            const int64_t pos = posv[r];
            if (pos < 0 || pos >= Tcap) {
                if (status != nullptr && threadIdx.x == 0 && l0 == 0) atomicOr(status, SK_DEV_POS_OUT_OF_RANGE);
            } else {
                cache_row[r] = ((int64_t)b * Hkv + kvh) * Tcap + pos;
                code_ptr[r] = codes + cache_row[r] * L;
#pragma unroll
                for (int i = 0; i < EPL; ++i) kd[r][i] = (double)to_f32(kraw[r][i]);
                if (threadIdx.x == 0 && l0 == 0 && kvh == 0 && b == 0) atomicMax(prefill_len, (int32_t)(pos + 1));
            }
        }
    }
    if (fast) hash_rows_planes8<EPL>(kd, pd, code_ptr, l, 1, lane);
    else if (l < L) hash_rows_generic<PT, EPL>(kd, code_ptr, planes, l, P, 1, lane);
    if (mover) {
        // static indexing of the per-row arrays
#pragma unroll
        for (int r = 0; r < HASH_ROWS; ++r) {
            if (warp != r || cache_row[r] < 0) continue;
            KT* kdst = k_cache + cache_row[r] * D;
            KT* vdst = v_cache + cache_row[r] * D;
            double ss = 0.0;
#pragma unroll
            for (int i = 0; i < EPL; ++i) {
                const int d = lane * EPL + i;
                kdst[d] = kraw[r][i];
                vdst[d] = vraw[i];
                const double xf = (double)to_f32(vraw[i]);
                ss = fma(xf, xf, ss);
            }
            ss = warp_sum_f64(ss);
            if (lane == 0) v_norm[cache_row[r]] = __float2half_rn((float)sqrt(ss));
        }
    }
}

}  // namespace sk
