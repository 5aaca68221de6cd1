// Device code of the query soft hash: for one KV-head group, one head tile and a few tables,
// the softmax over the R buckets of (tanh(<q, plane>) / sqrt(D)) . protos_T / temperature.
#pragma once
#include "common.cuh"

namespace sk {

constexpr int SH_THREADS = 256;
constexpr int SH_WARPS = SH_THREADS / 32;

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

// shared memory (floats): protos [P*R] | t [SH_WARPS*16] | red [SH_WARPS] | stage [tables_per_cta * R * ht]
inline size_t soft_hash_smem_bytes(int P, int R, int ht) {
    return sizeof(float) * ((size_t)P * R + SH_WARPS * 16 + SH_WARPS + (size_t)(SH_WARPS / ht) * R * ht);
}

// ---- 12-bit fixed-point copy of the scorer table (the filtering scorer's packed mode) ----------
// entry = floor((p - lo) * C), 0 <= entry <= PK_QMAX, with lo and C the same for every table and
// head of a call: they follow from a bound that needs no data, |tanh| <= 1, so every CTA computes
// the same constants on its own.  With lam = max_r sum_p |protos_T[p][r]| / (sqrt(D) * temperature)
// every logit lies in [-lam, lam], hence every probability in
//   [1 / (1 + (R-1) e^{2 lam}),  1 / (1 + (R-1) e^{-2 lam})].
// The sum of a key's L entries then satisfies   sum_l (p_l - lo) * C  in  [S - 0.1, S + L + 0.1),
// which is what the candidate select relies on (see select.cu).  K0 = L * lo * C is handed on.
constexpr int PK_QMAX = 4095;
struct PackedQuant {
    float lo, C, K0;
};
__device__ __forceinline__ PackedQuant packed_quant(float lam, int R, int L) {
    PackedQuant q;
    const float e2 = __expf(fminf(2.f * lam, 80.f));
    const float lo = 1.f / (1.f + (float)(R - 1) * e2);
    const float hi = 1.f / (1.f + (float)(R - 1) / e2);
    q.lo = lo * (1.f - 1e-5f);                       // margins: the softmax is rounded arithmetic
    const float range = fmaxf(hi * (1.f + 1e-5f) - q.lo, hi * 1e-6f);
    float C = (float)PK_QMAX * (1.f - 1e-4f) / range;
    // K0 <= 2^17, so S + K0 < 2^18: the fp32 summation error of an exact score (31 roundings,
    // each at most 2^-24 of the sum) stays below half a table unit, inside the bracket's slack
    const float cap = (float)(1 << 17) / ((float)L * fmaxf(q.lo, 1e-30f));
    q.C = fminf(C, cap);
    q.K0 = (float)L * q.lo * q.C;
    return q;
}
__device__ __forceinline__ uint32_t packed_entry(float p, const PackedQuant& q) {
    const int e = __float2int_rd((p - q.lo) * q.C);
    return (uint32_t)min(max(e, 0), PK_QMAX);
}

// One CTA: head tile `g` (= (b*Hkv + kvh)*tiles + tile) and tables [l0, l0 + SH_WARPS/ht).
// Warp w handles (table l0 + w / ht, head w % ht).  All global loads of a warp are issued
// before the first use, so a cold call costs one memory round trip.
template <typename QT, typename PT>
__device__ __forceinline__ void soft_hash_body(
    const QT* __restrict__ q, const PT* __restrict__ planes, const float* __restrict__ protos_T,
    float inv_temperature, int H, int Hkv, int D, int L, int P, int R, int ht, int g, int l0,
    float* __restrict__ q_probs, float* __restrict__ lut, float* smem,
    uint2* __restrict__ lutq = nullptr, float* __restrict__ qpar = nullptr) {
    const int rep = H / Hkv;
    const int tiles = rep / ht;
    const int tile = g % tiles;
    const int bk = g / tiles;
    const int b = bk / Hkv, kvh = bk - b * Hkv;
    const int h0 = kvh * rep + tile * ht;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tpc = SH_WARPS / ht;                // tables per CTA
    const int lt = warp / ht, j = warp - lt * ht;
    const int l = l0 + lt;
    const bool active = l < L;

    float* pr_s = smem;                           // [P][R]
    float* t_s = pr_s + (size_t)P * R;            // [SH_WARPS][16]
    float* red_s = t_s + SH_WARPS * 16;           // [SH_WARPS]
    float* stage = red_s + SH_WARPS;              // [tpc][R][ht]

    // every global load of the CTA is issued before the first one is consumed: the protos (kept in
    // registers until the dot products are done) together with the plane / query rows
    const bool fast = (P == 8 && R == 256);
    float prr[8];
    if (fast) {
#pragma unroll
        for (int i = 0; i < 8; ++i) prr[i] = protos_T[threadIdx.x + i * SH_THREADS];
    }
    float part[16];
#pragma unroll
    for (int p = 0; p < 16; ++p) part[p] = 0.f;
    if (active) {
        const QT* qh = q + ((size_t)b * H + h0 + j) * D;
        const PT* pl = planes + (size_t)l * P * D;
        if (D == 128 && P == 8) {
            // four consecutive elements per lane: every load of the warp is issued up front
            float qv[4], pv[8][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) qv[i] = to_f32(qh[lane * 4 + i]);
#pragma unroll
            for (int p = 0; p < 8; ++p)
#pragma unroll
                for (int i = 0; i < 4; ++i) pv[p][i] = to_f32(pl[p * 128 + lane * 4 + i]);
#pragma unroll
            for (int p = 0; p < 8; ++p)
#pragma unroll
                for (int i = 0; i < 4; ++i) part[p] = fmaf(qv[i], pv[p][i], part[p]);
        } else {
            for (int d = lane; d < D; d += 32) {
                const float qv = to_f32(qh[d]);
#pragma unroll
                for (int p = 0; p < 16; ++p)
                    if (p < P) part[p] = fmaf(qv, to_f32(pl[(size_t)p * D + d]), part[p]);
            }
        }
    }
    if (fast) {
#pragma unroll
        for (int i = 0; i < 8; ++i) pr_s[threadIdx.x + i * SH_THREADS] = prr[i];
    } else {
        for (int i = threadIdx.x; i < P * R; i += SH_THREADS) pr_s[i] = protos_T[i];
    }
    const float inv_sqrt_d = 1.0f / fmaxf(sqrtf((float)D), 1e-6f);
    // lane p keeps the p-th dot product, so the P tanh evaluations run side by side
    float mine = 0.f;
#pragma unroll
    for (int p = 0; p < 16; ++p) {
        if (p < P) {
            const float s = warp_sum_f(part[p]);
            if (lane == p) mine = s;
        }
    }
    if (lane < P) t_s[warp * 16 + lane] = tanhf(mine) * inv_sqrt_d;
    __syncthreads();
    if (lutq != nullptr) {
        // largest column sum of |protos_T|: one partial maximum per warp, combined after the next barrier
        float cs = 0.f;
        for (int r = threadIdx.x; r < R; r += SH_THREADS) {
            float a = 0.f;
            for (int p = 0; p < P; ++p) a += fabsf(pr_s[p * R + r]);
            cs = fmaxf(cs, a);
        }
        cs = warp_max_f(cs);
        if (lane == 0) red_s[warp] = cs;
    }

    if (active) {
        const float* t = t_s + warp * 16;
        float* qp_row = q_probs ? q_probs + (((size_t)b * H + h0 + j) * L + l) * R : nullptr;
        if (R == 256 && P <= 16) {
            // 8 buckets per lane, logits kept in registers
            float lg[8];
            float mx = -INFINITY;
            if (P == 8) {
                float tv[8];
#pragma unroll
                for (int p = 0; p < 8; ++p) tv[p] = t[p];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float a = 0.f;
#pragma unroll
                    for (int p = 0; p < 8; ++p) a = fmaf(tv[p], pr_s[p * 256 + lane + 32 * i], a);   // same order as below
                    lg[i] = a * inv_temperature;
                    mx = fmaxf(mx, lg[i]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float a = 0.f;
                    for (int p = 0; p < P; ++p) a = fmaf(t[p], pr_s[p * 256 + lane + 32 * i], a);
                    lg[i] = a * inv_temperature;
                    mx = fmaxf(mx, lg[i]);
                }
            }
            mx = warp_max_f(mx);
            float se = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                lg[i] = expf(lg[i] - mx);
                se += lg[i];
            }
            se = warp_sum_f(se);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int r = lane + 32 * i;
                const float pr = lg[i] / se;
                if (qp_row) qp_row[r] = pr;
                stage[((size_t)lt * 256 + r) * ht + j] = pr;
            }
        } else {
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
            for (int r = lane; r < R; r += 32) {
                float lg = 0.f;
                for (int p = 0; p < P; ++p) lg = fmaf(t[p], pr_s[p * R + r], lg);
                const float pr = expf(lg * inv_temperature - mx) / se;
                if (qp_row) qp_row[r] = pr;
                stage[((size_t)lt * R + r) * ht + j] = pr;
            }
        }
    }
    if (lut == nullptr && lutq == nullptr) return;
    __syncthreads();
    // scorer table rows: lut[g][r][l][0..ht) (fp32; not written when the caller keeps the packed table and
    // the probabilities only) and the packed copy
    float* lut_g = lut != nullptr ? lut + (size_t)g * R * L * ht : nullptr;
    const bool packed = lutq != nullptr && ht == 4;
    PackedQuant pq = {0.f, 0.f, 0.f};
    uint2* lutq_g = nullptr;
    if (packed) {
        float lam = 0.f;
#pragma unroll
        for (int w = 0; w < SH_WARPS; ++w) lam = fmaxf(lam, red_s[w]);
        pq = packed_quant(lam * inv_sqrt_d * inv_temperature, R, L);
        lutq_g = lutq + (size_t)g * 256 * L;          // 256 bucket slots whatever R is
        if (l0 == 0 && threadIdx.x == 0) qpar[g] = pq.K0;
    }
    for (int i = threadIdx.x; i < tpc * R; i += SH_THREADS) {
        const int lt2 = i / R, r = i - lt2 * R;
        if (l0 + lt2 >= L) continue;
        const float* src = stage + (size_t)i * ht;
        float* dst = lut_g + ((size_t)r * L + l0 + lt2) * ht;      // not dereferenced when lut_g is null
        if (ht == 4) {
            const float4 v = *reinterpret_cast<const float4*>(src);
            if (lut_g != nullptr) *reinterpret_cast<float4*>(dst) = v;
            if (packed)
                lutq_g[(size_t)r * L + l0 + lt2] =
                    make_uint2(packed_entry(v.x, pq) | (packed_entry(v.y, pq) << 16),
                               packed_entry(v.z, pq) | (packed_entry(v.w, pq) << 16));
        } else if (lut_g == nullptr) {
            continue;
        } else if (ht == 2) *reinterpret_cast<float2*>(dst) = *reinterpret_cast<const float2*>(src);
        else *dst = *src;
    }
}

}  // namespace sk
