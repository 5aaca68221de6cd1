// Device pieces shared by the scorer kernels: bulk copy of the scorer table into shared memory
// (cp.async.bulk completing on an mbarrier, bounded wait) and the per-key table walk.
#pragma once

#include "common.cuh"

namespace sk {
namespace {

constexpr uint32_t SC_WAIT_LIMIT = 1u << 20;   // bounded wait on the table copy
constexpr int SC_COPY_CHUNK = 16384;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
            "r"(smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
// Returns false if the phase did not complete within the iteration limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < SC_WAIT_LIMIT; ++it) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

template <int HT> struct Word;
template <> struct Word<4> { using type = float4; };
template <> struct Word<2> { using type = float2; };
template <> struct Word<1> { using type = float; };

template <int HT>
__device__ __forceinline__ void add_word(float (&acc)[HT], const char* p) {
    if constexpr (HT == 4) {
        const float4 w = *reinterpret_cast<const float4*>(p);
        acc[0] += w.x; acc[1] += w.y; acc[2] += w.z; acc[3] += w.w;
    } else if constexpr (HT == 2) {
        const float2 w = *reinterpret_cast<const float2*>(p);
        acc[0] += w.x; acc[1] += w.y;
    } else {
        acc[0] += *reinterpret_cast<const float*>(p);
    }
}

// Sum over the L tables of one key's table words (ht heads at once).
template <int L, int HT>
__device__ __forceinline__ void score_key(const uint4 (&c)[L / 16], const char* lut_s, uint32_t sel_lo,
                                          uint32_t sel_hi, uint32_t mL, float (&acc)[HT]) {
    constexpr int L_STRIDE = HT * 4;
    constexpr int CODE_STRIDE = L * L_STRIDE;
#pragma unroll
    for (int j = 0; j < HT; ++j) acc[j] = 0.f;
#pragma unroll
    for (int i = 0; i < L / 16; ++i) {
        const uint32_t w[4] = {c[i].x, c[i].y, c[i].z, c[i].w};
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            // 8 tables: bytes permuted so that byte j holds table j ^ m
            const uint32_t lo = __byte_perm(w[2 * half], w[2 * half + 1], sel_lo);
            const uint32_t hi = __byte_perm(w[2 * half], w[2 * half + 1], sel_hi);
            const int lbase = (i * 16 + half * 8) * L_STRIDE;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t src = j < 4 ? lo : hi;
                const uint32_t code = (src >> (8 * (j & 3))) & 0xffu;
                const uint32_t off = code * CODE_STRIDE + (((uint32_t)j * L_STRIDE) ^ mL);
                add_word<HT>(acc, lut_s + lbase + off);
            }
        }
    }
}

}  // namespace
}  // namespace sk
