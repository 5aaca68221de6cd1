// Bulk key hashing on the 5th-generation tensor cores (prefill: thousands of rows).
//
// codes = sign( K[N,128] . planes^T[128, L*P = 256] ) packed 8 planes -> one byte per table.
// Persistent CTAs, one per SM, walk the 128-row tiles of K.  The 256 plane rows stay in shared
// memory; TMA (cp.async.bulk.tensor, 128-byte swizzle) feeds a two-stage ring of K tiles, one
// elected thread issues eight tcgen05.mma.kind::f16 (M=128, N=256, K=16) per tile into one of two
// fp32 accumulators in tensor memory, and eight epilogue warps read the other accumulator back
// with tcgen05.ld (two threads per row), take the signs and write 32 code bytes per row, so
// loading, multiplying and the epilogue of consecutive tiles overlap.
//
// Exactness.  bf16 x bf16 products are exact in fp32, only the accumulation rounds, so a sign
// can be wrong only when |acc| is tiny compared with |k|.|p|.  Every projection with
// |acc| <= 2^-16 |k| |p| (a bound far above the accumulation error of 128 terms) is put on a
// list and decided again by a second kernel from the exact fp64 dot product, which patches the
// bit; ~1e-4 of the projections take that path.  Rows of zeros hash to all-ones bytes directly.
// If the list overflows (adversarial inputs), a third kernel rehashes everything exactly.
#include <cuda.h>

#include "hash_body.cuh"

namespace sk {
namespace {

constexpr int TC_ROWS = 128;          // rows of K per CTA (MMA M)
constexpr int TC_N = 256;             // L * P (MMA N)
constexpr int TC_D = 128;             // head dim (MMA K total)
constexpr int TC_KHALF = 64;          // bf16 elements per 128-byte swizzle row
constexpr uint32_t TC_A_HALF_BYTES = TC_ROWS * 128;   // 16 KiB
constexpr uint32_t TC_B_HALF_BYTES = TC_N * 128;      // 32 KiB
constexpr uint32_t TC_PIPE_SMEM = 2 * TC_B_HALF_BYTES + 4 * 2 * TC_A_HALF_BYTES;   // planes + four K tiles: 192 KiB
constexpr uint32_t TC_WAIT_LIMIT = 1u << 17;   // polls; a poll that fails takes microseconds, so well under a second
constexpr float TC_BAND = 1.52587890625e-05f;         // 2^-16

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_addr(bar);
    for (uint32_t it = 0; it < TC_WAIT_LIMIT; ++it) {
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

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_addr(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_addr(bar))
        : "memory");
}

// K-major operand tile, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);        // start address, 16-byte units
    d |= (uint64_t)1 << 16;                          // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                // stride byte offset: 8 rows x 128 B
    d |= (uint64_t)1 << 46;                          // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                          // SWIZZLE_128B
    return d;
}

// kind::f16, A = B = bf16 (K-major), D = fp32, M = 128, N = 256
constexpr uint32_t TC_IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((TC_N >> 3) << 17) | ((TC_ROWS >> 4) << 24);

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(TC_IDESC), "r"(accumulate), "r"(0u)
        : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

constexpr int TC_STAGES = 2;          // accumulators in tensor memory
constexpr int TC_ARING = 4;           // K tiles in flight
constexpr int TC_NSLOTS = 8;          // norm slots
constexpr int TC_NORM_WARPS = 4;      // one thread per row of the K tile
constexpr int TC_EPI_WARPS = 16;      // four threads per accumulator row, 64 columns each
constexpr int TC_PIPE_THREADS = 32 * (2 + TC_NORM_WARPS + TC_EPI_WARPS);   // TMA warp, MMA warp, norm warps, epilogue warps

struct TcShared {
    uint64_t b_full;                   // planes have landed (once)
    uint64_t a_full[TC_ARING];         // K tile of the ring slot has landed
    uint64_t a_empty[TC_ARING];        // MMAs and the norm warps are done with the slot's K tile
    uint64_t norm_full[TC_NSLOTS];     // row norms of tile i are in knorm[i % 8]
    uint64_t acc_full[TC_STAGES];      // accumulator is complete
    uint64_t acc_empty[TC_STAGES];     // accumulator has been read back
    uint32_t tmem_base;
    int failed;                        // some bounded wait ran out
    float plane_norm[TC_N + 1];        // [TC_N] = the largest norm
    float knorm[TC_NSLOTS][TC_ROWS];   // |k| * 1.001 of the rows of tile i in slot i % 8 (inf: decide every bit exactly)
};

__device__ __forceinline__ void mbar_init_count(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar))
                 : "memory");
}

// One projection inside the cheap near-zero band: apply the exact band of its plane and list it.
__device__ __noinline__ void list_near_zero(float acc, int col, int64_t row, float thr, const float* plane_norm_s,
                                            uint32_t* fix_count, uint32_t* __restrict__ fix_list, uint32_t fix_cap) {
    if (fabsf(acc) <= thr * plane_norm_s[col]) {
        const uint32_t slot = atomicAdd(fix_count, 1u);
        if (slot < fix_cap) fix_list[slot] = ((uint32_t)row << 8) | (uint32_t)col;
    }
}

// The careful version of one 32-column chunk of one accumulator row (see the epilogue).
__device__ __noinline__ uint32_t slow_chunk(uint32_t taddr, int c, int64_t row, float thr, float knorm,
                                            const float* plane_norm_s, uint32_t* fix_count,
                                            uint32_t* __restrict__ fix_list, uint32_t fix_cap) {
    uint32_t r[32];
    tmem_ld32(taddr, r);
    uint32_t word = 0;
#pragma unroll 1
    for (int k = 0; k < 32; ++k) {
        const float acc = __uint_as_float(r[k]);
        if (acc >= 0.f) word |= 1u << (8 * (k >> 3) + 7 - (k & 7));
        if (fabsf(acc) <= thr * plane_norm_s[c * 32 + k] && knorm > 0.f) {
            const uint32_t slot = atomicAdd(fix_count, 1u);
            if (slot < fix_cap) fix_list[slot] = ((uint32_t)row << 8) | (uint32_t)(c * 32 + k);
        }
    }
    return word;
}

// Persistent, warp-specialised: every CTA keeps the 256 plane rows in shared memory and walks the
// K tiles blockIdx.x, blockIdx.x + gridDim.x, ...  Warp 0 feeds a two-stage ring of K tiles by
// TMA, warp 1 issues the MMAs into one of two accumulators in tensor memory, warps 6-21 read the
// other accumulator back (tcgen05.ld), take the signs, apply the near-zero test and write the code
// bytes; warps 2-5 compute the row norms that test needs from the K tile in shared memory - so the
// load of tile i+1, the MMAs of tile i+1 and the epilogue of tile i overlap.  Every wait is bounded; a wait that runs out
// raises `failed`, which makes every role leave its loop, and the status flag.
__global__ void __launch_bounds__(TC_PIPE_THREADS, 1)
hash_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_p,
               const __nv_bfloat16* __restrict__ planes, int64_t N, uint8_t* __restrict__ codes,
               int64_t code_row_stride, const int64_t* __restrict__ dst_row, uint32_t* fix_count,
               uint32_t* __restrict__ fix_list, uint32_t fix_cap, int32_t* status) {
    extern __shared__ char tc_raw[];
    __shared__ TcShared ts;
    pdl_launch_dependents();                   // the fix-up kernels may start launching; they wait for this grid
    char* tiles = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(tc_raw) + 1023) & ~(uintptr_t)1023);
    char* b_half[2] = {tiles, tiles + TC_B_HALF_BYTES};
    char* a_base = tiles + 2 * TC_B_HALF_BYTES;                 // [ring slot][half][16 KiB]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t n_tiles = (N + TC_ROWS - 1) / TC_ROWS;
    const int64_t my_tiles = (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;     // >= 1: grid <= n_tiles

    // |plane| * 1.001 of the 256 planes, one warp per plane (every CTA computes them for itself:
    // 64 KiB from L2, cheaper than a launch of its own)
    for (int n = warp; n < TC_N; n += TC_PIPE_THREADS / 32) {
        const uint2 raw = __ldg(reinterpret_cast<const uint2*>(planes + (size_t)n * TC_D) + lane);
        const float x0 = __uint_as_float(raw.x << 16), x1 = __uint_as_float(raw.x & 0xffff0000u);
        const float x2 = __uint_as_float(raw.y << 16), x3 = __uint_as_float(raw.y & 0xffff0000u);
        float sq = fmaf(x0, x0, fmaf(x1, x1, fmaf(x2, x2, x3 * x3)));
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) sq += __shfl_xor_sync(FULL, sq, o);
        if (lane == 0) ts.plane_norm[n] = sqrtf(sq) * 1.001f;
    }
    if (tid == 0) {
        mbar_init_count(&ts.b_full, 1);
        for (int s = 0; s < TC_ARING; ++s) {
            mbar_init_count(&ts.a_full[s], 1);
            mbar_init_count(&ts.a_empty[s], 1 + TC_NORM_WARPS); // MMA commit + one arrival per norm warp
        }
        for (int s = 0; s < TC_NSLOTS; ++s) mbar_init_count(&ts.norm_full[s], TC_NORM_WARPS);
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init_count(&ts.acc_full[s], 1);
            mbar_init_count(&ts.acc_empty[s], TC_EPI_WARPS);
        }
        ts.failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_addr(&ts.tmem_base)),
                     "r"((uint32_t)(TC_STAGES * TC_N))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = ts.tmem_base;
    volatile int* failed = &ts.failed;
    if (warp == 2) {                          // the largest plane norm, for the cheap first test
        float v = 0.f;
        for (int n = lane; n < TC_N; n += 32) v = fmaxf(v, ts.plane_norm[n]);
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) v = fmaxf(v, __shfl_xor_sync(FULL, v, o));
        if (lane == 0) ts.plane_norm[TC_N] = v;
    }
    __syncthreads();

    if (warp == 0) {
        // ---- TMA producer
        if (lane == 0) {
            mbar_expect(&ts.b_full, 2 * TC_B_HALF_BYTES);
            tma_load_2d(b_half[0], &map_p, 0, 0, &ts.b_full);
            tma_load_2d(b_half[1], &map_p, TC_KHALF, 0, &ts.b_full);
            for (int64_t i = 0; i < my_tiles && !*failed; ++i) {
                const int ra = (int)(i % TC_ARING);
                if (i >= TC_ARING && !mbar_wait_bounded(&ts.a_empty[ra], (uint32_t)((i / TC_ARING - 1) & 1))) {
                    *failed = 1;
                    break;
                }
                const int row0 = (int)((blockIdx.x + i * gridDim.x) * TC_ROWS);
                char* a = a_base + (size_t)ra * 2 * TC_A_HALF_BYTES;
                mbar_expect(&ts.a_full[ra], 2 * TC_A_HALF_BYTES);
                tma_load_2d(a, &map_k, 0, row0, &ts.a_full[ra]);
                tma_load_2d(a + TC_A_HALF_BYTES, &map_k, TC_KHALF, row0, &ts.a_full[ra]);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer
        if (lane == 0) {
            if (!mbar_wait_bounded(&ts.b_full, 0)) *failed = 1;
            for (int64_t i = 0; i < my_tiles && !*failed; ++i) {
                const int s = (int)(i & 1), ra = (int)(i % TC_ARING);
                const uint32_t par = (uint32_t)((i >> 1) & 1);
                if (!mbar_wait_bounded(&ts.a_full[ra], (uint32_t)((i / TC_ARING) & 1)) ||
                    (i >= TC_STAGES && !mbar_wait_bounded(&ts.acc_empty[s], par ^ 1u))) {
                    *failed = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_addr(a_base + (size_t)ra * 2 * TC_A_HALF_BYTES);
#pragma unroll
                for (int k = 0; k < TC_D / 16; ++k) {
                    const int half = k >> 2, kb = k & 3;           // 16 bf16 = 32 bytes along the swizzled row
                    const uint64_t da = umma_desc_sw128(a_addr + half * TC_A_HALF_BYTES + kb * 32);
                    const uint64_t db = umma_desc_sw128(smem_addr(b_half[half]) + kb * 32);
                    umma_bf16(tmem + (uint32_t)s * TC_N, da, db, k > 0 ? 1u : 0u);
                }
                umma_commit(&ts.acc_full[s]);                       // accumulator complete ...
                umma_commit(&ts.a_empty[ra]);                       // ... and the K tile no longer read by the MMAs
            }
        }
    } else if (warp < 2 + TC_NORM_WARPS) {
        // ---- row norms: one thread per row of the K tile, read from the swizzled tile in shared memory
        // (16-byte chunk c of row r sits at chunk c ^ (r & 7))
        const int r_in_tile = (warp - 2) * 32 + lane;
        for (int64_t i = 0; i < my_tiles; ++i) {
            if (__any_sync(FULL, *failed != 0)) break;                 // warp-uniform
            const int ra = (int)(i % TC_ARING);
            // The tile has landed.  Its norms go to slot i % 8, which has a barrier of its own (the norm
            // warps may be several tiles ahead of the epilogue, and a barrier must not complete two
            // phases ahead of a waiter): tile i can only have been loaded after the MMAs of tile i-4
            // were done, which started after the epilogue of tile i-6 had finished, so the last reader
            // of the slot (tile i-8) is long gone and the norm warps never wait for the epilogue.
            if (!__all_sync(FULL, mbar_wait_bounded(&ts.a_full[ra], (uint32_t)((i / TC_ARING) & 1)))) {
                *failed = 1;
                break;
            }
            float ss = 0.f;
            const char* a = a_base + (size_t)ra * 2 * TC_A_HALF_BYTES + (size_t)r_in_tile * 128;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 w = *reinterpret_cast<const uint4*>(a + h * TC_A_HALF_BYTES + ((c ^ (r_in_tile & 7)) << 4));
                    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float x = __uint_as_float(u[j] << 16), y = __uint_as_float(u[j] & 0xffff0000u);
                        ss = fmaf(x, x, fmaf(y, y, ss));
                    }
                }
            }
            float kn = sqrtf(ss) * 1.001f;
            // a row whose products could overflow fp32 gets an infinite norm: every projection of it is
            // then listed for the exact kernel (a NaN norm stays NaN and is handled in the epilogue)
            if (kn * ts.plane_norm[TC_N] >= 1e38f) kn = INFINITY;
            ts.knorm[i % TC_NSLOTS][r_in_tile] = kn;
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&ts.norm_full[i % TC_NSLOTS]);
                mbar_arrive(&ts.a_empty[ra]);
            }
        }
    } else {
        // ---- epilogue: the four warps with the same (warp % 4) share the 32 accumulator lanes of that
        // quarter, a quarter of the columns each; a thread owns one row and 64 columns = 8 tables
        const int quad = warp & 3, cq = (warp - 2 - TC_NORM_WARPS) >> 2;
        const int r_in_tile = quad * 32 + lane;
        for (int64_t i = 0; i < my_tiles; ++i) {
            if (__any_sync(FULL, *failed != 0)) break;                 // warp-uniform
            const int s = (int)(i & 1);
            const uint32_t par = (uint32_t)((i >> 1) & 1);
            const int64_t row = (blockIdx.x + i * gridDim.x) * TC_ROWS + r_in_tile;
            const bool valid = row < N;
            int64_t dst = valid ? row : -1;
            if (valid && dst_row != nullptr) dst = dst_row[row];    // requested before the waits below
            if (!__all_sync(FULL, mbar_wait_bounded(&ts.norm_full[i % TC_NSLOTS], (uint32_t)((i / TC_NSLOTS) & 1)))) {  // warp-uniform decision
                *failed = 1;
                break;
            }
            const float knorm = valid ? ts.knorm[i % TC_NSLOTS][r_in_tile] : 0.f;
            const float thr = TC_BAND * knorm;
            const float thr_max = valid ? thr * ts.plane_norm[TC_N] : -1.f;  // cheap first test, exact test inside
            if (!__all_sync(FULL, mbar_wait_bounded(&ts.acc_full[s], par))) {
                *failed = 1;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t words[2];
#pragma unroll
            for (int c4 = 0; c4 < 2; ++c4) {
                const int c = cq * 2 + c4;
                uint32_t r[32];
                tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)s * TC_N + c * 32, r);
                // Fast path, two instructions per projection and no branch: the sign bits are shifted
                // into one register per table (first plane = most significant bit) and the smallest
                // |acc| of the chunk decides whether anything needs the near-zero treatment.  A finite
                // norm below the overflow guard means every accumulator is finite.
                uint32_t neg[4] = {0u, 0u, 0u, 0u};
                float mn[4] = {INFINITY, INFINITY, INFINITY, INFINITY};
#pragma unroll
                for (int k = 0; k < 32; ++k) {
                    neg[k >> 3] = __funnelshift_l(r[k], neg[k >> 3], 1);
                    mn[k & 3] = fminf(mn[k & 3], fabsf(__uint_as_float(r[k])));
                }
                uint32_t word = ~(neg[0] | (neg[1] << 8) | (neg[2] << 16) | (neg[3] << 24));
                const float m = fminf(fminf(mn[0], mn[1]), fminf(mn[2], mn[3]));
                if (m <= thr_max && knorm < INFINITY && knorm > 0.f) {
                    // some projection of this row is near zero (about one chunk in seven has one): list
                    // it for the exact kernel.  The bits above stay as they are - the only value whose
                    // sign bit disagrees with (acc >= 0) is -0, and that one is always listed.  Only the
                    // eight columns of a residue class whose minimum fell inside the band are looked at.
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        if (mn[q] <= thr_max) {
#pragma unroll
                            for (int k = q; k < 32; k += 4)
                                if (fabsf(__uint_as_float(r[k])) <= thr_max)
                                    list_near_zero(__uint_as_float(r[k]), c * 32 + k, row, thr, ts.plane_norm, fix_count,
                                                   fix_list, fix_cap);
                        }
                    }
                }
                // warp-uniform: the reload in the careful path is a warp-wide instruction
                if (__any_sync(FULL, !(knorm < INFINITY) || knorm == 0.f)) {
                    // rare: a row that may overflow or holds NaN, or a row of zeros - decide every bit
                    // the plain way (a rolled loop over a second copy of the chunk, out of line)
                    const uint32_t w2 = slow_chunk(tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)s * TC_N + c * 32, c,
                                                   row, thr, knorm, ts.plane_norm, fix_count, fix_list, fix_cap);
                    if (!(knorm < INFINITY) || knorm == 0.f) word = w2;
                }
                words[c4] = word;
            }
            // accumulator and K tile of this stage are free again
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&ts.acc_empty[s]);
            if (dst >= 0)                                          // negative = row not to be written
                reinterpret_cast<uint2*>(codes + dst * code_row_stride)[cq] = make_uint2(words[0], words[1]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0 && ts.failed && status != nullptr) atomicOr(status, SK_DEV_WAIT_TIMEOUT);
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem),
                     "r"((uint32_t)(TC_STAGES * TC_N))
                     : "memory");
    }
}

// One warp per listed projection: exact fp64 dot product, then set or clear the code bit.
__global__ void __launch_bounds__(256)
hash_fix_kernel(const __nv_bfloat16* __restrict__ keys, int64_t key_row_stride,
                const __nv_bfloat16* __restrict__ planes, uint8_t* __restrict__ codes,
                int64_t code_row_stride, const int64_t* __restrict__ dst_row,
                const uint32_t* __restrict__ fix_count, const uint32_t* __restrict__ fix_list,
                uint32_t fix_cap) {
    const int lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();                                // the list, its length and the codes come from the kernel before
    const uint32_t n = min(__ldcg(fix_count), fix_cap);
    const uint32_t warps = gridDim.x * (blockDim.x >> 5);
    for (uint32_t e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); e < n; e += warps) {
        const uint32_t ent = __ldcg(fix_list + e);
        const int64_t row = ent >> 8;
        const int col = (int)(ent & 0xffu);               // l * 8 + p
        const __nv_bfloat16* k = keys + row * key_row_stride;
        const __nv_bfloat16* p = planes + (size_t)col * TC_D;
        double s = 0.0;
#pragma unroll
        for (int i = 0; i < TC_D / 32; ++i) {
            const int d = lane * (TC_D / 32) + i;
            s = fma((double)__bfloat162float(k[d]), (double)__bfloat162float(p[d]), s);
        }
        s = warp_sum_f64(s);
        if (lane == 0) {
            const int64_t dst = dst_row ? dst_row[row] : row;
            if (dst < 0) continue;
            const int l = col >> 3, bit = 7 - (col & 7);
            uint8_t* byte = codes + dst * code_row_stride + l;
            uint32_t* word = reinterpret_cast<uint32_t*>(reinterpret_cast<uintptr_t>(byte) & ~(uintptr_t)3);
            const uint32_t m = 1u << (8 * (int)(reinterpret_cast<uintptr_t>(byte) & 3) + bit);
            if (s >= 0.0) atomicOr(word, m); else atomicAnd(word, ~m);
        }
    }
}

// Runs only when the list overflowed: exact hashing of every row (the slow, always-right path).
__global__ void __launch_bounds__(HASH_THREADS)
hash_exact_if_overflow_kernel(const __nv_bfloat16* __restrict__ keys, int64_t key_row_stride,
                              const __nv_bfloat16* __restrict__ planes, int64_t N, uint8_t* codes,
                              int64_t code_row_stride, const int64_t* __restrict__ dst_row,
                              const uint32_t* __restrict__ fix_count, uint32_t fix_cap) {
    pdl_wait();                                // after the fix-up kernel, which may still be patching codes
    if (__ldcg(fix_count) <= fix_cap) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int l = blockIdx.y * HASH_WARPS + warp;
    for (int64_t n0 = (int64_t)blockIdx.x * HASH_ROWS; n0 < N; n0 += (int64_t)gridDim.x * HASH_ROWS) {
        double kd[HASH_ROWS][4];
        void* code_ptr[HASH_ROWS];
#pragma unroll
        for (int r = 0; r < HASH_ROWS; ++r) {
            const int64_t n = n0 + r;
            if (n < N) {
                load_row_f64<__nv_bfloat16, 4>(keys + n * key_row_stride, lane, kd[r]);
                const int64_t dst = dst_row ? dst_row[n] : n;
                code_ptr[r] = dst >= 0 ? codes + dst * code_row_stride : nullptr;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) kd[r][i] = 0.0;
                code_ptr[r] = nullptr;
            }
        }
        if (l < TC_N / 8) hash_table_rows<__nv_bfloat16, 4>(kd, code_ptr, planes, l, 8, 1, lane);
    }
}

// Cache row of every new (b, s, kvh) row; -1 (and a status flag) for positions outside the cache.
__global__ void __launch_bounds__(256)
cache_rows_kernel(const int64_t* __restrict__ input_pos, int B, int S, int Hkv, int64_t Tcap,
                  int64_t* __restrict__ dst_row, int32_t* status) {
    const int64_t N = (int64_t)B * S * Hkv;
    for (int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; n < N; n += (int64_t)gridDim.x * blockDim.x) {
        const int kvh = (int)(n % Hkv);
        const int s = (int)((n / Hkv) % S);
        const int b = (int)(n / ((int64_t)Hkv * S));
        const int64_t pos = input_pos[s];
        const bool ok = pos >= 0 && pos < Tcap;
        dst_row[n] = ok ? ((int64_t)b * Hkv + kvh) * Tcap + pos : -1;
        if (!ok && status != nullptr) atomicOr(status, SK_DEV_POS_OUT_OF_RANGE);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// [rows, 128] bf16 row-major (row stride in elements) -> boxes of 64 columns x box_rows rows
int make_map(CUtensorMap* map, const void* base, uint64_t rows, int64_t row_stride, uint32_t box_rows) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (enc == nullptr) return fail(SK_ERR_CUDA, "sk_hash_keys_tc: cuTensorMapEncodeTiled is not available");
    const cuuint64_t dims[2] = {(cuuint64_t)TC_D, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
    const cuuint32_t box[2] = {(cuuint32_t)TC_KHALF, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                           estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SK_ERR_CUDA, "sk_hash_keys_tc: cuTensorMapEncodeTiled failed (%d)", (int)r);
    return SK_OK;
}

constexpr size_t TC_WS_HEADER = 256 + (TC_N + 16) * sizeof(float);   // list counter | plane norms + max

}  // namespace

int launch_cache_rows(const int64_t* input_pos, int B, int S, int Hkv, int64_t Tcap, int64_t* dst_row,
                      int32_t* status, cudaStream_t st) {
    const int64_t N = (int64_t)B * S * Hkv;
    int64_t g = (N + 255) / 256;
    if (g > sm_count() * 8) g = sm_count() * 8;
    cache_rows_kernel<<<(unsigned)g, 256, 0, st>>>(input_pos, B, S, Hkv, Tcap, dst_row, status);
    return check_launch("cache_rows_kernel");
}

size_t hash_keys_tc_workspace_bytes(int64_t N) {
    const int64_t cap = N > 4096 ? N : 4096;
    return TC_WS_HEADER + (size_t)cap * sizeof(uint32_t);
}

int launch_hash_keys_tc(const void* keys, int64_t key_row_stride, const void* planes, int64_t N, uint8_t* codes,
                        int64_t code_row_stride, const int64_t* dst_row, void* workspace, size_t workspace_bytes,
                        int32_t* status, cudaStream_t st) {
    if (N == 0) return SK_OK;
    if (N >= (1 << 24)) return fail(SK_ERR_UNSUPPORTED, "sk_hash_keys_tc: at most 2^24 - 1 rows per call");
    if (workspace_bytes < TC_WS_HEADER + 1024 * sizeof(uint32_t))
        return fail(SK_ERR_WORKSPACE, "sk_hash_keys_tc: workspace %zu bytes is too small", workspace_bytes);
    char* ws = static_cast<char*>(workspace);
    uint32_t* fix_count = reinterpret_cast<uint32_t*>(ws);
    uint32_t* fix_list = reinterpret_cast<uint32_t*>(ws + TC_WS_HEADER);
    const uint32_t fix_cap = (uint32_t)((workspace_bytes - TC_WS_HEADER) / sizeof(uint32_t));
    CUtensorMap map_k, map_p;
    int rc = make_map(&map_k, keys, (uint64_t)N, key_row_stride, TC_ROWS);
    if (rc != SK_OK) return rc;
    rc = make_map(&map_p, planes, TC_N, TC_D, TC_N);
    if (rc != SK_OK) return rc;
    cudaError_t e = cudaMemsetAsync(fix_count, 0, sizeof(uint32_t), st);
    if (e != cudaSuccess) return fail(SK_ERR_CUDA, "sk_hash_keys_tc: cudaMemsetAsync: %s", cudaGetErrorString(e));
    const __nv_bfloat16* kb = static_cast<const __nv_bfloat16*>(keys);
    const __nv_bfloat16* pb = static_cast<const __nv_bfloat16*>(planes);
    const size_t smem = TC_PIPE_SMEM + 1024;
    e = cudaFuncSetAttribute(hash_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(SK_ERR_CUDA, "hash_tc_kernel smem attribute: %s", cudaGetErrorString(e));
    const int64_t tiles = (N + TC_ROWS - 1) / TC_ROWS;
    const unsigned n_cta = (unsigned)(tiles < sm_count() ? tiles : sm_count());     // one persistent CTA per SM
    hash_tc_kernel<<<n_cta, TC_PIPE_THREADS, smem, st>>>(map_k, map_p, pb, N, codes, code_row_stride, dst_row,
                                                        fix_count, fix_list, fix_cap, status);
    rc = check_launch("hash_tc_kernel");
    if (rc != SK_OK) return rc;
    // one listed projection per warp in the common case (about 1.4e-4 of the projections are listed)
    e = launch_after(hash_fix_kernel, dim3(sm_count() * 8), dim3(256), 0, st, kb, key_row_stride, pb, codes, code_row_stride,
                     dst_row, (const uint32_t*)fix_count, (const uint32_t*)fix_list, fix_cap);
    if (e != cudaSuccess) return fail(SK_ERR_CUDA, "hash_fix_kernel: %s", cudaGetErrorString(e));
    dim3 grid(sm_count(), TC_N / 8 / HASH_WARPS);
    e = launch_after(hash_exact_if_overflow_kernel, grid, dim3(HASH_THREADS), 0, st, kb, key_row_stride, pb, N, codes,
                     code_row_stride, dst_row, (const uint32_t*)fix_count, fix_cap);
    if (e != cudaSuccess) return fail(SK_ERR_CUDA, "hash_exact_if_overflow_kernel: %s", cudaGetErrorString(e));
    return check_launch("hash_tc fix-up kernels");
}

}  // namespace sk
