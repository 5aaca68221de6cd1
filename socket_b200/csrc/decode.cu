// GQA sparse flash-decode: exact softmax attention of one query per head over the K/V rows
// named by that head's sparse list, read in place from the KV cache.
//
// Work split: grid (splits, B*H), sized so that every CTA is resident at once (two per SM).  A CTA owns a
// contiguous slice of one row's list, each of its 8 warps a contiguous part of that slice.
// A warp streams its rows through a private two-stage ring in shared memory with 16-byte
// asynchronous copies (cp.async): a stage is 8 list entries = 8 K rows + 8 V rows (4 KiB for
// bf16), the next stage is in flight while the current one is consumed, and the list indices
// are fetched 32 at a time one batch ahead, so the gather never waits on an index load.
// Each half-warp then handles one entry at a time (16 lanes x 16 bytes = one 256-byte row),
// with a private online-softmax state (max, sum, 8 output lanes per thread) in fp32 registers.
// The half-warp states are merged through shared memory, the CTA writes one partial
// (max, sum, acc[D]) and takes a ticket; the CTA that draws the last ticket of a row merges
// the row's partials and writes the output.  No CTA ever waits for another one.
#include <mutex>
#include <type_traits>

#include "common.cuh"

// Scratch for sk_sparse_decode_static: lives in the library image, one copy per GPU that
// loads the library, for the life of the process.  In host code this name is only a handle
// for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_static_decode_scratch[SK_SPARSE_DECODE_STATIC_BYTES];

namespace sk {
namespace {

constexpr int DEC_THREADS = 256;
constexpr int DEC_WARPS = DEC_THREADS / 32;
constexpr int DEC_HW = DEC_THREADS / 16;   // half-warps per CTA
constexpr int DEC_G = 8;                   // list entries per stage and warp
constexpr int DEC_STAGES = 2;
constexpr int DEC_D = 128;
constexpr float LOG2E = 1.4426950408889634f;

__host__ __device__ inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

// The ticket counters sit in a region of fixed size at the start of the workspace, whatever
// the shape of the call, so that one zero-initialised buffer can serve calls of any shape:
// every call leaves the counters at zero and nothing else is ever written there.
constexpr int64_t DEC_MAX_ROWS = 65536;
constexpr size_t DEC_TICKET_BYTES = DEC_MAX_ROWS * sizeof(int32_t);

inline int decode_splits(int64_t rows, int64_t max_len) {
    // Few fat CTAs rather than many thin ones: the block scheduler starts roughly 150 CTAs per
    // microsecond, so a grid of 900 small CTAs spends more time ramping up than gathering.
    const int n_sm = sm_count();
    int64_t s = (n_sm * 2) / rows;                      // all CTAs resident: 2 per SM
    // long lists are bandwidth work: a third CTA per SM keeps more rows in flight
    if (s >= 1 && max_len / s > 64 * DEC_WARPS) s = (n_sm * 3) / rows;
    const int64_t cap = (max_len + DEC_G * DEC_WARPS - 1) / (DEC_G * DEC_WARPS);   // at least one stage per warp
    if (s > cap) s = cap;
    if (s < 1) s = 1;
    if (s > 256) s = 256;
    return (int)s;
}

// smem_dst: 32-bit shared-window address (converted once per kernel, not per copy)
__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// eight consecutive elements -> fp32
__device__ __forceinline__ void cvt8(const float* p, float (&d)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *(reinterpret_cast<const float4*>(p) + 1);
    d[0] = a.x; d[1] = a.y; d[2] = a.z; d[3] = a.w;
    d[4] = b.x; d[5] = b.y; d[6] = b.z; d[7] = b.w;
}
__device__ __forceinline__ void cvt8(const __nv_bfloat16* p, float (&d)[8]) {
    const uint4 w = *reinterpret_cast<const uint4*>(p);
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        d[2 * i] = __uint_as_float(u[i] << 16);
        d[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ void cvt8(const __half* p, float (&d)[8]) {
    const uint4 w = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&w);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        d[2 * i] = f.x;
        d[2 * i + 1] = f.y;
    }
}

// Dot product of eight 16-bit elements with fp32 accumulation, no conversion instructions: the
// mixed-precision fma takes both factors in their 16-bit form (the product of two bf16 or fp16
// numbers is exact in fp32, so the result equals converting first), accumulating in the order
// element 0..7.
template <typename KT> struct MixedDot { static constexpr bool ok = false; };
template <> struct MixedDot<__nv_bfloat16> {
    static constexpr bool ok = true;
    static __device__ __forceinline__ float word(uint32_t k, uint32_t q, float d) {
        asm("{\n\t.reg .b16 kl, kh, ql, qh;\n\t"
            "mov.b32 {kl, kh}, %1;\n\t"
            "mov.b32 {ql, qh}, %2;\n\t"
            "fma.rn.f32.bf16 %0, kl, ql, %0;\n\t"
            "fma.rn.f32.bf16 %0, kh, qh, %0;\n\t}"
            : "+f"(d) : "r"(k), "r"(q));
        return d;
    }
};
template <> struct MixedDot<__half> {
    static constexpr bool ok = true;
    static __device__ __forceinline__ float word(uint32_t k, uint32_t q, float d) {
        asm("{\n\t.reg .b16 kl, kh, ql, qh;\n\t"
            "mov.b32 {kl, kh}, %1;\n\t"
            "mov.b32 {ql, qh}, %2;\n\t"
            "fma.rn.f32.f16 %0, kl, ql, %0;\n\t"
            "fma.rn.f32.f16 %0, kh, qh, %0;\n\t}"
            : "+f"(d) : "r"(k), "r"(q));
        return d;
    }
};

template <typename KT> struct DecSmem {
    static constexpr int ROW = DEC_D * (int)sizeof(KT);                 // bytes per K or V row
    static constexpr int STAGE = DEC_G * 2 * ROW;                       // K rows then V rows
    static constexpr int RING = DEC_WARPS * DEC_STAGES * STAGE;
    static constexpr int IDX = DEC_WARPS * DEC_STAGES * DEC_G * 4;
    static constexpr int MERGE = DEC_HW * (DEC_D + 2) * 4;              // aliases the ring
    static constexpr int TOTAL = RING + IDX + 16;
    static_assert(MERGE <= RING, "merge buffers alias the ring");
};

template <typename QT, typename KT>
__global__ void __launch_bounds__(DEC_THREADS)
sparse_decode_kernel(const QT* __restrict__ q, const KT* __restrict__ k_cache,
                     const KT* __restrict__ v_cache, int64_t kv_bs, int64_t kv_hs, int64_t kv_rs,
                     const int32_t* __restrict__ list, int64_t list_rs,
                     const int32_t* __restrict__ list_len, int64_t max_len, QT* __restrict__ out,
                     int H, int Hkv, int64_t T, const int32_t* __restrict__ T_dev, int32_t* tickets,
                     float* ws_ml, float* ws_acc, int32_t* status) {
    using S = DecSmem<KT>;
    constexpr int CPR = S::ROW / 16;                    // 16-byte chunks per row
    constexpr int COPIES = DEC_G * CPR / 32;            // cp.async per lane for the K (or V) rows
    constexpr int EPC = 16 / (int)sizeof(KT);           // elements per chunk
    extern __shared__ __align__(128) char smem[];
    int32_t* sidx_all = reinterpret_cast<int32_t*>(smem + S::RING);
    int* is_last = reinterpret_cast<int*>(smem + S::RING + S::IDX);

    const int splits = gridDim.x, split = blockIdx.x;
    const int row = blockIdx.y;                    // b*H + h
    const int b = row / H, h = row - b * H;
    const int kvh = h / (H / Hkv);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hw = tid >> 4, hw2 = lane >> 4, hl = tid & 15;
    pdl_launch_dependents();

    // the query is an input of the whole step, so it can be fetched before the list exists
    // 16-bit query and keys of one type: the query stays packed and the scale is applied to the
    // finished dot product; otherwise the query is converted and scaled once
    constexpr bool MIXED = MixedDot<KT>::ok && std::is_same<QT, KT>::value;
    float qf[8];
    uint4 qw = make_uint4(0u, 0u, 0u, 0u);
    const float qscale = rsqrtf((float)DEC_D) * LOG2E;
    if constexpr (MIXED) {
        qw = *reinterpret_cast<const uint4*>(q + (size_t)row * DEC_D + hl * 8);
    } else {
        cvt8(q + (size_t)row * DEC_D + hl * 8, qf);
#pragma unroll
        for (int i = 0; i < 8; ++i) qf[i] *= qscale;
    }

    pdl_wait();                               // list, list_len, the live length and the newest K/V row
    // The slice bounds come from max_len alone, so the first two index batches are requested
    // together with the row's length and the live length (the list row has max_len slots; entries
    // at or beyond the length are masked once it has arrived).
    const int chunk = (int)((max_len + splits - 1) / splits);
    const int c0 = split * chunk;
    const int per_warp = ((chunk + DEC_WARPS - 1) / DEC_WARPS + DEC_G - 1) / DEC_G * DEC_G;
    const int w0 = c0 + warp * per_warp;
    const int w1_cap = (int)min((int64_t)min(c0 + chunk, w0 + per_warp), max_len);
    const int32_t* lst = list + (size_t)row * list_rs;
    int raw0 = -1, raw1 = -1;
    if (w0 + lane < w1_cap) raw0 = __ldcg(lst + w0 + lane);
    if (w0 + 32 + lane < w1_cap) raw1 = __ldcg(lst + w0 + 32 + lane);
    int len = __ldcg(list_len + row);         // requested before the live length is consumed
    const int Teff = effective_len(T, T_dev);
    if (len > max_len) len = (int)max_len;
    const int c1 = min(len, c0 + chunk);
    // this warp's part of the slice, a multiple of the stage size
    const int w1 = min(c1, w0 + per_warp);
    const int n_stage = w1 > w0 ? (w1 - w0 + DEC_G - 1) / DEC_G : 0;

    const KT* kb = k_cache + (size_t)b * kv_bs + (size_t)kvh * kv_hs;
    const KT* vb = v_cache + (size_t)b * kv_bs + (size_t)kvh * kv_hs;
    char* ring = smem + (size_t)warp * DEC_STAGES * S::STAGE;
    const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring);
    int32_t* sidx = sidx_all + warp * DEC_STAGES * DEC_G;
    bool bad_index = false;

    // list indices, 32 per batch, validated once
    auto load_batch = [&](int batch) -> int {
        const int e = w0 + batch * 32 + lane;
        int idx = -1;
        if (e < w1) {
            idx = __ldcg(lst + e);
            if (idx >= Teff) {
                bad_index = true;
                idx = -1;
            }
        }
        return idx;
    };
    auto check_batch = [&](int batch, int raw) -> int {   // the same validation for a batch fetched early
        const int e = w0 + batch * 32 + lane;
        if (e >= w1) return -1;
        if (raw >= Teff) {
            bad_index = true;
            return -1;
        }
        return raw;
    };
    int idx0 = check_batch(0, raw0), idx1 = check_batch(1, raw1);

    auto issue = [&](int s) {
        if (s < n_stage) {
            const int reg = ((s >> 2) & 1) ? idx1 : idx0;
            const uint32_t buf = ring_s + (uint32_t)((s % DEC_STAGES) * S::STAGE);
#pragma unroll
            for (int i = 0; i < COPIES; ++i) {
                const int c = lane + 32 * i;
                const int r = c / CPR, ch = c % CPR;
                const int ridx = __shfl_sync(FULL, reg, (s & 3) * DEC_G + r);
                if (ridx >= 0) {
                    const size_t goff = (size_t)ridx * kv_rs + ch * EPC;
                    cp_async16(buf + (uint32_t)(r * S::ROW + ch * 16), kb + goff);
                    cp_async16(buf + (uint32_t)((DEC_G + r) * S::ROW + ch * 16), vb + goff);
                }
            }
            const int mine = __shfl_sync(FULL, reg, (s & 3) * DEC_G + (lane & (DEC_G - 1)));
            if (lane < DEC_G) sidx[(s % DEC_STAGES) * DEC_G + lane] = mine;
            if ((s & 3) == 3) {               // batch fully issued: fetch the one after next
                const int nb = load_batch((s >> 2) + 2);
                if ((s >> 2) & 1) idx1 = nb; else idx0 = nb;
            }
        }
        cp_async_commit();
    };

    float m = -INFINITY, l = 0.f, acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;

#pragma unroll
    for (int s = 0; s < DEC_STAGES; ++s) issue(s);

    for (int s = 0; s < n_stage; ++s) {
        cp_async_wait<DEC_STAGES - 1>();
        __syncwarp();
        const char* buf = ring + (s % DEC_STAGES) * S::STAGE;
        const int32_t* si = sidx + (s % DEC_STAGES) * DEC_G;
        // A stage whose eight entries are all real rows (every stage but a warp's last, unless the
        // list holds an index beyond the live length) runs without per-row tests.
        const bool all_rows = __all_sync(FULL, si[lane & (DEC_G - 1)] >= 0);
        auto attend = [&](auto full_tag) {
            constexpr bool FULL_STAGE = decltype(full_tag)::value;
            static_assert(DEC_G == 8, "the reduction below is written for four rows per half-warp");
            float sc[DEC_G / 2];
            bool ok[DEC_G / 2];
            float d[DEC_G / 2];
#pragma unroll
            for (int j = 0; j < DEC_G / 2; ++j) {
                const int e = 2 * j + hw2;
                ok[j] = FULL_STAGE || si[e] >= 0;
                d[j] = 0.f;
                if (ok[j]) {
                    if constexpr (MIXED) {
                        const uint4 kw = *reinterpret_cast<const uint4*>(reinterpret_cast<const KT*>(buf + e * S::ROW) + hl * 8);
                        d[j] = MixedDot<KT>::word(kw.x, qw.x, d[j]);
                        d[j] = MixedDot<KT>::word(kw.y, qw.y, d[j]);
                        d[j] = MixedDot<KT>::word(kw.z, qw.z, d[j]);
                        d[j] = MixedDot<KT>::word(kw.w, qw.w, d[j]);
                    } else {
                        float kf[8];
                        cvt8(reinterpret_cast<const KT*>(buf + e * S::ROW) + hl * 8, kf);
#pragma unroll
                        for (int i = 0; i < 8; ++i) d[j] = fmaf(qf[i], kf[i], d[j]);
                    }
                }
            }
            // The four partial products of a lane are summed over the 16 lanes of the half-warp as a
            // transposed butterfly: each exchange halves the number of values a lane carries, so the sums
            // cost 5 shuffles instead of 16, and 4 more hand every lane all four results.
            {
                const bool up8 = (hl & 8) != 0, up4 = (hl & 4) != 0;
                float a0 = up8 ? d[2] : d[0], a1 = up8 ? d[3] : d[1];
                const float b0 = up8 ? d[0] : d[2], b1 = up8 ? d[1] : d[3];
                a0 += __shfl_xor_sync(FULL, b0, 8);
                a1 += __shfl_xor_sync(FULL, b1, 8);
                float c = up4 ? a1 : a0;
                const float t = up4 ? a0 : a1;
                c += __shfl_xor_sync(FULL, t, 4);
                c += __shfl_xor_sync(FULL, c, 2);
                c += __shfl_xor_sync(FULL, c, 1);
                if constexpr (MIXED) c *= qscale;
                // lanes 0-3 of the half-warp now hold row 0's sum, 4-7 row 1's, 8-11 row 2's, 12-15 row 3's
                const int base = lane & 16;
#pragma unroll
                for (int j = 0; j < DEC_G / 2; ++j) d[j] = __shfl_sync(FULL, c, base + 4 * j);
            }
            float m_new = m;
#pragma unroll
            for (int j = 0; j < DEC_G / 2; ++j) {
                sc[j] = ok[j] ? d[j] : -INFINITY;
                m_new = fmaxf(m_new, sc[j]);
            }
            if (FULL_STAGE || m_new > -INFINITY) {
                const float resc = exp2f(m - m_new);
                l *= resc;
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] *= resc;
#pragma unroll
                for (int j = 0; j < DEC_G / 2; ++j) {
                    if (ok[j]) {
                        const int e = 2 * j + hw2;
                        const float p = exp2f(sc[j] - m_new);
                        l += p;
                        float vf[8];
                        cvt8(reinterpret_cast<const KT*>(buf + (DEC_G + e) * S::ROW) + hl * 8, vf);
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[i] = fmaf(p, vf[i], acc[i]);
                    }
                }
                m = m_new;
            }
        };
        if (all_rows) attend(std::true_type{});
        else attend(std::false_type{});
        __syncwarp();                      // the stage is free again
        issue(s + DEC_STAGES);
    }
    cp_async_wait<0>();
    if (bad_index && status != nullptr) atomicOr(status, SK_DEV_INDEX_OUT_OF_RANGE);

    // ---- merge the half-warps of this CTA (buffers alias the ring, all copies have landed)
    __syncthreads();
    float* m_s = reinterpret_cast<float*>(smem);
    float* l_s = m_s + DEC_HW;
    float* acc_s = l_s + DEC_HW;           // [DEC_HW][DEC_D]
    if (hl == 0) {
        m_s[hw] = m;
        l_s[hw] = l;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) acc_s[hw * DEC_D + hl * 8 + i] = acc[i];
    __syncthreads();
    if (tid < DEC_D) {                     // one output element per thread
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_HW; ++w) mm = fmaxf(mm, m_s[w]);
        float ll = 0.f, a = 0.f;
        if (mm > -INFINITY) {
#pragma unroll
            for (int w = 0; w < DEC_HW; ++w) {
                const float f = exp2f(m_s[w] - mm);
                ll += l_s[w] * f;
                a += acc_s[w * DEC_D + tid] * f;
            }
        }
        const size_t slot = (size_t)row * splits + split;
        ws_acc[slot * DEC_D + tid] = a;
        if (tid == 0) {
            ws_ml[slot * 2] = mm;
            ws_ml[slot * 2 + 1] = ll;
        }
    }
    // ---- ticket: the last CTA of this row merges the partials
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int t = atomicAdd(&tickets[row], 1);
        *is_last = (t == splits - 1);
    }
    __syncthreads();
    if (!*is_last || tid >= DEC_D) return;
    __threadfence();
    // one pass, all loads independent of each other: running maximum with rescaling, splits in
    // ascending order (so the result does not depend on which CTA came last)
    float mm = -INFINITY, ll = 0.f, a = 0.f;
#pragma unroll 4
    for (int i = 0; i < splits; ++i) {
        const size_t slot = (size_t)row * splits + i;
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(ws_ml + slot * 2));
        const float av = __ldcg(ws_acc + slot * DEC_D + tid);
        if (ml.x > -INFINITY) {
            const float mn = fmaxf(mm, ml.x);
            const float fo = exp2f(mm - mn), fn = exp2f(ml.x - mn);
            ll = ll * fo + ml.y * fn;
            a = a * fo + av * fn;
            mm = mn;
        }
    }
    out[(size_t)row * DEC_D + tid] = from_f32<QT>(ll > 0.f ? a / ll : 0.f);
    if (tid == 0) tickets[row] = 0;   // ready for the next call
}

template <typename QT, typename KT>
int decode_launch(dim3 grid, cudaStream_t st, const void* q, const void* k_cache, const void* v_cache,
                  int64_t kv_bs, int64_t kv_hs, int64_t kv_rs, const int32_t* list, int64_t list_rs,
                  const int32_t* list_len, int64_t max_list_len, void* out, int H, int Hkv, int64_t T,
                  const int32_t* T_dev, int32_t* tickets, float* ws_ml, float* ws_acc, int32_t* status) {
    auto kern = sparse_decode_kernel<QT, KT>;
    constexpr int smem = DecSmem<KT>::TOTAL;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess)
            return fail(SK_ERR_CUDA, "sparse_decode_kernel smem attribute: %s", cudaGetErrorString(e));
    }
    cudaError_t e = launch_chained(kern, grid, dim3(DEC_THREADS), (size_t)smem, st, (const QT*)q, (const KT*)k_cache,
                                   (const KT*)v_cache, kv_bs, kv_hs, kv_rs, list, list_rs, list_len, max_list_len,
                                   (QT*)out, H, Hkv, T, T_dev, tickets, ws_ml, ws_acc, status);
    if (e != cudaSuccess) return fail(SK_ERR_CUDA, "sparse_decode_kernel: %s", cudaGetErrorString(e));
    return check_launch("sparse_decode_kernel");
}

}  // namespace

size_t sparse_decode_workspace_bytes(int B, int H, int D, int64_t max_list_len) {
    const int64_t rows = (int64_t)B * H;
    if (rows <= 0) return DEC_TICKET_BYTES;
    const int splits = decode_splits(rows, max_list_len > 0 ? max_list_len : 1);
    return DEC_TICKET_BYTES + align256((size_t)rows * splits * 2 * sizeof(float)) +
           align256((size_t)rows * splits * D * sizeof(float));
}

int launch_sparse_decode(const void* q, int q_dtype, const void* k_cache, const void* v_cache,
                         int kv_dtype, int64_t kv_bs, int64_t kv_hs, int64_t kv_rs,
                         const int32_t* list, int64_t list_rs, const int32_t* list_len,
                         int64_t max_list_len, void* out, int B, int H, int Hkv, int D, int64_t T,
                         const int32_t* T_dev, void* workspace, size_t workspace_bytes,
                         int32_t* status, cudaStream_t st) {
    const int64_t rows = (int64_t)B * H;
    if (rows == 0) return SK_OK;
    if (D != DEC_D) return fail(SK_ERR_UNSUPPORTED, "sk_sparse_decode: head_dim %d not supported (128)", D);
    if (max_list_len <= 0) return fail(SK_ERR_INVALID_ARGUMENT, "sk_sparse_decode: max_list_len must be positive");
    if (rows >= DEC_MAX_ROWS) return fail(SK_ERR_UNSUPPORTED, "sk_sparse_decode: B*H > 65535");
    const size_t need = sparse_decode_workspace_bytes(B, H, D, max_list_len);
    if (workspace_bytes < need)
        return fail(SK_ERR_WORKSPACE, "sk_sparse_decode: workspace %zu < %zu bytes", workspace_bytes, need);
    const int splits = decode_splits(rows, max_list_len);
    char* ws = static_cast<char*>(workspace);
    int32_t* tickets = reinterpret_cast<int32_t*>(ws);
    float* ws_ml = reinterpret_cast<float*>(ws + DEC_TICKET_BYTES);
    float* ws_acc = reinterpret_cast<float*>(ws + DEC_TICKET_BYTES +
                                             align256((size_t)rows * splits * 2 * sizeof(float)));
    dim3 grid(splits, (unsigned)rows);
#define SK_DEC_LAUNCH(QT, KT)                                                                        \
    return decode_launch<QT, KT>(grid, st, q, k_cache, v_cache, kv_bs, kv_hs, kv_rs, list, list_rs,  \
                                 list_len, max_list_len, out, H, Hkv, T, T_dev, tickets, ws_ml,      \
                                 ws_acc, status)
    if (q_dtype == SK_BF16 && kv_dtype == SK_BF16) SK_DEC_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    if (q_dtype == SK_F32 && kv_dtype == SK_F32) SK_DEC_LAUNCH(float, float);
    if (q_dtype == SK_F16 && kv_dtype == SK_F16) SK_DEC_LAUNCH(__half, __half);
    if (q_dtype == SK_F32 && kv_dtype == SK_BF16) SK_DEC_LAUNCH(float, __nv_bfloat16);
#undef SK_DEC_LAUNCH
    return fail(SK_ERR_UNSUPPORTED, "sk_sparse_decode: unsupported q/kv dtype pair (%d,%d)", q_dtype, kv_dtype);
}

}  // namespace sk

// ------------------------------------------------------------------------------------------
// Allocation-free variant
// ------------------------------------------------------------------------------------------
namespace {
constexpr int MAX_DEVICES = 64;
std::mutex g_static_mu;
void* g_static_ptr[MAX_DEVICES] = {nullptr};

// Device address of the static scratch on the current device, resolved once per device.
int static_scratch_address(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return sk::fail(SK_ERR_CUDA, "sk_sparse_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= MAX_DEVICES)
        return sk::fail(SK_ERR_UNSUPPORTED, "sk_sparse_decode_static: device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (g_static_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_decode_scratch);
        if (e != cudaSuccess || p == nullptr)
            return sk::fail(SK_ERR_CUDA, "sk_sparse_decode_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_static_ptr[dev] = p;
    }
    *out = g_static_ptr[dev];
    return SK_OK;
}
}  // namespace

extern "C" SK_API int sk_sparse_decode_static(
    const void* q, int q_dtype, const void* k_cache, const void* v_cache, int kv_dtype,
    int64_t kv_batch_stride, int64_t kv_head_stride, int64_t kv_row_stride, const int32_t* list,
    int64_t list_row_stride, const int32_t* list_len, int64_t max_list_len, void* out, int B, int H,
    int Hkv, int D, int64_t T, const int32_t* T_dev, int32_t* status, void* stream) {
    using namespace sk;
    if (B < 0 || H <= 0 || Hkv <= 0 || D <= 0 || T < 0 || max_list_len <= 0)
        return fail(SK_ERR_INVALID_ARGUMENT, "sk_sparse_decode_static: sizes must be positive");
    if (B == 0) return SK_OK;
    if (H % Hkv != 0) return fail(SK_ERR_INVALID_ARGUMENT, "sk_sparse_decode_static: H=%d not a multiple of Hkv=%d", H, Hkv);
    if (!q || !k_cache || !v_cache || !list || !list_len || !out)
        return fail(SK_ERR_INVALID_ARGUMENT, "sk_sparse_decode_static: null pointer");
    if (list_row_stride < max_list_len)
        return fail(SK_ERR_INVALID_ARGUMENT, "sk_sparse_decode_static: list_row_stride smaller than max_list_len");
    if ((q_dtype != SK_F32 && q_dtype != SK_BF16 && q_dtype != SK_F16) ||
        (kv_dtype != SK_F32 && kv_dtype != SK_BF16 && kv_dtype != SK_F16))
        return fail(SK_ERR_INVALID_ARGUMENT, "sk_sparse_decode_static: bad dtype");
    const int64_t per16 = kv_dtype == SK_F32 ? 4 : 8;   // elements per 16 bytes
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) |
         reinterpret_cast<uintptr_t>(v_cache)) & 15u)
        return fail(SK_ERR_MISALIGNED, "sk_sparse_decode_static: q, k_cache and v_cache must be 16-byte aligned");
    if (kv_batch_stride % per16 || kv_head_stride % per16 || kv_row_stride % per16)
        return fail(SK_ERR_MISALIGNED, "sk_sparse_decode_static: K/V strides must be multiples of 16 bytes");
    const size_t need = sparse_decode_workspace_bytes(B, H, D, max_list_len);
    if (need > (size_t)SK_SPARSE_DECODE_STATIC_BYTES)
        return fail(SK_ERR_WORKSPACE,
                    "sk_sparse_decode_static: B=%d H=%d max_list_len=%lld needs %zu bytes of scratch, the "
                    "built-in buffer holds %zu; use sk_sparse_decode with a caller-provided workspace",
                    B, H, (long long)max_list_len, need, (size_t)SK_SPARSE_DECODE_STATIC_BYTES);
    void* scratch = nullptr;
    int rc = static_scratch_address(&scratch);
    if (rc != SK_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    // the ticket counters must read zero when the kernel starts, whatever an earlier call left
    cudaError_t e = cudaMemsetAsync(scratch, 0, (size_t)B * H * sizeof(int32_t), st);
    if (e != cudaSuccess) return fail(SK_ERR_CUDA, "sk_sparse_decode_static: cudaMemsetAsync: %s", cudaGetErrorString(e));
    return launch_sparse_decode(q, q_dtype, k_cache, v_cache, kv_dtype, kv_batch_stride, kv_head_stride,
                                kv_row_stride, list, list_row_stride, list_len, max_list_len, out, B, H,
                                Hkv, D, T, T_dev, scratch, (size_t)SK_SPARSE_DECODE_STATIC_BYTES, status, st);
}

