// GQA sparse flash-decode: exact softmax attention of one query per head over the K/V rows
// named by that head's sparse list, read in place from the KV cache.
//
// Work split: grid (splits, B*H).  A CTA owns a contiguous slice of one row's list; each of
// its 8 half-warps streams whole K and V rows (16 lanes x 16 bytes = one 256-byte bf16 row
// per load instruction), four list entries at a time so that 8 independent 16-byte loads per
// lane are in flight, and keeps a private online-softmax state (max, sum, 8 output lanes per
// thread) in registers with fp32 accumulation.  The half-warp states are merged through
// shared memory, the CTA writes one partial (max, sum, acc[D]) and takes a ticket; the CTA
// that draws the last ticket of a row merges the row's partials and writes the output.  No
// CTA ever waits for another one.
#include "common.cuh"

namespace sk {
namespace {

constexpr int DEC_THREADS = 128;
constexpr int DEC_HW = DEC_THREADS / 16;   // half-warps per CTA
constexpr int DEC_U = 4;                   // list entries per half-warp per iteration
constexpr int DEC_D = 128;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void load8(const float* p, float (&d)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p));
    const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    d[0] = a.x; d[1] = a.y; d[2] = a.z; d[3] = a.w;
    d[4] = b.x; d[5] = b.y; d[6] = b.z; d[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&d)[8]) {
    const uint4 w = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        d[2 * i] = __uint_as_float(u[i] << 16);
        d[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ void load8(const __half* p, float (&d)[8]) {
    const uint4 w = __ldg(reinterpret_cast<const uint4*>(p));
    const __half2* h = reinterpret_cast<const __half2*>(&w);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        d[2 * i] = f.x;
        d[2 * i + 1] = f.y;
    }
}

struct DecodeWs {
    int32_t* tickets;   // [rows]
    float* ml;          // [rows][splits][2]
    float* acc;         // [rows][splits][D]
};

__host__ __device__ inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

// The ticket counters sit in a region of fixed size at the start of the workspace, whatever
// the shape of the call, so that one zero-initialised buffer can serve calls of any shape:
// every call leaves the counters at zero and nothing else is ever written there.
constexpr int64_t DEC_MAX_ROWS = 65536;
constexpr size_t DEC_TICKET_BYTES = DEC_MAX_ROWS * sizeof(int32_t);

inline int decode_splits(int64_t rows, int64_t max_len) {
    int64_t s = (148 * 6 + rows - 1) / rows;
    const int64_t cap = (max_len + 31) / 32;
    if (s > cap) s = cap;
    if (s < 1) s = 1;
    if (s > 256) s = 256;
    return (int)s;
}

template <typename QT, typename KT>
__global__ void __launch_bounds__(DEC_THREADS)
sparse_decode_kernel(const QT* __restrict__ q, const KT* __restrict__ k_cache,
                     const KT* __restrict__ v_cache, int64_t kv_bs, int64_t kv_hs, int64_t kv_rs,
                     const int32_t* __restrict__ list, int64_t list_rs,
                     const int32_t* __restrict__ list_len, int64_t max_len, QT* __restrict__ out,
                     int H, int Hkv, int64_t T, const int32_t* __restrict__ T_dev, int32_t* tickets,
                     float* ws_ml, float* ws_acc, int32_t* status) {
    __shared__ float m_s[DEC_HW], l_s[DEC_HW];
    __shared__ float acc_s[DEC_HW][DEC_D];
    __shared__ int is_last;

    const int splits = gridDim.x, split = blockIdx.x;
    const int row = blockIdx.y;                    // b*H + h
    const int b = row / H, h = row - b * H;
    const int kvh = h / (H / Hkv);
    const int tid = threadIdx.x, hw = tid >> 4, hl = tid & 15;
    const int Teff = effective_len(T, T_dev);

    int len = list_len[row];
    if (len > max_len) len = (int)max_len;
    const int chunk = (int)((max_len + splits - 1) / splits);
    const int c0 = split * chunk;
    const int c1 = min(len, c0 + chunk);

    float qf[8];
    load8(q + (size_t)row * DEC_D + hl * 8, qf);
    const float qscale = rsqrtf((float)DEC_D) * LOG2E;
#pragma unroll
    for (int i = 0; i < 8; ++i) qf[i] *= qscale;

    const KT* kb = k_cache + (size_t)b * kv_bs + (size_t)kvh * kv_hs + hl * 8;
    const KT* vb = v_cache + (size_t)b * kv_bs + (size_t)kvh * kv_hs + hl * 8;
    const int32_t* lst = list + (size_t)row * list_rs;

    float m = -INFINITY, l = 0.f, acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    bool bad_index = false;

    // trip count is uniform over the CTA: the shuffles below need whole warps
    const int n_iter = c1 > c0 ? (c1 - c0 + DEC_HW * DEC_U - 1) / (DEC_HW * DEC_U) : 0;
    for (int it = 0; it < n_iter; ++it) {
        const int e0 = c0 + (it * DEC_HW + hw) * DEC_U;
        int idx[DEC_U];
        float kf[DEC_U][8], vf[DEC_U][8];
#pragma unroll
        for (int u = 0; u < DEC_U; ++u) {
            idx[u] = (e0 + u < c1) ? __ldg(lst + e0 + u) : -1;
            if (idx[u] >= Teff) {
                bad_index = true;
                idx[u] = -1;
            }
        }
#pragma unroll
        for (int u = 0; u < DEC_U; ++u) {
            if (idx[u] >= 0) {
                load8(kb + (size_t)idx[u] * kv_rs, kf[u]);
                load8(vb + (size_t)idx[u] * kv_rs, vf[u]);
            }
        }
        float s[DEC_U];
        float m_new = m;
#pragma unroll
        for (int u = 0; u < DEC_U; ++u) {
            float d = 0.f;
            if (idx[u] >= 0) {
#pragma unroll
                for (int i = 0; i < 8; ++i) d = fmaf(qf[i], kf[u][i], d);
            }
            d += __shfl_xor_sync(FULL, d, 8);
            d += __shfl_xor_sync(FULL, d, 4);
            d += __shfl_xor_sync(FULL, d, 2);
            d += __shfl_xor_sync(FULL, d, 1);
            s[u] = idx[u] >= 0 ? d : -INFINITY;
            m_new = fmaxf(m_new, s[u]);
        }
        if (m_new > -INFINITY) {
            const float resc = exp2f(m - m_new);
            l *= resc;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] *= resc;
#pragma unroll
            for (int u = 0; u < DEC_U; ++u) {
                if (idx[u] >= 0) {
                    const float p = exp2f(s[u] - m_new);
                    l += p;
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[i] = fmaf(p, vf[u][i], acc[i]);
                }
            }
            m = m_new;
        }
    }
    if (bad_index && status != nullptr) atomicOr(status, SK_DEV_INDEX_OUT_OF_RANGE);

    // ---- merge the half-warps of this CTA
    if (hl == 0) {
        m_s[hw] = m;
        l_s[hw] = l;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) acc_s[hw][hl * 8 + i] = acc[i];
    __syncthreads();
    {
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_HW; ++w) mm = fmaxf(mm, m_s[w]);
        float ll = 0.f, a = 0.f;
        if (mm > -INFINITY) {
#pragma unroll
            for (int w = 0; w < DEC_HW; ++w) {
                const float f = exp2f(m_s[w] - mm);
                ll += l_s[w] * f;
                a += acc_s[w][tid] * f;
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
        is_last = (t == splits - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    float mm = -INFINITY;
    for (int sidx = 0; sidx < splits; ++sidx)
        mm = fmaxf(mm, __ldcg(ws_ml + ((size_t)row * splits + sidx) * 2));
    float ll = 0.f, a = 0.f;
    if (mm > -INFINITY) {
        for (int sidx = 0; sidx < splits; ++sidx) {
            const size_t slot = (size_t)row * splits + sidx;
            const float f = exp2f(__ldcg(ws_ml + slot * 2) - mm);
            ll += __ldcg(ws_ml + slot * 2 + 1) * f;
            a += __ldcg(ws_acc + slot * DEC_D + tid) * f;
        }
    }
    out[(size_t)row * DEC_D + tid] = from_f32<QT>(ll > 0.f ? a / ll : 0.f);
    if (tid == 0) tickets[row] = 0;   // ready for the next call
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
#define SK_DEC_LAUNCH(QT, KT)                                                                       \
    sparse_decode_kernel<QT, KT><<<grid, DEC_THREADS, 0, st>>>(                                     \
        (const QT*)q, (const KT*)k_cache, (const KT*)v_cache, kv_bs, kv_hs, kv_rs, list, list_rs,   \
        list_len, max_list_len, (QT*)out, H, Hkv, T, T_dev, tickets, ws_ml, ws_acc, status)
    if (q_dtype == SK_BF16 && kv_dtype == SK_BF16) SK_DEC_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (q_dtype == SK_F32 && kv_dtype == SK_F32) SK_DEC_LAUNCH(float, float);
    else if (q_dtype == SK_F16 && kv_dtype == SK_F16) SK_DEC_LAUNCH(__half, __half);
    else if (q_dtype == SK_F32 && kv_dtype == SK_BF16) SK_DEC_LAUNCH(float, __nv_bfloat16);
    else return fail(SK_ERR_UNSUPPORTED, "sk_sparse_decode: unsupported q/kv dtype pair (%d,%d)", q_dtype, kv_dtype);
#undef SK_DEC_LAUNCH
    return check_launch("sparse_decode_kernel");
}

}  // namespace sk
