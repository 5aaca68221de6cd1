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
// Streaming multiprocessors of the current device (queried once per device; 148, the B200 count,
// when no device can be asked, e.g. a size query on a machine without a GPU).
int sm_count();

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

__device__ __forceinline__ float order_key_inverse(uint32_t key) {
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

__device__ __forceinline__ int effective_len(int64_t T, const int32_t* T_dev) {
    int64_t t = T;
    if (T_dev != nullptr) {
        int64_t d = (int64_t)__ldcg(T_dev);   // written by a kernel this one may overlap: no cached copy
        t = d < t ? d : t;
    }
    return t < 0 ? 0 : (int)t;
}

// ---------------------------------------------------------------- programmatic dependent launch
// The kernels of one decode step are chained with programmatic stream serialisation: a kernel
// lets its successor start launching right away (launch_dependents) and the successor does its
// set-up that needs no input, then waits (pdl_wait) until the predecessor has completed and its
// writes are visible before it touches anything the predecessor produces.  Both instructions do
// nothing in a kernel that was launched without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Host side: true while sk_decode_step chains its launches (thread-local); launch_chained() adds
// the attribute exactly then.
bool pdl_chain_active();
struct PdlChain {
    PdlChain();
    ~PdlChain();
};
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                  Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    const bool chained = pdl_chain_active();
    cfg.attrs = chained ? &attr : nullptr;
    cfg.numAttrs = chained ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
// Always chained to the kernel before it on the stream (that kernel must be one of this library's,
// executing pdl_launch_dependents).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_after(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                Args... args) {
    PdlChain chain;
    return launch_chained(kern, grid, block, smem, st, args...);
}

// ---------------------------------------------------------------- shared-memory histograms
// Histogram increment by all 32 lanes of a warp.  The lanes that hit the same bin as the first
// active lane are merged into one atomic (score keys cluster, so one dominant bin per warp is the
// common way thousands of atomics end up serialised on one address); the others add on their own.
// Two warp collectives; match.any, which costs a round per distinct value, is kept for
// hist_add_match() below.
__device__ __forceinline__ void warp_hist_add(uint32_t* hist, uint32_t bin, bool active) {
    const unsigned live = __ballot_sync(FULL, active);
    if (live == 0u) return;
    const int leader = __ffs(live) - 1;
    const uint32_t first = __shfl_sync(FULL, bin, leader);
    const unsigned same = __ballot_sync(FULL, active && bin == first);
    if ((int)(threadIdx.x & 31) == leader) atomicAdd(&hist[first], (uint32_t)__popc(same));
    else if (active && bin != first) atomicAdd(&hist[bin], 1u);
}
// Every group of equal bins merged into one atomic: for digits with very few distinct values.
__device__ __forceinline__ void warp_hist_add_match(uint32_t* hist, uint32_t bin, bool active) {
    const unsigned live = __ballot_sync(FULL, active);
    if (active) {
        const unsigned peers = __match_any_sync(live, bin);
        if ((int)(threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&hist[bin], (uint32_t)__popc(peers));
    }
}

// ---------------------------------------------------------------- scorer work split
// How the flat (KV-head group, key) space is cut into CTAs; shared by the scorer, which writes
// per-(row, chunk, warp) candidate runs in its filtering mode, and the select kernel, which
// reads them back.  chunk = CTA index - first CTA of the group.
struct ScorePlan {
    int64_t Tslots;       // slots per group (>= T; padded in the small mode)
    int64_t per_cta;      // slots per CTA, multiple of 32
    int64_t grid;         // CTAs
    int chunks_max;       // upper bound of chunks per group
    int cap_w;            // candidate capacity of one warp's run (filter mode)
    float frac;           // fraction of keys the filter aims to keep
};
constexpr int SC_THREADS = 896;    // 28 warps at 72 registers: measured a little faster than 32 warps at 64 (both scans)
constexpr int SC_WARPS = SC_THREADS / 32;
constexpr int SEL_CAP = 16384;   // candidates the select kernel can hold on chip
constexpr int SC_TAIL = 1024;    // newest keys of a row that the filtering scorer always keeps (see FilterArgs::tail)
constexpr int64_t SC_SWITCH_PAD = 3584;   // empty slots after each group in the flat split, see make_score_plan

inline ScorePlan make_score_plan(int n_groups, int64_t T, int64_t M) {
    ScorePlan p;
    const int n_sm = sm_count();
    const int64_t total = (int64_t)n_groups * T;
    if (total / n_sm >= 16384) {
        // large: split the flat (group, key) space evenly; a CTA may cross one group boundary.
        // Crossing costs a second table load, sample and cut - about what 3.5 K keys cost (measured:
        // 128K context, 91.5 us without padding, 87.2 us with 3-4 K, 89.9 us with 8 K) - so every
        // group ends with that many empty slots: the CTA that crosses gets fewer keys
        p.Tslots = T + SC_SWITCH_PAD;
        const int64_t slots = (int64_t)n_groups * p.Tslots;
        p.per_cta = (slots + n_sm - 1) / n_sm;
        p.per_cta = (p.per_cta + 31) / 32 * 32;
        p.grid = (slots + p.per_cta - 1) / p.per_cta;
        p.chunks_max = (int)((p.Tslots + p.per_cta - 1) / p.per_cta) + 1;
    } else {
        // small: whole CTAs per group, no CTA loads two tables
        int64_t chunks = n_groups >= n_sm ? 1 : n_sm / n_groups;
        const int64_t max_chunks = (T + 1023) / 1024;
        if (chunks > max_chunks) chunks = max_chunks;
        if (chunks > 32) chunks = 32;   // the candidate select handles at most 32 chunks x 32 runs
        p.per_cta = (T + chunks - 1) / chunks;
        p.per_cta = (p.per_cta + 31) / 32 * 32;
        chunks = (T + p.per_cta - 1) / p.per_cta;
        p.Tslots = chunks * p.per_cta;
        p.grid = (int64_t)n_groups * chunks;
        p.chunks_max = (int)chunks;
    }
    const int64_t per_warp = ((p.per_cta + SC_WARPS - 1) / SC_WARPS + 31) / 32 * 32;
    double f = T > 0 ? 3.0 * (double)M / (double)T : 1.0;
    if (f > 1.0) f = 1.0;
    p.frac = (float)f;
    p.cap_w = (int)((int64_t)(4.0 * f * (double)per_warp + 7) / 8 * 8) + 16;
    // room for whole runs of short segments (up to 64 keys per warp), which are kept unfiltered
    if (p.cap_w < 64) p.cap_w = (int)(per_warp < 64 ? per_warp : 64);
    return p;
}
// The filtering scorer pays off (and its buffers stay small) only for small k / T.
inline bool fused_filter_applicable(const ScorePlan& p, int64_t T, int64_t M) {
    return M > 0 && T >= 4096 && 12 * M <= T && 3 * M <= (SEL_CAP * 3) / 4 &&
           p.chunks_max * SC_WARPS <= 1024 && p.cap_w <= 250;   // run lengths are kept in 8 bits
}

// Workspace of the fused scorer + select: [fallback counter | cnt | cut | cand | scratch scores]
struct FusedLayout {
    size_t stats, cnt, cut, cand, tail, scores, total;
    int64_t score_stride;
};
inline size_t sk_up256(size_t x) { return (x + 255) & ~(size_t)255; }
inline FusedLayout make_fused_layout(int64_t rows, const ScorePlan& p, int64_t T) {
    FusedLayout f;
    f.score_stride = (T + 3) / 4 * 4;
    size_t off = 0;
    f.stats = off;  off += 256;
    f.cnt = off;    off += sk_up256((size_t)rows * p.chunks_max * SC_WARPS * sizeof(int32_t));
    f.cut = off;    off += sk_up256((size_t)rows * p.chunks_max * sizeof(float));
    f.cand = off;   off += sk_up256((size_t)rows * p.chunks_max * SC_WARPS * p.cap_w * 8);
    f.tail = off;   off += sk_up256((size_t)rows * SC_TAIL * 8);
    f.scores = off; off += sk_up256((size_t)rows * f.score_stride * sizeof(float));
    f.total = off;
    return f;
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
                     int P, int R, float* q_probs, float* lut, cudaStream_t st, void* lutq = nullptr,
                     float* qpar = nullptr);
int launch_lut_from_probs(const void* q_probs, int dtype, int B, int H, int Hkv, int L, int R,
                          float* lut, cudaStream_t st);
int launch_score(const float* lut, const uint8_t* codes, const uint16_t* v_norm,
                 const uint8_t* allowed, int B, int H, int Hkv, int L, int R, int64_t T,
                 const int32_t* T_dev, int64_t Tcap, float* scores, int64_t score_row_stride,
                 int32_t* status, cudaStream_t st);
// (L, heads per table word, R) combinations the native scorer has a kernel for
bool score_shape_supported(int L, int ht, int R);
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

// Filtering scorer + candidate select (fused path of the decode step)
size_t score_select_workspace_bytes(int B, int H, int Hkv, int L, int64_t T, int64_t M);
int launch_score_filter(const float* lut, const uint8_t* codes, const uint16_t* v_norm, int B, int H,
                        int Hkv, int L, int R, int64_t T, const int32_t* T_dev, int64_t Tcap, int64_t M,
                        void* workspace, int32_t* status, cudaStream_t st, const void* lutq = nullptr,
                        const float* qpar = nullptr);
// The packed (12-bit table) form of the filtering scorer exists for this shape
bool packed_filter_applicable(int H, int Hkv, int L, int R);
int launch_select_candidates(const float* lut, const uint8_t* codes, const uint16_t* v_norm, int B, int H,
                             int Hkv, int L, int R, int64_t T, const int32_t* T_dev, int64_t Tcap, int64_t M,
                             int sink, int window, int sorted, int32_t* list, int64_t list_row_stride,
                             int32_t* list_len, void* workspace, int32_t* status, cudaStream_t st,
                             const float* qpar = nullptr, const float* probs = nullptr);

// One-launch scorer + exact select on thread-block clusters (score_cluster.cu)
int score_select_cluster_size(int B, int H, int Hkv, int L, int R, int64_t T, int64_t M);
int launch_score_select_cluster(const float* lut, const uint8_t* codes, const uint16_t* v_norm, int B, int H,
                                int Hkv, int L, int R, int64_t T, const int32_t* T_dev, int64_t Tcap, int64_t M,
                                int sink, int window, int32_t* list, int64_t list_row_stride, int32_t* list_len,
                                int32_t* status, cudaStream_t st);

// Tensor-core bulk hashing (bf16, head_dim 128, L*P = 256)
size_t hash_keys_tc_workspace_bytes(int64_t N);
int launch_hash_keys_tc(const void* keys, int64_t key_row_stride, const void* planes, int64_t N, uint8_t* codes,
                        int64_t code_row_stride, const int64_t* dst_row, void* workspace, size_t workspace_bytes,
                        int32_t* status, cudaStream_t st);
int launch_cache_rows(const int64_t* input_pos, int B, int S, int Hkv, int64_t Tcap, int64_t* dst_row,
                      int32_t* status, cudaStream_t st);
int launch_kv_copy(const void* k_new, const void* v_new, int kv_dtype, const int64_t* input_pos, void* k_cache,
                   void* v_cache, uint16_t* v_norm, int32_t* prefill_len, int32_t* status, int B, int S,
                   int Hkv, int D, int64_t Tcap, cudaStream_t st);

int launch_rope_split(const void* qkv, int dtype, const void* freqs_cis, int freq_dtype, const int64_t* input_pos,
                      int B, int H, int Hkv, int D, int64_t n_pos, void* q_out, void* k_out, void* v_out,
                      int32_t* status, cudaStream_t st);

// Row-parallel projection fused with the tensor-parallel sum (gemv_allreduce.cu)
size_t gemv_allreduce_buffer_bytes(int world, int max_batch, int N);
int launch_gemv_allreduce(const void* x, const void* W, int64_t w_row_stride, const void* res, void* out, int dtype,
                          int B, int N, int K, void* const* peer_base, int world, int rank, int max_batch,
                          uint32_t* counters, int32_t* status, cudaStream_t st);

int lut_head_tile(int rep);
int launch_decode_prologue(const void* q, const void* k_new, const void* v_new, int dtype,
                           const int64_t* input_pos, const void* planes, int plane_dtype,
                           const float* protos_T, float temperature, void* k_cache, void* v_cache,
                           uint8_t* codes, uint16_t* v_norm, int32_t* prefill_len, int32_t* status,
                           float* lut, int B, int H, int Hkv, int D, int64_t Tcap, int L, int P, int R,
                           cudaStream_t st, bool* launched, void* lutq = nullptr, float* qpar = nullptr,
                           float* q_probs = nullptr);

}  // namespace sk
