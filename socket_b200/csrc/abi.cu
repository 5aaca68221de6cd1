// extern "C" entry points: argument validation, workspace carving, kernel launches.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace sk {

static thread_local char g_err[512] = "";
static thread_local int g_pdl_depth = 0;

bool pdl_chain_active() {
    static const bool off = getenv("SOCKET_B200_NO_PDL") != nullptr;   // debugging aid: launch the step's kernels unchained
    return g_pdl_depth > 0 && !off;
}
PdlChain::PdlChain() { ++g_pdl_depth; }
PdlChain::~PdlChain() { --g_pdl_depth; }

int fail(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return status;
}

int sm_count() {
    constexpr int MAX_DEV = 64;
    static std::atomic<int> cached[MAX_DEV];
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) {
        cudaGetLastError();   // a size query without a device is not an error of the next launch
        return 148;
    }
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n > 0) return n;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        return 148;
    }
    cached[dev].store(n, std::memory_order_relaxed);
    return n;
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(SK_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return SK_OK;
}

static inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
static inline bool valid_dtype(int d) { return d == SK_F32 || d == SK_BF16 || d == SK_F16; }
static inline size_t esize(int d) { return d == SK_F32 ? 4 : 2; }
static inline size_t up256(size_t x) { return (x + 255) & ~(size_t)255; }

static int64_t list_len_host(int64_t T, int sink, int window, int64_t M) {
    if (T <= 0) return 0;
    int64_t s = sink < 0 ? 0 : (sink > T ? T : sink);
    int64_t w = window < 0 ? 0 : (window > T ? T : window);
    int64_t nb = s;
    if (w > 0) {
        int64_t st = T - w > s ? T - w : s;
        if (st < T) nb += T - st;
    }
    if (nb == 0) nb = 1;
    return nb + (M < T ? (M < 0 ? 0 : M) : T);
}

}  // namespace sk

using namespace sk;

#define SK_REQUIRE(cond, ...)                                          \
    do {                                                               \
        if (!(cond)) return fail(SK_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
    } while (0)
#define SK_ALIGNED(ptr, a, name)                                                         \
    do {                                                                                 \
        if (!aligned(ptr, a)) return fail(SK_ERR_MISALIGNED, name " must be %d-byte aligned", (int)(a)); \
    } while (0)

extern "C" {

int sk_abi_version(void) { return SK_ABI_VERSION; }

const char* sk_status_string(int status) {
    switch (status) {
        case SK_OK: return "ok";
        case SK_ERR_INVALID_ARGUMENT: return "invalid argument";
        case SK_ERR_UNSUPPORTED: return "unsupported shape or dtype";
        case SK_ERR_MISALIGNED: return "misaligned pointer or stride";
        case SK_ERR_WORKSPACE: return "workspace too small";
        case SK_ERR_CUDA: return "CUDA runtime error";
        default: return "unknown status";
    }
}

const char* sk_last_error(void) { return g_err; }

int sk_hash_keys(const void* keys, int key_dtype, int64_t key_row_stride, const void* planes,
                 int plane_dtype, int64_t N, int D, int L, int P, void* codes, int code_bytes,
                 int64_t code_row_stride, void* stream) {
    SK_REQUIRE(N >= 0 && D > 0 && L > 0 && P > 0, "sk_hash_keys: sizes must be positive");
    if (N == 0) return SK_OK;
    SK_REQUIRE(keys && planes && codes, "sk_hash_keys: null pointer");
    SK_REQUIRE(valid_dtype(key_dtype) && valid_dtype(plane_dtype), "sk_hash_keys: bad dtype");
    SK_REQUIRE(code_bytes == 1 || code_bytes == 2, "sk_hash_keys: code_bytes must be 1 or 2");
    SK_REQUIRE(P <= (code_bytes == 1 ? 8 : 15), "sk_hash_keys: P=%d does not fit %d-byte codes", P, code_bytes);
    SK_REQUIRE(key_row_stride >= D && code_row_stride >= L, "sk_hash_keys: row stride smaller than row");
    return launch_hash_keys(keys, key_dtype, key_row_stride, planes, plane_dtype, N, D, L, P, codes,
                            code_bytes, code_row_stride, (cudaStream_t)stream);
}

int sk_kv_append(const void* k_new, const void* v_new, int kv_dtype, const int64_t* input_pos,
                 const void* planes, int plane_dtype, void* k_cache, void* v_cache,
                 uint8_t* codes, uint16_t* v_norm, int32_t* prefill_len, int32_t* status, int B,
                 int S, int Hkv, int D, int64_t Tcap, int L, int P, void* stream) {
    SK_REQUIRE(B >= 0 && S >= 0 && Hkv > 0 && D > 0 && Tcap > 0 && L > 0 && P > 0,
               "sk_kv_append: sizes must be positive");
    if (B == 0 || S == 0) return SK_OK;
    SK_REQUIRE(k_new && v_new && input_pos && planes && k_cache && v_cache && codes && v_norm && prefill_len,
               "sk_kv_append: null pointer");
    SK_REQUIRE(valid_dtype(kv_dtype) && valid_dtype(plane_dtype), "sk_kv_append: bad dtype");
    SK_REQUIRE(P <= 8, "sk_kv_append: the cache stores uint8 codes, P must be <= 8 (got %d)", P);
    return launch_kv_append(k_new, v_new, kv_dtype, input_pos, planes, plane_dtype, k_cache, v_cache,
                            codes, v_norm, prefill_len, status, B, S, Hkv, D, Tcap, L, P,
                            (cudaStream_t)stream);
}

size_t sk_hash_keys_tc_workspace_bytes(int64_t N) { return hash_keys_tc_workspace_bytes(N < 0 ? 0 : N); }

int sk_hash_keys_tc(const void* keys, int64_t key_row_stride, const void* planes, int64_t N, int D, int L, int P,
                    uint8_t* codes, int64_t code_row_stride, const int64_t* dst_row, void* workspace,
                    size_t workspace_bytes, int32_t* status, void* stream) {
    SK_REQUIRE(N >= 0, "sk_hash_keys_tc: N must be non-negative");
    if (N == 0) return SK_OK;
    SK_REQUIRE(keys && planes && codes && workspace, "sk_hash_keys_tc: null pointer");
    if (D != 128 || L * P != 256 || P != 8)
        return fail(SK_ERR_UNSUPPORTED, "sk_hash_keys_tc: needs head_dim 128, P = 8 and L = 32 (got D=%d L=%d P=%d)", D, L, P);
    SK_REQUIRE(key_row_stride >= D && code_row_stride >= L, "sk_hash_keys_tc: row stride smaller than row");
    SK_ALIGNED(keys, 16, "sk_hash_keys_tc: keys");
    SK_ALIGNED(planes, 16, "sk_hash_keys_tc: planes");
    SK_ALIGNED(codes, 16, "sk_hash_keys_tc: codes");
    SK_ALIGNED(workspace, 256, "sk_hash_keys_tc: workspace");
    if (key_row_stride % 8 || code_row_stride % 16)
        return fail(SK_ERR_MISALIGNED, "sk_hash_keys_tc: key rows and code rows must start on 16-byte boundaries");
    return launch_hash_keys_tc(keys, key_row_stride, planes, N, codes, code_row_stride, dst_row, workspace,
                               workspace_bytes, status, (cudaStream_t)stream);
}

size_t sk_kv_append_tc_workspace_bytes(int B, int S, int Hkv) {
    const int64_t N = (int64_t)(B > 0 ? B : 0) * (S > 0 ? S : 0) * (Hkv > 0 ? Hkv : 0);
    return up256((size_t)N * sizeof(int64_t)) + hash_keys_tc_workspace_bytes(N);
}

int sk_kv_append_tc(const void* k_new, const void* v_new, int kv_dtype, const int64_t* input_pos,
                    const void* planes, int plane_dtype, void* k_cache, void* v_cache, uint8_t* codes,
                    uint16_t* v_norm, int32_t* prefill_len, int32_t* status, int B, int S, int Hkv, int D,
                    int64_t Tcap, int L, int P, void* workspace, size_t workspace_bytes, void* stream) {
    SK_REQUIRE(B >= 0 && S >= 0 && Hkv > 0 && Tcap > 0, "sk_kv_append_tc: sizes must be positive");
    if (B == 0 || S == 0) return SK_OK;
    SK_REQUIRE(k_new && v_new && input_pos && planes && k_cache && v_cache && codes && v_norm && prefill_len && workspace,
               "sk_kv_append_tc: null pointer");
    if (kv_dtype != SK_BF16 || plane_dtype != SK_BF16 || D != 128 || L != 32 || P != 8)
        return fail(SK_ERR_UNSUPPORTED, "sk_kv_append_tc: bf16 keys and planes, head_dim 128, L = 32, P = 8 only; "
                                        "use sk_kv_append otherwise");
    SK_ALIGNED(workspace, 256, "sk_kv_append_tc: workspace");
    SK_ALIGNED(k_new, 16, "sk_kv_append_tc: k_new");
    SK_ALIGNED(codes, 16, "sk_kv_append_tc: codes");
    if (workspace_bytes < sk_kv_append_tc_workspace_bytes(B, S, Hkv))
        return fail(SK_ERR_WORKSPACE, "sk_kv_append_tc: workspace too small");
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t N = (int64_t)B * S * Hkv;
    char* ws = static_cast<char*>(workspace);
    int64_t* dst_row = reinterpret_cast<int64_t*>(ws);
    const size_t off = up256((size_t)N * sizeof(int64_t));
    int rc = launch_cache_rows(input_pos, B, S, Hkv, Tcap, dst_row, status, st);
    if (rc != SK_OK) return rc;
    rc = launch_kv_copy(k_new, v_new, kv_dtype, input_pos, k_cache, v_cache, v_norm, prefill_len, nullptr, B, S,
                        Hkv, D, Tcap, st);
    if (rc != SK_OK) return rc;
    return launch_hash_keys_tc(k_new, D, planes, N, codes, L, dst_row, ws + off, workspace_bytes - off, status, st);
}

int sk_rope_split(const void* qkv, int dtype, const void* freqs_cis, int freq_dtype, const int64_t* input_pos,
                  int B, int H, int Hkv, int D, int64_t n_pos, void* q_out, void* k_out, void* v_out,
                  int32_t* status, void* stream) {
    SK_REQUIRE(B >= 0 && H > 0 && Hkv > 0 && D > 0 && n_pos > 0, "sk_rope_split: sizes must be positive");
    if (B == 0) return SK_OK;
    SK_REQUIRE(D % 2 == 0, "sk_rope_split: head_dim %d is odd", D);
    SK_REQUIRE(qkv && freqs_cis && input_pos && q_out && k_out && v_out, "sk_rope_split: null pointer");
    SK_REQUIRE(valid_dtype(dtype) && (freq_dtype == SK_BF16 || freq_dtype == SK_F32), "sk_rope_split: bad dtype");
    SK_REQUIRE(B <= 65535, "sk_rope_split: B > 65535");
    return launch_rope_split(qkv, dtype, freqs_cis, freq_dtype, input_pos, B, H, Hkv, D, n_pos, q_out, k_out, v_out,
                             status, (cudaStream_t)stream);
}

size_t sk_gemv_allreduce_buffer_bytes(int world, int max_batch, int N) {
    if (world < 1 || max_batch < 1 || N < 1) return 0;
    return gemv_allreduce_buffer_bytes(world, max_batch, N);
}

int sk_gemv_allreduce(const void* x, const void* W, int64_t w_row_stride, const void* res, void* out, int dtype,
                      int B, int N, int K, void* const* peer_base, int world, int rank, int max_batch,
                      uint32_t* counters, int32_t* status, void* stream) {
    SK_REQUIRE(B >= 0 && N > 0 && K > 0, "sk_gemv_allreduce: sizes must be positive");
    if (B == 0) return SK_OK;
    SK_REQUIRE(x && W && out && peer_base && counters, "sk_gemv_allreduce: null pointer");
    SK_REQUIRE(w_row_stride >= K, "sk_gemv_allreduce: weight row stride smaller than K");
    SK_ALIGNED(x, 16, "sk_gemv_allreduce: x");
    SK_ALIGNED(W, 16, "sk_gemv_allreduce: W");
    return launch_gemv_allreduce(x, W, w_row_stride, res, out, dtype, B, N, K, peer_base, world, rank, max_batch,
                                 counters, status, (cudaStream_t)stream);
}

int sk_lut_head_tile(int rep) { return rep > 0 ? lut_head_tile(rep) : 0; }

int sk_soft_hash(const void* q, int q_dtype, const void* planes, int plane_dtype,
                 const float* protos_T, float temperature, int B, int H, int Hkv, int D, int L,
                 int P, int R, float* q_probs, float* lut, void* stream) {
    SK_REQUIRE(B >= 0 && H > 0 && Hkv > 0 && D > 0 && L > 0 && P > 0 && R > 0,
               "sk_soft_hash: sizes must be positive");
    if (B == 0) return SK_OK;
    SK_REQUIRE(H % Hkv == 0, "sk_soft_hash: H=%d not a multiple of Hkv=%d", H, Hkv);
    SK_REQUIRE(q && planes && protos_T, "sk_soft_hash: null pointer");
    SK_REQUIRE(q_probs || lut, "sk_soft_hash: no output requested");
    SK_REQUIRE(valid_dtype(q_dtype) && valid_dtype(plane_dtype), "sk_soft_hash: bad dtype");
    SK_REQUIRE(temperature > 0.f, "sk_soft_hash: temperature must be positive");
    return launch_soft_hash(q, q_dtype, planes, plane_dtype, protos_T, temperature, B, H, Hkv, D, L, P,
                            R, q_probs, lut, (cudaStream_t)stream);
}

int sk_lut_from_probs(const void* q_probs, int dtype, int B, int H, int Hkv, int L, int R,
                      float* lut, void* stream) {
    SK_REQUIRE(B >= 0 && H > 0 && Hkv > 0 && L > 0 && R > 0, "sk_lut_from_probs: sizes must be positive");
    if (B == 0) return SK_OK;
    SK_REQUIRE(H % Hkv == 0, "sk_lut_from_probs: H=%d not a multiple of Hkv=%d", H, Hkv);
    SK_REQUIRE(q_probs && lut, "sk_lut_from_probs: null pointer");
    SK_REQUIRE(valid_dtype(dtype), "sk_lut_from_probs: bad dtype");
    return launch_lut_from_probs(q_probs, dtype, B, H, Hkv, L, R, lut, (cudaStream_t)stream);
}

int sk_score(const float* lut, const uint8_t* codes, const uint16_t* v_norm,
             const uint8_t* allowed, int B, int H, int Hkv, int L, int R, int64_t T,
             const int32_t* T_dev, int64_t Tcap, float* scores, int64_t score_row_stride,
             int32_t* status, void* stream) {
    SK_REQUIRE(B >= 0 && H > 0 && Hkv > 0 && L > 0 && R > 0 && T >= 0, "sk_score: sizes must be positive");
    if (B == 0 || T == 0) return SK_OK;
    SK_REQUIRE(H % Hkv == 0, "sk_score: H=%d not a multiple of Hkv=%d", H, Hkv);
    SK_REQUIRE(lut && codes && v_norm && scores, "sk_score: null pointer");
    SK_REQUIRE(T <= Tcap, "sk_score: T=%lld exceeds cache capacity %lld", (long long)T, (long long)Tcap);
    SK_REQUIRE(R <= 256, "sk_score: uint8 codes need R <= 256 (got %d)", R);
    SK_REQUIRE(score_row_stride >= T, "sk_score: score_row_stride smaller than T");
    SK_ALIGNED(lut, 16, "sk_score: lut");
    SK_ALIGNED(codes, 16, "sk_score: codes");
    if (L % 16 != 0) return fail(SK_ERR_UNSUPPORTED, "sk_score: L=%d must be a multiple of 16", L);
    return launch_score(lut, codes, v_norm, allowed, B, H, Hkv, L, R, T, T_dev, Tcap, scores,
                        score_row_stride, status, (cudaStream_t)stream);
}

int sk_score_compat(const float* q_probs, const int16_t* key_buckets, const uint8_t* allowed,
                    const float* v_hist, float* out, int B, int H, int L, int R, int64_t T,
                    void* stream) {
    SK_REQUIRE(B >= 0 && H >= 0 && L > 0 && R > 0 && T >= 0, "sk_score_compat: sizes must be positive");
    if (B == 0 || H == 0 || T == 0) return SK_OK;
    SK_REQUIRE(q_probs && key_buckets && allowed && v_hist && out, "sk_score_compat: null pointer");
    SK_REQUIRE((int64_t)B * H <= 65535, "sk_score_compat: B*H > 65535");
    return launch_score_compat(q_probs, key_buckets, allowed, v_hist, out, B, H, L, R, T,
                               (cudaStream_t)stream);
}

int64_t sk_list_len(int64_t T, int sink, int window, int64_t M) { return list_len_host(T, sink, window, M); }

int sk_select_list(const float* scores, int64_t score_row_stride, const uint8_t* allowed,
                   int64_t rows, int64_t T, const int32_t* T_dev, int64_t M, int sink,
                   int window, int sorted, int32_t* list, int64_t list_row_stride,
                   int32_t* list_len, int32_t* status, void* stream) {
    SK_REQUIRE(rows >= 0 && T >= 0 && M >= 0, "sk_select_list: sizes must be non-negative");
    if (rows == 0) return SK_OK;
    SK_REQUIRE(scores && list && list_len, "sk_select_list: null pointer");
    SK_REQUIRE(score_row_stride >= T, "sk_select_list: score_row_stride smaller than T");
    SK_REQUIRE(list_row_stride >= list_len_host(T, sink, window, M),
               "sk_select_list: list_row_stride %lld smaller than the list length %lld",
               (long long)list_row_stride, (long long)list_len_host(T, sink, window, M));
    return launch_select_list(scores, score_row_stride, allowed, rows, T, T_dev, M, sink, window, sorted,
                              list, list_row_stride, list_len, status, (cudaStream_t)stream);
}

size_t sk_score_select_workspace_bytes(int B, int H, int Hkv, int L, int64_t T, int64_t M) {
    return score_select_workspace_bytes(B, H, Hkv, L, T, M);
}

int sk_score_select_applicable(int B, int H, int Hkv, int L, int R, int64_t T, int64_t M) {
    if (B <= 0 || H <= 0 || Hkv <= 0 || H % Hkv || L != 32 || R > 256 || T <= 0) return 0;
    const int ht = lut_head_tile(H / Hkv);
    const ScorePlan plan = make_score_plan(B * Hkv * ((H / Hkv) / ht), T, M);
    // the scorer addresses the candidate buffer with 32-bit entry indices
    if ((int64_t)B * H * plan.chunks_max * SC_WARPS * plan.cap_w >= (int64_t)1 << 31) return 0;
    return fused_filter_applicable(plan, T, M) ? 1 : 0;
}

int sk_score_select_list(const float* lut, const uint8_t* codes, const uint16_t* v_norm, int B, int H,
                         int Hkv, int L, int R, int64_t T, const int32_t* T_dev, int64_t Tcap, int64_t M,
                         int sink, int window, int32_t* list, int64_t list_row_stride, int32_t* list_len,
                         void* workspace, size_t workspace_bytes, int32_t* status, void* stream) {
    SK_REQUIRE(B >= 0 && H > 0 && Hkv > 0 && L > 0 && R > 0 && T > 0 && M >= 0,
               "sk_score_select_list: sizes must be positive");
    if (B == 0) return SK_OK;
    SK_REQUIRE(H % Hkv == 0, "sk_score_select_list: H=%d not a multiple of Hkv=%d", H, Hkv);
    SK_REQUIRE(lut && codes && v_norm && list && list_len && workspace, "sk_score_select_list: null pointer");
    SK_REQUIRE(T <= Tcap, "sk_score_select_list: T exceeds the cache capacity");
    SK_REQUIRE(list_row_stride >= list_len_host(T, sink, window, M),
               "sk_score_select_list: list_row_stride smaller than the list length");
    SK_ALIGNED(lut, 16, "sk_score_select_list: lut");
    SK_ALIGNED(codes, 16, "sk_score_select_list: codes");
    SK_ALIGNED(workspace, 256, "sk_score_select_list: workspace");
    if (!sk_score_select_applicable(B, H, Hkv, L, R, T, M))
        return fail(SK_ERR_UNSUPPORTED,
                    "sk_score_select_list: shape outside the fused path (needs L=32, R<=256, T>=4096, 12*M<=T, M<=4096); "
                    "use sk_score + sk_select_list");
    if (workspace_bytes < score_select_workspace_bytes(B, H, Hkv, L, T, M))
        return fail(SK_ERR_WORKSPACE, "sk_score_select_list: workspace %zu < %zu bytes", workspace_bytes,
                    score_select_workspace_bytes(B, H, Hkv, L, T, M));
    cudaStream_t st = (cudaStream_t)stream;
    int rc = launch_score_filter(lut, codes, v_norm, B, H, Hkv, L, R, T, T_dev, Tcap, M, workspace, status, st);
    if (rc != SK_OK) return rc;
    return launch_select_candidates(lut, codes, v_norm, B, H, Hkv, L, R, T, T_dev, Tcap, M, sink, window, 0,
                                    list, list_row_stride, list_len, workspace, status, st);
}

int sk_score_select_cluster_size(int B, int H, int Hkv, int L, int R, int64_t T, int64_t M) {
    return score_select_cluster_size(B, H, Hkv, L, R, T, M);
}

int sk_score_select_cluster(const float* lut, const uint8_t* codes, const uint16_t* v_norm, int B, int H,
                            int Hkv, int L, int R, int64_t T, const int32_t* T_dev, int64_t Tcap, int64_t M,
                            int sink, int window, int32_t* list, int64_t list_row_stride, int32_t* list_len,
                            int32_t* status, void* stream) {
    SK_REQUIRE(B >= 0 && H > 0 && Hkv > 0 && L > 0 && R > 0 && T > 0 && M >= 0,
               "sk_score_select_cluster: sizes must be positive");
    if (B == 0) return SK_OK;
    SK_REQUIRE(H % Hkv == 0, "sk_score_select_cluster: H=%d not a multiple of Hkv=%d", H, Hkv);
    SK_REQUIRE(lut && codes && v_norm && list && list_len, "sk_score_select_cluster: null pointer");
    SK_REQUIRE(T <= Tcap, "sk_score_select_cluster: T exceeds the cache capacity");
    SK_REQUIRE(list_row_stride >= list_len_host(T, sink, window, M),
               "sk_score_select_cluster: list_row_stride smaller than the list length");
    SK_ALIGNED(lut, 16, "sk_score_select_cluster: lut");
    SK_ALIGNED(codes, 16, "sk_score_select_cluster: codes");
    if (score_select_cluster_size(B, H, Hkv, L, R, T, M) == 0)
        return fail(SK_ERR_UNSUPPORTED,
                    "sk_score_select_cluster: shape outside the one-launch path (needs L=32, R=256, 4 | H/Hkv, "
                    "T <= 16 * 5120 and every cluster resident); use sk_score_select_list or sk_score + sk_select_list");
    return launch_score_select_cluster(lut, codes, v_norm, B, H, Hkv, L, R, T, T_dev, Tcap, M, sink, window, list,
                                       list_row_stride, list_len, status, (cudaStream_t)stream);
}

int sk_score_filter(const float* lut, const uint8_t* codes, const uint16_t* v_norm, int B, int H, int Hkv,
                    int L, int R, int64_t T, const int32_t* T_dev, int64_t Tcap, int64_t M, void* workspace,
                    size_t workspace_bytes, int32_t* status, void* stream) {
    SK_REQUIRE(lut && codes && v_norm && workspace, "sk_score_filter: null pointer");
    if (!sk_score_select_applicable(B, H, Hkv, L, R, T, M))
        return fail(SK_ERR_UNSUPPORTED, "sk_score_filter: shape outside the fused path");
    SK_REQUIRE(T <= Tcap, "sk_score_filter: T exceeds the cache capacity");
    SK_ALIGNED(lut, 16, "sk_score_filter: lut");
    SK_ALIGNED(codes, 16, "sk_score_filter: codes");
    SK_ALIGNED(workspace, 256, "sk_score_filter: workspace");
    if (workspace_bytes < score_select_workspace_bytes(B, H, Hkv, L, T, M))
        return fail(SK_ERR_WORKSPACE, "sk_score_filter: workspace too small");
    return launch_score_filter(lut, codes, v_norm, B, H, Hkv, L, R, T, T_dev, Tcap, M, workspace, status,
                               (cudaStream_t)stream);
}

int sk_select_candidates(const float* lut, const uint8_t* codes, const uint16_t* v_norm, int B, int H, int Hkv,
                         int L, int R, int64_t T, const int32_t* T_dev, int64_t Tcap, int64_t M, int sink,
                         int window, int32_t* list, int64_t list_row_stride, int32_t* list_len,
                         void* workspace, size_t workspace_bytes, int32_t* status, void* stream) {
    SK_REQUIRE(lut && codes && v_norm && workspace && list && list_len, "sk_select_candidates: null pointer");
    if (!sk_score_select_applicable(B, H, Hkv, L, R, T, M))
        return fail(SK_ERR_UNSUPPORTED, "sk_select_candidates: shape outside the fused path");
    SK_REQUIRE(list_row_stride >= list_len_host(T, sink, window, M),
               "sk_select_candidates: list_row_stride smaller than the list length");
    SK_ALIGNED(workspace, 256, "sk_select_candidates: workspace");
    if (workspace_bytes < score_select_workspace_bytes(B, H, Hkv, L, T, M))
        return fail(SK_ERR_WORKSPACE, "sk_select_candidates: workspace too small");
    return launch_select_candidates(lut, codes, v_norm, B, H, Hkv, L, R, T, T_dev, Tcap, M, sink, window, 0,
                                    list, list_row_stride, list_len, workspace, status, (cudaStream_t)stream);
}

static inline int packed_groups(int B, int H, int Hkv) { return B * Hkv * ((H / Hkv) / 4); }
static inline size_t packed_param_offset(int B, int H, int Hkv) { return (size_t)packed_groups(B, H, Hkv) * 65536; }

// [12-bit tables, 64 KiB per group | K0 per group | q_probs fp32, 32 KiB per (batch, head) row]
static inline size_t packed_probs_offset(int B, int H, int Hkv) {
    return packed_param_offset(B, H, Hkv) + up256((size_t)packed_groups(B, H, Hkv) * sizeof(float));
}
size_t sk_packed_table_bytes(int B, int H, int Hkv) {
    if (B <= 0 || H <= 0 || Hkv <= 0 || H % Hkv || (H / Hkv) % 4) return 0;
    return packed_probs_offset(B, H, Hkv) + (size_t)B * H * 32 * 256 * sizeof(float);
}

int sk_packed_applicable(int B, int H, int Hkv, int L, int R, int64_t T, int64_t M) {
    return sk_score_select_applicable(B, H, Hkv, L, R, T, M) && packed_filter_applicable(H, Hkv, L, R) ? 1 : 0;
}

// The packed scan pays for its extra table and the bracketed select once an SM scans several
// thousand keys.  Measured per layer-step at 128K context, batch 4: 8 KV heads on one GPU (28 K keys
// per SM) 135 vs 150 us, 4 KV heads (14 K) 98 vs 106, 2 KV heads (7 K) 79 vs 82, 1 KV head (3.5 K)
// 68 vs 68; 32K context, batch 1 (1.8 K keys per SM) is faster on the fp32 table.
int sk_packed_preferred(int B, int H, int Hkv, int L, int R, int64_t T, int64_t M) {
    if (!sk_packed_applicable(B, H, Hkv, L, R, T, M)) return 0;
    return (int64_t)packed_groups(B, H, Hkv) * T / sm_count() >= 6144 ? 1 : 0;
}

int sk_soft_hash_packed(const void* q, int q_dtype, const void* planes, int plane_dtype,
                        const float* protos_T, float temperature, int B, int H, int Hkv, int D, int L,
                        int P, int R, float* lut, void* packed, void* stream) {
    SK_REQUIRE(B >= 0 && H > 0 && Hkv > 0 && D > 0 && L > 0 && P > 0 && R > 0,
               "sk_soft_hash_packed: sizes must be positive");
    if (B == 0) return SK_OK;
    SK_REQUIRE(H % Hkv == 0, "sk_soft_hash_packed: H=%d not a multiple of Hkv=%d", H, Hkv);
    SK_REQUIRE(q && planes && protos_T && lut && packed, "sk_soft_hash_packed: null pointer");
    SK_REQUIRE(valid_dtype(q_dtype) && valid_dtype(plane_dtype), "sk_soft_hash_packed: bad dtype");
    SK_REQUIRE(temperature > 0.f, "sk_soft_hash_packed: temperature must be positive");
    if (!packed_filter_applicable(H, Hkv, L, R))
        return fail(SK_ERR_UNSUPPORTED, "sk_soft_hash_packed: needs L=32, R=256 and a multiple of 4 query heads per KV head");
    SK_ALIGNED(lut, 16, "sk_soft_hash_packed: lut");
    SK_ALIGNED(packed, 256, "sk_soft_hash_packed: packed");
    char* pk = static_cast<char*>(packed);
    if (R != 256)
        return fail(SK_ERR_UNSUPPORTED, "sk_soft_hash_packed: R=%d (the packed path keeps 256 buckets per table)", R);
    return launch_soft_hash(q, q_dtype, planes, plane_dtype, protos_T, temperature, B, H, Hkv, D, L, P, R,
                            reinterpret_cast<float*>(pk + packed_probs_offset(B, H, Hkv)), lut,
                            (cudaStream_t)stream, pk, reinterpret_cast<float*>(pk + packed_param_offset(B, H, Hkv)));
}

int sk_score_select_packed(const float* lut, const void* packed, const uint8_t* codes,
                           const uint16_t* v_norm, int B, int H, int Hkv, int L, int R, int64_t T,
                           const int32_t* T_dev, int64_t Tcap, int64_t M, int sink, int window,
                           int32_t* list, int64_t list_row_stride, int32_t* list_len, void* workspace,
                           size_t workspace_bytes, int32_t* status, int stages, void* stream) {
    SK_REQUIRE(B >= 0 && H > 0 && Hkv > 0 && L > 0 && R > 0 && T > 0 && M >= 0,
               "sk_score_select_packed: sizes must be positive");
    if (B == 0) return SK_OK;
    SK_REQUIRE(H % Hkv == 0, "sk_score_select_packed: H=%d not a multiple of Hkv=%d", H, Hkv);
    SK_REQUIRE(lut && packed && codes && v_norm && workspace, "sk_score_select_packed: null pointer");
    SK_REQUIRE((stages & 3) != 0 && (stages & ~3) == 0, "sk_score_select_packed: stages must be 1, 2 or 3");
    SK_REQUIRE(!(stages & 2) || (list && list_len), "sk_score_select_packed: null list");
    SK_REQUIRE(T <= Tcap, "sk_score_select_packed: T exceeds the cache capacity");
    SK_REQUIRE(!(stages & 2) || list_row_stride >= list_len_host(T, sink, window, M),
               "sk_score_select_packed: list_row_stride smaller than the list length");
    SK_ALIGNED(lut, 16, "sk_score_select_packed: lut");
    SK_ALIGNED(packed, 256, "sk_score_select_packed: packed");
    SK_ALIGNED(codes, 32, "sk_score_select_packed: codes");
    SK_ALIGNED(workspace, 256, "sk_score_select_packed: workspace");
    if (!sk_packed_applicable(B, H, Hkv, L, R, T, M))
        return fail(SK_ERR_UNSUPPORTED,
                    "sk_score_select_packed: shape outside the packed path (needs L=32, R=256, 4 | H/Hkv, T>=4096, "
                    "12*M<=T, M<=4096); use sk_score_select_list or sk_score + sk_select_list");
    if (workspace_bytes < score_select_workspace_bytes(B, H, Hkv, L, T, M))
        return fail(SK_ERR_WORKSPACE, "sk_score_select_packed: workspace %zu < %zu bytes", workspace_bytes,
                    score_select_workspace_bytes(B, H, Hkv, L, T, M));
    cudaStream_t st = (cudaStream_t)stream;
    const char* pk = static_cast<const char*>(packed);
    const float* qpar = reinterpret_cast<const float*>(pk + packed_param_offset(B, H, Hkv));
    if (stages & 1) {
        int rc = launch_score_filter(lut, codes, v_norm, B, H, Hkv, L, R, T, T_dev, Tcap, M, workspace, status, st,
                                     pk, qpar);
        if (rc != SK_OK) return rc;
    }
    if (stages & 2)
        return launch_select_candidates(lut, codes, v_norm, B, H, Hkv, L, R, T, T_dev, Tcap, M, sink, window, 0,
                                        list, list_row_stride, list_len, workspace, status, st, qpar,
                                        reinterpret_cast<const float*>(pk + packed_probs_offset(B, H, Hkv)));
    return SK_OK;
}

size_t sk_sparse_decode_workspace_bytes(int B, int H, int D, int64_t max_list_len) {
    return sparse_decode_workspace_bytes(B, H, D, max_list_len);
}

int sk_sparse_decode(const void* q, int q_dtype, const void* k_cache, const void* v_cache,
                     int kv_dtype, int64_t kv_batch_stride, int64_t kv_head_stride,
                     int64_t kv_row_stride, const int32_t* list, int64_t list_row_stride,
                     const int32_t* list_len, int64_t max_list_len, void* out, int B, int H,
                     int Hkv, int D, int64_t T, const int32_t* T_dev, void* workspace,
                     size_t workspace_bytes, int32_t* status, void* stream) {
    SK_REQUIRE(B >= 0 && H > 0 && Hkv > 0 && D > 0 && T >= 0, "sk_sparse_decode: sizes must be positive");
    if (B == 0) return SK_OK;
    SK_REQUIRE(H % Hkv == 0, "sk_sparse_decode: H=%d not a multiple of Hkv=%d", H, Hkv);
    SK_REQUIRE(q && k_cache && v_cache && list && list_len && out && workspace, "sk_sparse_decode: null pointer");
    SK_REQUIRE(valid_dtype(q_dtype) && valid_dtype(kv_dtype), "sk_sparse_decode: bad dtype");
    SK_REQUIRE(list_row_stride >= max_list_len, "sk_sparse_decode: list_row_stride smaller than max_list_len");
    SK_ALIGNED(q, 16, "sk_sparse_decode: q");
    SK_ALIGNED(k_cache, 16, "sk_sparse_decode: k_cache");
    SK_ALIGNED(v_cache, 16, "sk_sparse_decode: v_cache");
    SK_ALIGNED(workspace, 256, "sk_sparse_decode: workspace");
    const int64_t per16 = 16 / (int64_t)esize(kv_dtype);
    if (kv_batch_stride % per16 || kv_head_stride % per16 || kv_row_stride % per16)
        return fail(SK_ERR_MISALIGNED, "sk_sparse_decode: K/V strides must be multiples of 16 bytes");
    return launch_sparse_decode(q, q_dtype, k_cache, v_cache, kv_dtype, kv_batch_stride, kv_head_stride,
                                kv_row_stride, list, list_row_stride, list_len, max_list_len, out, B, H,
                                Hkv, D, T, T_dev, workspace, workspace_bytes, status,
                                (cudaStream_t)stream);
}

/* Workspace of one fused step: [decode scratch | table | scores | list | list_len] */
struct StepLayout {
    size_t dec, lut, scores, list, len, packed, total;
    int64_t score_stride, list_stride;
    bool fused;      // scores region holds the fused scorer+select workspace instead
    bool has_packed; // a packed-table region exists (the packed scan applies to the shape)
};

static StepLayout step_layout(int B, int H, int Hkv, int D, int L, int R, int64_t T_max, int64_t M,
                              int sink, int window) {
    StepLayout s;
    s.fused = sk_score_select_applicable(B, H, Hkv, L, R, T_max, M) != 0;
    s.list_stride = list_len_host(T_max, sink, window, M);
    if (s.list_stride < 1) s.list_stride = 1;
    s.score_stride = (T_max + 3) / 4 * 4;
    size_t off = 0;
    s.dec = off;    off += up256(sparse_decode_workspace_bytes(B, H, D, s.list_stride));
    s.lut = off;    off += up256((size_t)B * H * L * R * sizeof(float));
    s.scores = off;
    off += s.fused ? up256(score_select_workspace_bytes(B, H, Hkv, L, T_max, M))
                   : up256((size_t)B * H * s.score_stride * sizeof(float));
    s.list = off;   off += up256((size_t)B * H * s.list_stride * sizeof(int32_t));
    s.len = off;    off += up256((size_t)B * H * sizeof(int32_t));
    s.has_packed = s.fused && packed_filter_applicable(H, Hkv, L, R);
    s.packed = off;
    if (s.has_packed) off += up256(sk_packed_table_bytes(B, H, Hkv));
    s.total = off;
    return s;
}

size_t sk_decode_step_workspace_bytes(int B, int H, int Hkv, int D, int L, int R, int64_t T_max,
                                      int64_t M, int sink, int window) {
    if (B <= 0 || H <= 0 || Hkv <= 0 || T_max <= 0) return 256;
    return step_layout(B, H, Hkv, D, L, R, T_max, M, sink, window).total;
}

int64_t sk_decode_step_rescored_rows_offset(int B, int H, int Hkv, int D, int L, int R, int64_t T_max,
                                            int64_t M, int sink, int window) {
    if (B <= 0 || H <= 0 || Hkv <= 0 || T_max <= 0) return -1;
    const StepLayout lay = step_layout(B, H, Hkv, D, L, R, T_max, M, sink, window);
    if (!lay.fused) return -1;
    const int ht = lut_head_tile(H / Hkv);
    const ScorePlan plan = make_score_plan(B * Hkv * ((H / Hkv) / ht), T_max, M);
    return (int64_t)(lay.scores + make_fused_layout((int64_t)B * H, plan, T_max).stats);
}

int sk_decode_step(const sk_decode_params* p, void* stream) {
    SK_REQUIRE(p != nullptr, "sk_decode_step: null params");
    SK_REQUIRE(p->B > 0 && p->H > 0 && p->Hkv > 0 && p->D > 0 && p->L > 0 && p->P > 0 && p->R > 0,
               "sk_decode_step: sizes must be positive");
    SK_REQUIRE(p->H % p->Hkv == 0, "sk_decode_step: H not a multiple of Hkv");
    SK_REQUIRE(p->T_max > 0 && p->T_max <= p->Tcap, "sk_decode_step: T_max must be in (0, Tcap]");
    SK_REQUIRE(p->P <= 8 && p->R <= 256, "sk_decode_step: the cache stores uint8 codes (P <= 8, R <= 256)");
    SK_REQUIRE(p->temperature > 0.f, "sk_decode_step: temperature must be positive");
    SK_REQUIRE(p->q && p->planes && p->protos_T && p->k_cache && p->v_cache && p->codes && p->v_norm &&
                   p->prefill_len && p->out && p->workspace,
               "sk_decode_step: null pointer");
    SK_REQUIRE((p->k_new == nullptr) == (p->v_new == nullptr), "sk_decode_step: k_new and v_new go together");
    SK_REQUIRE(p->k_new == nullptr || p->input_pos != nullptr, "sk_decode_step: input_pos missing");
    SK_REQUIRE((p->list == nullptr) == (p->list_len == nullptr), "sk_decode_step: list and list_len go together");
    SK_ALIGNED(p->workspace, 256, "sk_decode_step: workspace");
    // Everything the chain can refuse is refused here, before the first launch: a step either runs
    // whole or leaves the cache untouched.  The kernels use 16-byte loads and asynchronous copies
    // on q, the new rows, the caches, the codes and the output.
    SK_REQUIRE(valid_dtype(p->q_dtype) && valid_dtype(p->kv_dtype) && valid_dtype(p->plane_dtype),
               "sk_decode_step: bad dtype");
    SK_ALIGNED(p->q, 16, "sk_decode_step: q");
    SK_ALIGNED(p->k_cache, 16, "sk_decode_step: k_cache");
    SK_ALIGNED(p->v_cache, 16, "sk_decode_step: v_cache");
    SK_ALIGNED(p->codes, 16, "sk_decode_step: codes");
    SK_ALIGNED(p->out, 16, "sk_decode_step: out");
    SK_ALIGNED(p->v_norm, 2, "sk_decode_step: v_norm");
    SK_ALIGNED(p->prefill_len, 4, "sk_decode_step: prefill_len");
    SK_ALIGNED(p->protos_T, 4, "sk_decode_step: protos_T");
    SK_ALIGNED(p->planes, 16, "sk_decode_step: planes");
    if (p->k_new != nullptr) {
        SK_ALIGNED(p->k_new, 16, "sk_decode_step: k_new");
        SK_ALIGNED(p->v_new, 16, "sk_decode_step: v_new");
        SK_ALIGNED(p->input_pos, 8, "sk_decode_step: input_pos");
    }
    if (p->list != nullptr) {
        SK_ALIGNED(p->list, 4, "sk_decode_step: list");
        SK_ALIGNED(p->list_len, 4, "sk_decode_step: list_len");
    }
    if (p->D != 128)
        return fail(SK_ERR_UNSUPPORTED, "sk_decode_step: head_dim %d not supported (128)", p->D);
    if (!((p->q_dtype == p->kv_dtype) || (p->q_dtype == SK_F32 && p->kv_dtype == SK_BF16)))
        return fail(SK_ERR_UNSUPPORTED, "sk_decode_step: unsupported q/kv dtype pair (%d,%d)", p->q_dtype, p->kv_dtype);
    if (!score_shape_supported(p->L, lut_head_tile(p->H / p->Hkv), p->R))
        return fail(SK_ERR_UNSUPPORTED, "sk_decode_step: L=%d with %d query heads per KV head (R=%d) not supported "
                                        "by the scorer", p->L, p->H / p->Hkv, p->R);
    SK_REQUIRE((int64_t)p->B * p->H < 65535, "sk_decode_step: B*H must stay below 65535");
    const StepLayout lay = step_layout(p->B, p->H, p->Hkv, p->D, p->L, p->R, p->T_max, p->M, p->sink, p->window);
    if (p->workspace_bytes < lay.total)
        return fail(SK_ERR_WORKSPACE, "sk_decode_step: workspace %zu < %zu bytes", p->workspace_bytes, lay.total);
    SK_REQUIRE(p->list == nullptr || p->list_row_stride >= lay.list_stride,
               "sk_decode_step: list_row_stride smaller than the list length %lld", (long long)lay.list_stride);
    SK_REQUIRE(p->select_path >= SK_SELECT_AUTO && p->select_path <= SK_SELECT_FILTER_PACKED,
               "sk_decode_step: select_path %d is not an sk_select_path", p->select_path);
    const bool can_cluster = score_select_cluster_size(p->B, p->H, p->Hkv, p->L, p->R, p->T_max, p->M) != 0;
    int path = p->select_path;
    if (path == SK_SELECT_AUTO) path = lay.fused ? SK_SELECT_FILTER : (can_cluster ? SK_SELECT_CLUSTER : SK_SELECT_TWO_LAUNCH);
    if (path == SK_SELECT_CLUSTER && !can_cluster)
        return fail(SK_ERR_UNSUPPORTED, "sk_decode_step: shape outside the one-launch scorer + select");
    if (path == SK_SELECT_FILTER_PACKED && !(lay.has_packed && aligned(p->codes, 32)))
        return fail(SK_ERR_UNSUPPORTED, "sk_decode_step: shape outside the packed scorer (L=32, R=256, 4 | H/Hkv, "
                                        "32-byte aligned codes)");
    if ((path == SK_SELECT_FILTER || path == SK_SELECT_FILTER_F32 || path == SK_SELECT_FILTER_PACKED) && !lay.fused)
        return fail(SK_ERR_UNSUPPORTED, "sk_decode_step: shape outside the filtering scorer + candidate select");
    if (path == SK_SELECT_TWO_LAUNCH && lay.fused)
        return fail(SK_ERR_UNSUPPORTED, "sk_decode_step: the workspace of this shape holds no score matrix; "
                                        "use SK_SELECT_FILTER or SK_SELECT_AUTO");
    cudaStream_t st = (cudaStream_t)stream;
    char* ws = static_cast<char*>(p->workspace);
    float* lut = reinterpret_cast<float*>(ws + lay.lut);
    float* scores = reinterpret_cast<float*>(ws + lay.scores);
    int32_t* list = p->list ? p->list : reinterpret_cast<int32_t*>(ws + lay.list);
    int32_t* list_len = p->list ? p->list_len : reinterpret_cast<int32_t*>(ws + lay.len);
    const int64_t list_stride = p->list ? p->list_row_stride : lay.list_stride;
    // the packed scan needs 32-byte aligned code rows (one 256-bit load per key)
    const bool use_packed = path == SK_SELECT_FILTER_PACKED ||
                            (path == SK_SELECT_FILTER && lay.has_packed && aligned(p->codes, 32) &&
                             sk_packed_preferred(p->B, p->H, p->Hkv, p->L, p->R, p->T_max, p->M));
    char* pk = use_packed ? ws + lay.packed : nullptr;
    float* qpar = use_packed ? reinterpret_cast<float*>(pk + packed_param_offset(p->B, p->H, p->Hkv)) : nullptr;
    float* probs = use_packed ? reinterpret_cast<float*>(pk + packed_probs_offset(p->B, p->H, p->Hkv)) : nullptr;
    // the packed scan and its select work from the packed table and the probabilities: the fp32 scorer
    // table (4 MB of scattered 16-byte stores at 128 rows) is not written
    if (use_packed) lut = nullptr;
    int rc;
    bool fused = false;
    if (p->k_new != nullptr && p->q_dtype == p->kv_dtype) {
        // append + soft hash in one launch
        rc = launch_decode_prologue(p->q, p->k_new, p->v_new, p->kv_dtype, p->input_pos, p->planes,
                                    p->plane_dtype, p->protos_T, p->temperature, p->k_cache, p->v_cache,
                                    p->codes, p->v_norm, p->prefill_len, p->status, lut, p->B, p->H, p->Hkv,
                                    p->D, p->Tcap, p->L, p->P, p->R, st, &fused, pk, qpar, probs);
        if (rc != SK_OK) return rc;
    }
    if (!fused) {
        if (p->k_new != nullptr) {
            rc = sk_kv_append(p->k_new, p->v_new, p->kv_dtype, p->input_pos, p->planes, p->plane_dtype,
                              p->k_cache, p->v_cache, p->codes, p->v_norm, p->prefill_len, p->status, p->B,
                              1, p->Hkv, p->D, p->Tcap, p->L, p->P, stream);
            if (rc != SK_OK) return rc;
        }
        rc = launch_soft_hash(p->q, p->q_dtype, p->planes, p->plane_dtype, p->protos_T, p->temperature, p->B,
                              p->H, p->Hkv, p->D, p->L, p->P, p->R, probs, lut, st, pk, qpar);
        if (rc != SK_OK) return rc;
    }
    // from here on every launch may start while its predecessor drains (see pdl_wait in the kernels)
    PdlChain chain;
    if (path == SK_SELECT_CLUSTER) {
        // one launch: scores stay in shared memory, select across the cluster
        rc = launch_score_select_cluster(lut, p->codes, p->v_norm, p->B, p->H, p->Hkv, p->L, p->R, p->T_max,
                                         p->prefill_len, p->Tcap, p->M, p->sink, p->window, list, list_stride,
                                         list_len, p->status, st);
        if (rc != SK_OK) return rc;
    } else if (path == SK_SELECT_FILTER || path == SK_SELECT_FILTER_F32 || path == SK_SELECT_FILTER_PACKED) {
        // filtering scorer + candidate select: no score array is written or re-read
        rc = launch_score_filter(lut, p->codes, p->v_norm, p->B, p->H, p->Hkv, p->L, p->R, p->T_max,
                                 p->prefill_len, p->Tcap, p->M, ws + lay.scores, p->status, st, pk, qpar);
        if (rc != SK_OK) return rc;
        rc = launch_select_candidates(lut, p->codes, p->v_norm, p->B, p->H, p->Hkv, p->L, p->R, p->T_max,
                                      p->prefill_len, p->Tcap, p->M, p->sink, p->window, 0, list, list_stride,
                                      list_len, ws + lay.scores, p->status, st, qpar, probs);
        if (rc != SK_OK) return rc;
    } else {
        rc = sk_score(lut, p->codes, p->v_norm, nullptr, p->B, p->H, p->Hkv, p->L, p->R, p->T_max,
                      p->prefill_len, p->Tcap, scores, lay.score_stride, p->status, stream);
        if (rc != SK_OK) return rc;
        rc = sk_select_list(scores, lay.score_stride, nullptr, (int64_t)p->B * p->H, p->T_max, p->prefill_len,
                            p->M, p->sink, p->window, 0, list, list_stride, list_len, p->status, stream);
        if (rc != SK_OK) return rc;
    }
    const int64_t kv_hs = p->Tcap * p->D;
    rc = launch_sparse_decode(p->q, p->q_dtype, p->k_cache, p->v_cache, p->kv_dtype, kv_hs * p->Hkv, kv_hs,
                              p->D, list, list_stride, list_len, lay.list_stride, p->out, p->B, p->H,
                              p->Hkv, p->D, p->T_max, p->prefill_len, ws + lay.dec,
                              up256(sparse_decode_workspace_bytes(p->B, p->H, p->D, lay.list_stride)),
                              p->status, st);
    return rc;
}

}  // extern "C"
