/* socket_b200 — C ABI of the B200-native SOCKET sparse-attention decode path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as an
 * opaque pointer, i.e. a cudaStream_t), enqueues its kernels on that stream and returns
 * without synchronising.  Nothing here allocates device memory: outputs and scratch are
 * provided by the caller (sizes from the *_workspace_bytes queries).
 *
 * Return value: 0 on success, a negative sk_status on an argument / launch error detected
 * on the host (nothing was enqueued for argument errors).  sk_last_error() returns a
 * thread-local description of the most recent failure.  Conditions that only the device
 * can see (a cache position out of range, a list index out of range, a wait that ran out)
 * are reported through the optional `status` word: a device int32 the kernels OR flags
 * into (SK_DEV_*); the offending access is skipped, the context stays usable.
 *
 * File:line citations name the reference interface (amarka8/SOCKET, paths relative to the
 * reference root) each entry point replaces.
 */
#ifndef SOCKET_B200_H_
#define SOCKET_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SK_ABI_VERSION 1

#if defined(__GNUC__)
#define SK_API __attribute__((visibility("default")))
#else
#define SK_API
#endif

/* element types of q / K / V / planes */
enum { SK_F32 = 0, SK_BF16 = 1, SK_F16 = 2 };

enum sk_status {
    SK_OK = 0,
    SK_ERR_INVALID_ARGUMENT = -1, /* null pointer, non-positive size, inconsistent shapes   */
    SK_ERR_UNSUPPORTED = -2,      /* a shape / dtype this build has no kernel for            */
    SK_ERR_MISALIGNED = -3,       /* pointer or stride not aligned as the kernel requires    */
    SK_ERR_WORKSPACE = -4,        /* workspace too small                                     */
    SK_ERR_CUDA = -5              /* the CUDA runtime reported a launch / configuration error */
};

/* flags OR-ed into the device status word */
#define SK_DEV_POS_OUT_OF_RANGE 1   /* sk_kv_append: input_pos outside [0, Tcap)           */
#define SK_DEV_INDEX_OUT_OF_RANGE 2 /* sk_sparse_decode: list entry >= T (entry skipped)   */
#define SK_DEV_WAIT_TIMEOUT 4       /* a bounded wait on an asynchronous copy gave up      */

SK_API int sk_abi_version(void);
SK_API const char* sk_status_string(int status);
SK_API const char* sk_last_error(void);

/* ------------------------------------------------------------------------------------
 * Key hashing.  Replaces Attention.hard_hash_keys + pack_bits (GPT-FAST/model.py:403-413):
 * code[n,l] = sum_p [<keys[n,:], planes[l,p,:]> >= 0] << (P-1-p).  The sign is decided on
 * the exact dot product (fp64 accumulation), so it does not depend on summation order.
 *   keys    [N, D] rows, `key_row_stride` elements apart
 *   planes  [L, P, D] contiguous
 *   codes   [N, L], `code_row_stride` elements apart; uint8 when code_bytes == 1 (P <= 8),
 *           int16 when code_bytes == 2 (P <= 15, the reference's dtype)
 * ---------------------------------------------------------------------------------- */
SK_API int sk_hash_keys(const void* keys, int key_dtype, int64_t key_row_stride, const void* planes,
                 int plane_dtype, int64_t N, int D, int L, int P, void* codes, int code_bytes,
                 int64_t code_row_stride, void* stream);

/* ------------------------------------------------------------------------------------
 * KV-cache append with hashing.  Replaces, in one launch, hard_hash_keys + the v-norm +
 * KVCache.update (GPT-FAST/model.py:449-451, 187-229) for S new tokens:
 *   k_new, v_new [B, S, Hkv, D] contiguous (kv_dtype)
 *   input_pos    [S] int64, device: cache position of each new token
 *   k_cache, v_cache [B, Hkv, Tcap, D]; codes [B, Hkv, Tcap, L] uint8;
 *   v_norm [B, Hkv, Tcap] fp16 (||v||_2, model.py:450)
 *   prefill_len  device int32, updated to max(prefill_len, max(input_pos)+1) (model.py:228)
 *   status       device int32 or NULL; a position outside [0,Tcap) sets
 *                SK_DEV_POS_OUT_OF_RANGE and that token is not written (the reference
 *                raises from a host-side check, model.py:211-217)
 * ---------------------------------------------------------------------------------- */
SK_API int sk_kv_append(const void* k_new, const void* v_new, int kv_dtype, const int64_t* input_pos,
                 const void* planes, int plane_dtype, void* k_cache, void* v_cache,
                 uint8_t* codes, uint16_t* v_norm, int32_t* prefill_len, int32_t* status, int B,
                 int S, int Hkv, int D, int64_t Tcap, int L, int P, void* stream);

/* ------------------------------------------------------------------------------------
 * The same hashing for bulk (prefill-sized) inputs on the tensor cores: the [N,128]x[128,256]
 * projection runs as tcgen05 MMAs fed by TMA; projections too close to zero for the fp32
 * accumulator to decide are decided again exactly, so the codes equal sk_hash_keys' bit for
 * bit.  bf16 keys and planes, D = 128, L = 32, P = 8; codes are uint8.
 *   dst_row    NULL, or [N] int64: row n's codes go to codes + dst_row[n] * code_row_stride
 *              (negative = skip the row); lets a [B,S,Hkv] batch land in a [B,Hkv,Tcap] cache
 *   workspace  sk_hash_keys_tc_workspace_bytes(N) bytes, 256-byte aligned
 * sk_kv_append_tc = sk_kv_append for many tokens at once (prefill) on that path.
 * Replaces the same reference code as sk_hash_keys / sk_kv_append.
 * ---------------------------------------------------------------------------------- */
SK_API size_t sk_hash_keys_tc_workspace_bytes(int64_t N);
SK_API int sk_hash_keys_tc(const void* keys, int64_t key_row_stride, const void* planes, int64_t N, int D, int L, int P,
                    uint8_t* codes, int64_t code_row_stride, const int64_t* dst_row, void* workspace,
                    size_t workspace_bytes, int32_t* status, void* stream);
SK_API size_t sk_kv_append_tc_workspace_bytes(int B, int S, int Hkv);
SK_API int sk_kv_append_tc(const void* k_new, const void* v_new, int kv_dtype, const int64_t* input_pos,
                    const void* planes, int plane_dtype, void* k_cache, void* v_cache, uint8_t* codes,
                    uint16_t* v_norm, int32_t* prefill_len, int32_t* status, int B, int S, int Hkv, int D,
                    int64_t Tcap, int L, int P, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------
 * Front end of a decode step: split one token's fused QKV projection [B, (H + 2 Hkv) * D] into
 * q [B,H,D], k [B,1,Hkv,D], v [B,1,Hkv,D] and apply the rotary embedding of position
 * input_pos[0] (device) to q and k.  Replaces the split + two apply_rotary_emb calls of
 * Attention.sparse_forward (GPT-FAST/model.py:436-445, 626-637): same fp32 arithmetic, one launch.
 * freqs_cis: [n_pos, D/2, 2] (cos, sin), bf16 as the reference stores it or fp32.  A position
 * outside [0, n_pos) writes nothing and sets SK_DEV_POS_OUT_OF_RANGE.
 * ---------------------------------------------------------------------------------- */
SK_API int sk_rope_split(const void* qkv, int dtype, const void* freqs_cis, int freq_dtype,
                  const int64_t* input_pos, int B, int H, int Hkv, int D, int64_t n_pos, void* q_out,
                  void* k_out, void* v_out, int32_t* status, void* stream);

/* ------------------------------------------------------------------------------------
 * Tensor-parallel glue of a decode step: the row-parallel projection that follows the attention
 * (`wo`) or closes the feed-forward (`w2`) fused with the sum over the ranks,
 *     out[b,:] = res[b,:] + sum_r x_r[b,:] . W_r^T,      B <= 8 rows, bf16 / fp16.
 * Replaces the GEMM + NCCL all-reduce pair of GPT-FAST/tp.py:117-118,122,130,139-140 (whose hook
 * does not even fire on the reference's sparse path) by ONE kernel per rank: partial sums are
 * pushed into every rank's receive buffer with peer stores over NVLink as self-validating 8-byte
 * words {value, call number}; the owner of a block of output columns polls its buffer until all
 * `world` partials of this call have arrived and adds them in rank order.
 *   peer_base   device array of `world` pointers: rank r's buffer of
 *               sk_gemv_allreduce_buffer_bytes(world, max_batch, N) bytes as THIS GPU addresses it
 *               (peer-mapped memory, e.g. torch's symmetric memory); zero it once, on every rank,
 *               before the first call
 *   counters    ceil(N/32) uint32 in this GPU's own memory (one per CTA), zero before the first call
 * Every rank must make the same sequence of calls (same N, same max_batch) on its buffer.  All
 * CTAs are resident (N/64 <= number of SMs is required) and every wait is bounded: if a peer does
 * not show up the call sets SK_DEV_WAIT_TIMEOUT in `status` and returns whatever arrived.
 * ---------------------------------------------------------------------------------- */
SK_API size_t sk_gemv_allreduce_buffer_bytes(int world, int max_batch, int N);
SK_API int sk_gemv_allreduce(const void* x, const void* W, int64_t w_row_stride, const void* res, void* out,
                      int dtype, int B, int N, int K, void* const* peer_base, int world, int rank,
                      int max_batch, uint32_t* counters, int32_t* status, void* stream);

/* ------------------------------------------------------------------------------------
 * Query soft hash.  Replaces Attention.soft_hash (GPT-FAST/model.py:392-401):
 * q_probs[b,h,l,:] = softmax_r( (tanh(<q, planes[l,p]>) / sqrt(D)) . protos_T[p,r] / temperature )
 * (temperature 1.0 = the GPT-FAST formula; the HuggingFace variant divides by 0.3,
 * pipeline/train_quest/modeling/modeling_llama.py:638).
 *   q [B,H,D]; planes [L,P,D]; protos_T [P,R] fp32
 *   q_probs  [B,H,L,R] fp32 or NULL
 *   lut      scorer table or NULL: [B*Hkv*tiles][R][L][ht] fp32 with ht = sk_lut_head_tile(H/Hkv),
 *            tiles = (H/Hkv)/ht — the same numbers, grouped so that the ht query heads of a
 *            KV head that are scored together sit in one 4*ht-byte word.  B*H*L*R*4 bytes.
 * ---------------------------------------------------------------------------------- */
SK_API int sk_lut_head_tile(int rep);
SK_API int sk_soft_hash(const void* q, int q_dtype, const void* planes, int plane_dtype,
                 const float* protos_T, float temperature, int B, int H, int Hkv, int D, int L,
                 int P, int R, float* q_probs, float* lut, void* stream);

/* Scorer table from a q_probs tensor the caller already has ([B,H,L,R], any SK_* dtype);
 * used by the drop-in build_sparse_list_decode, whose first argument is q_probs
 * (GPT-FAST/kernels/sparse.py:16-17). */
SK_API int sk_lut_from_probs(const void* q_probs, int dtype, int B, int H, int Hkv, int L, int R,
                      float* lut, void* stream);

/* ------------------------------------------------------------------------------------
 * Soft-collision scorer on the cache-native layout.  Computes what
 * soft_hash_collision_kernel_3 computes (GPT-FAST/kernels/soft_hash_collision.cu:25-54)
 * without the relayout that feeds it (GPT-FAST/model.py:494-506):
 * scores[b,h,t] = allowed ? (sum_l q_probs[b,h,l,codes[b,h/rep,t,l]]) * v_norm[b,h/rep,t] : -inf
 *   lut      from sk_soft_hash / sk_lut_from_probs
 *   codes    [B,Hkv,Tcap,L] uint8 (16-byte aligned rows: L % 16 == 0)
 *   v_norm   [B,Hkv,Tcap] fp16
 *   allowed  [B,H,T] bytes (0 = masked) or NULL (every position allowed, the decode case,
 *            model.py:490-492)
 *   T        number of live positions; when T_dev != NULL the kernels use min(*T_dev, T)
 *            (device-side length, e.g. KVCache.prefill_len) and T only bounds the grid
 *   scores   [B,H,score_row_stride] fp32
 * ---------------------------------------------------------------------------------- */
SK_API int sk_score(const float* lut, const uint8_t* codes, const uint16_t* v_norm,
             const uint8_t* allowed, int B, int H, int Hkv, int L, int R, int64_t T,
             const int32_t* T_dev, int64_t Tcap, float* scores, int64_t score_row_stride,
             int32_t* status, void* stream);

/* Exact surface of the reference's scorer extension, soft_hash_collision(q_probs,
 * key_buckets, allowed_ext, v_hist) (GPT-FAST/kernels/soft_hash_collision_loader.py:16-72):
 *   q_probs [B,H,1,L,R] fp32, key_buckets [B,H,L,T] int16, allowed [B,H,1,T] bool bytes,
 *   v_hist [B,H,1,T] fp32, out [B,H,1,T] fp32.  Tables are added in ascending order, so
 *   the result is bit-identical to the reference kernel's. */
SK_API int sk_score_compat(const float* q_probs, const int16_t* key_buckets, const uint8_t* allowed,
                    const float* v_hist, float* out, int B, int H, int L, int R, int64_t T,
                    void* stream);

/* ------------------------------------------------------------------------------------
 * Top-k select + list assembly.  Replaces torch.topk and the list code of
 * build_sparse_list_decode (GPT-FAST/kernels/sparse.py:57-95).  Per row r = (b,h):
 *   list[r] = [0..sink) ++ [max(T-window,sink)..T) ++ topM(scores[r]),  list_len[r] = its length
 * (a single entry T-1 replaces an empty sink+window part; duplicates between the parts are
 * kept; entries whose position is not allowed become -1, as in the reference).  Among equal
 * scores the smallest index wins.  Order of the top-M part: descending score like torch.topk
 * when sorted != 0; otherwise a deterministic order that is a function of the scores only
 * (runs of ascending indices) — attention over the list does not depend on it.
 *   scores [rows, score_row_stride] fp32, allowed [rows, T] bytes or NULL
 *   list   [rows, list_row_stride] int32, list_row_stride >= sk_list_len(T, sink, window, M)
 * ---------------------------------------------------------------------------------- */
SK_API int64_t sk_list_len(int64_t T, int sink, int window, int64_t M);
SK_API int sk_select_list(const float* scores, int64_t score_row_stride, const uint8_t* allowed,
                   int64_t rows, int64_t T, const int32_t* T_dev, int64_t M, int sink,
                   int window, int sorted, int32_t* list, int64_t list_row_stride,
                   int32_t* list_len, int32_t* status, void* stream);

/* ------------------------------------------------------------------------------------
 * Scorer and select fused: the same list as sk_score followed by sk_select_list (sorted == 0,
 * no mask), without writing the [B,H,T] score array.  The scorer keeps only keys above a cut
 * estimated from a sample (about 3*M per row), the select kernel proves that this candidate
 * set contains the exact top-M and otherwise rescores the row itself, so the result is exact
 * in every case.  Replaces the same reference code as the two calls it fuses
 * (GPT-FAST/kernels/soft_hash_collision.cu:25-54 + GPT-FAST/kernels/sparse.py:57-95).
 *   applicable shapes: sk_score_select_applicable(...) != 0  (L = 32, R <= 256, T >= 4096,
 *   12*M <= T, M <= 4096); workspace: sk_score_select_workspace_bytes, 256-byte aligned,
 *   zero-initialised once.
 * ---------------------------------------------------------------------------------- */
SK_API int sk_score_select_applicable(int B, int H, int Hkv, int L, int R, int64_t T, int64_t M);
SK_API size_t sk_score_select_workspace_bytes(int B, int H, int Hkv, int L, int64_t T, int64_t M);
/* The two halves of sk_score_select_list, for callers that want to time or overlap them: the
 * filtering scorer fills the workspace, the candidate select consumes it.  Same arguments. */
SK_API int sk_score_filter(const float* lut, const uint8_t* codes, const uint16_t* v_norm, int B, int H, int Hkv,
                    int L, int R, int64_t T, const int32_t* T_dev, int64_t Tcap, int64_t M, void* workspace,
                    size_t workspace_bytes, int32_t* status, void* stream);
SK_API int sk_select_candidates(const float* lut, const uint8_t* codes, const uint16_t* v_norm, int B, int H, int Hkv,
                         int L, int R, int64_t T, const int32_t* T_dev, int64_t Tcap, int64_t M, int sink,
                         int window, int32_t* list, int64_t list_row_stride, int32_t* list_len,
                         void* workspace, size_t workspace_bytes, int32_t* status, void* stream);
SK_API int sk_score_select_list(const float* lut, const uint8_t* codes, const uint16_t* v_norm, int B, int H,
                         int Hkv, int L, int R, int64_t T, const int32_t* T_dev, int64_t Tcap, int64_t M,
                         int sink, int window, int32_t* list, int64_t list_row_stride, int32_t* list_len,
                         void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* ------------------------------------------------------------------------------------
 * Scorer and select in ONE launch on thread-block clusters: a cluster of up to 16 CTAs per KV
 * head scores its keys for the four query heads of a table word, keeps all scores on chip and
 * finds the exact top-M with a radix select whose histograms are combined through distributed
 * shared memory.  Same list as sk_score followed by sk_select_list (sorted == 0, no mask), the
 * top-M part in ascending index order.  No workspace.  Replaces the same reference code as
 * sk_score_select_list.
 *   sk_score_select_cluster_size(...) -> the cluster size used for the shape on the current
 *   device, or 0 when the shape is outside this path (needs L = 32, R = 256, 4 | H/Hkv,
 *   ceil(T / cluster size) <= 5120 keys per CTA and all B*Hkv*(H/Hkv/4) clusters resident at once).
 * ---------------------------------------------------------------------------------- */
SK_API int sk_score_select_cluster_size(int B, int H, int Hkv, int L, int R, int64_t T, int64_t M);
SK_API int sk_score_select_cluster(const float* lut, const uint8_t* codes, const uint16_t* v_norm, int B, int H,
                            int Hkv, int L, int R, int64_t T, const int32_t* T_dev, int64_t Tcap, int64_t M,
                            int sink, int window, int32_t* list, int64_t list_row_stride, int32_t* list_len,
                            int32_t* status, void* stream);

/* ------------------------------------------------------------------------------------
 * GQA sparse flash-decode.  Replaces sparse_attention_fwd and its two Triton kernels
 * (GPT-FAST/kernels/sparse.py:309-329, 102-235):
 *   out[b,h,:] = sum_j softmax_j(<q[b,h], K[b,h/rep,idx_j]>/sqrt(D)) V[b,h/rep,idx_j],
 *   j < list_len[b,h]; repeated indices count as often as they appear; negative entries
 *   are skipped.  K/V rows are read in place from the cache (strides in elements), no
 *   contiguous copy of the prefix is needed (compare GPT-FAST/model.py:541-542).
 *   q, out [B,H,D] (q_dtype); k_cache, v_cache (kv_dtype) with batch/head/row strides
 *   T: positions >= T are rejected (SK_DEV_INDEX_OUT_OF_RANGE), T_dev as in sk_score
 *   workspace: sk_sparse_decode_workspace_bytes(B,H,D,max_list_len) bytes, 256-byte aligned.
 *              Its first 256 KiB (ticket counters, independent of the shape) must be zero
 *              before the first call; every call leaves them zero again, so one buffer
 *              zeroed once serves calls of any shape, one call at a time.
 * ---------------------------------------------------------------------------------- */
SK_API size_t sk_sparse_decode_workspace_bytes(int B, int H, int D, int64_t max_list_len);
SK_API int sk_sparse_decode(const void* q, int q_dtype, const void* k_cache, const void* v_cache,
                     int kv_dtype, int64_t kv_batch_stride, int64_t kv_head_stride,
                     int64_t kv_row_stride, const int32_t* list, int64_t list_row_stride,
                     const int32_t* list_len, int64_t max_list_len, void* out, int B, int H,
                     int Hkv, int D, int64_t T, const int32_t* T_dev, void* workspace,
                     size_t workspace_bytes, int32_t* status, void* stream);

/* ------------------------------------------------------------------------------------
 * Packed form of the fused scorer + select (L = 32, R = 256, query heads per KV head a multiple
 * of 4): the scan reads a 12-bit fixed-point copy of the scorer table (8 bytes per bucket and table
 * for the four heads, summed as exact integers), which halves the shared-memory traffic of the scan;
 * the select brackets the k-th score with rigorous bounds and scores the few keys inside the
 * bracket with the fp32 table.  The list is the one sk_score + sk_select_list return, element for
 * element.  Replaces the same reference span as sk_score_select_list
 * (GPT-FAST/kernels/sparse.py:39-95 with soft_hash_collision.cu:25-54); the fixed-point table has no
 * counterpart in the reference.
 *
 *   sk_packed_table_bytes      size of the packed-table buffer [B*Hkv*(H/Hkv/4) x 64 KiB | constants |
 *                              q_probs fp32, 32 KiB per (batch, head) row - read by the select]
 *   sk_soft_hash_packed        sk_soft_hash that writes the fp32 table AND its packed copy; the
 *                              quantisation range follows from protos_T and the temperature alone
 *                              (|tanh| <= 1), so it needs the soft hash, not just q_probs
 *   sk_score_select_packed     stages & 1: the scan, stages & 2: the select (3 = both, the normal
 *                              call); workspace as for sk_score_select_list; codes 32-byte aligned
 * ---------------------------------------------------------------------------------- */
SK_API size_t sk_packed_table_bytes(int B, int H, int Hkv);
SK_API int sk_packed_applicable(int B, int H, int Hkv, int L, int R, int64_t T, int64_t M);
/* 1 where sk_decode_step's SK_SELECT_AUTO / SK_SELECT_FILTER take the packed form: shapes in which a
 * CTA scans tens of thousands of keys; below that the fp32 scan is as fast and its select cheaper. */
SK_API int sk_packed_preferred(int B, int H, int Hkv, int L, int R, int64_t T, int64_t M);
SK_API int sk_soft_hash_packed(const void* q, int q_dtype, const void* planes, int plane_dtype,
                        const float* protos_T, float temperature, int B, int H, int Hkv, int D, int L,
                        int P, int R, float* lut, void* packed, void* stream);
SK_API int sk_score_select_packed(const float* lut, const void* packed, const uint8_t* codes,
                           const uint16_t* v_norm, int B, int H, int Hkv, int L, int R, int64_t T,
                           const int32_t* T_dev, int64_t Tcap, int64_t M, int sink, int window,
                           int32_t* list, int64_t list_row_stride, int32_t* list_len, void* workspace,
                           size_t workspace_bytes, int32_t* status, int stages, void* stream);

/* ------------------------------------------------------------------------------------
 * sk_sparse_decode without any caller-provided or allocated scratch.  No counterpart in the
 * reference (its sparse_attention_fwd allocates its partial-result tensors on every call,
 * GPT-FAST/kernels/sparse.py:323-325).
 *
 * For callers that may not allocate device memory at the point of the call: a serving
 * process that handed the whole GPU to its own memory pool at start-up (a later cudaMalloc
 * fails there), a plug-in that only receives tensors and a stream and owns no allocator, or a
 * latency-critical loop in which an allocator call (and its possible implicit synchronisation)
 * is not acceptable.  The partial results of the split list and the per-row ticket counters
 * live in a buffer of SK_SPARSE_DECODE_STATIC_BYTES that is part of the library image: every
 * GPU that loads the library holds one copy until the process exits.
 *
 * Same arguments and result as sk_sparse_decode, minus the workspace.  Limits and rules:
 *   - shapes whose scratch need (sk_sparse_decode_workspace_bytes) exceeds the built-in
 *     buffer are rejected with SK_ERR_WORKSPACE and a message naming both sizes; nothing is
 *     enqueued.  The buffer covers e.g. B*H = 128 rows with lists of a few thousand entries.
 *   - the first call on each device looks up the buffer's device address (with that device
 *     current); make that first call outside any stream capture.  The address is kept for
 *     the life of the process: after a cudaDeviceReset of that device it is stale, so a
 *     process that resets a device must not call this entry point on it again.
 *   - all calls on a device share the one buffer: calls that can overlap on the GPU (two
 *     streams, two threads) race on it.  Serialise them, or use sk_sparse_decode with
 *     separate workspaces.  Each call clears the ticket counters it uses before its kernel.
 *   - it calls no cudaMalloc / cudaFree and no allocating library routine.
 * ---------------------------------------------------------------------------------- */
#define SK_SPARSE_DECODE_STATIC_BYTES (2u << 20)
SK_API int sk_sparse_decode_static(const void* q, int q_dtype, const void* k_cache, const void* v_cache,
                     int kv_dtype, int64_t kv_batch_stride, int64_t kv_head_stride,
                     int64_t kv_row_stride, const int32_t* list, int64_t list_row_stride,
                     const int32_t* list_len, int64_t max_list_len, void* out, int B, int H,
                     int Hkv, int D, int64_t T, const int32_t* T_dev, int32_t* status, void* stream);

/* ------------------------------------------------------------------------------------
 * One decode step of one layer, fused on one stream with no host synchronisation: the
 * body of Attention.sparse_forward between the QKV projection and the output projection
 * (GPT-FAST/model.py:449-552): append+hash the new token, soft-hash the query, score,
 * select, attend.  Graph-capturable: the live length is read from `prefill_len` on the
 * device, grids are sized from `T_max`.
 * ---------------------------------------------------------------------------------- */
enum sk_select_path {
    SK_SELECT_AUTO = 0,
    SK_SELECT_TWO_LAUNCH = 1,   /* sk_score + sk_select_list (score matrix in the workspace) */
    SK_SELECT_FILTER = 2,       /* filtering scorer + candidate select, packed table where it applies */
    SK_SELECT_CLUSTER = 3,      /* sk_score_select_cluster                                   */
    SK_SELECT_FILTER_F32 = 4,   /* sk_score_filter + sk_select_candidates on the fp32 table  */
    SK_SELECT_FILTER_PACKED = 5 /* sk_score_select_packed, whatever the size                 */
};

typedef struct sk_decode_params {
    /* new token */
    const void* q;         /* [B,H,D]      q_dtype                                   */
    const void* k_new;     /* [B,1,Hkv,D]  kv_dtype, NULL = cache already holds it   */
    const void* v_new;     /* [B,1,Hkv,D]                                             */
    const int64_t* input_pos; /* [1] device                                           */
    /* hash parameters */
    const void* planes;    /* [L,P,D] plane_dtype */
    const float* protos_T; /* [P,R] */
    float temperature;
    /* cache */
    void* k_cache;         /* [B,Hkv,Tcap,D] */
    void* v_cache;
    uint8_t* codes;        /* [B,Hkv,Tcap,L] */
    uint16_t* v_norm;      /* [B,Hkv,Tcap] fp16 */
    int32_t* prefill_len;  /* device int32 */
    /* outputs */
    void* out;             /* [B,H,D] q_dtype */
    int32_t* list;         /* [B,H,list_row_stride] or NULL (then taken from workspace) */
    int32_t* list_len;     /* [B,H] or NULL */
    int64_t list_row_stride;
    /* scratch */
    void* workspace;
    size_t workspace_bytes;
    int32_t* status;       /* device int32 or NULL */
    /* shapes */
    int q_dtype, kv_dtype, plane_dtype;
    int B, H, Hkv, D, L, P, R;
    int64_t Tcap;
    int64_t T_max;         /* upper bound of the live length during this call.  Grids, chunks and
                            * candidate capacities are sized from it: keep it within about 4x of
                            * the live length (the result is exact either way, but far below that
                            * rows start to take the slow rescoring path, see
                            * sk_decode_step_rescored_rows_offset) */
    int64_t M;
    int sink, window;
    /* how the list is built: SK_SELECT_AUTO picks the fastest path the shape allows; the others pin
     * one (SK_ERR_UNSUPPORTED if the shape is outside it).  All give the same list. */
    int select_path;
} sk_decode_params;

SK_API size_t sk_decode_step_workspace_bytes(int B, int H, int Hkv, int D, int L, int R, int64_t T_max,
                                      int64_t M, int sink, int window);
SK_API int sk_decode_step(const sk_decode_params* p, void* stream);
/* Byte offset, inside a workspace of sk_decode_step_workspace_bytes() of the same shape, of an int32
 * counter: the (batch, head) rows whose candidate set could not be proven complete and that were
 * rescored in full (an exact but slow path) by the steps run on that workspace so far.  -1 if the
 * shape's select path keeps no such counter.  The counter starts from whatever the caller put
 * there (zero the workspace once).  Eight more int32 counters follow it: [1] keys scored exactly
 * inside the k-th score's bracket (packed table), [2] rows whose bracket took the radix ranking,
 * the reason of each rescored row - [3] a run overflowed, [4] too few / too many candidates,
 * [5] result not provable on the candidates - and, for [5] with the packed table, [6] bracket
 * reaching below the largest cut, [7] bracket too large for the chip, [8] inconsistent counts. */
SK_API int64_t sk_decode_step_rescored_rows_offset(int B, int H, int Hkv, int D, int L, int R, int64_t T_max,
                                            int64_t M, int sink, int window);

#ifdef __cplusplus
}
#endif
#endif /* SOCKET_B200_H_ */
