/* Plain-C restatement of the SOCKET sparse-attention decode path.  TEST INFRASTRUCTURE ONLY:
 * it is the checker for the CUDA kernels and the timed CPU baseline, never a product path.
 *
 * Reference lines followed (paths relative to the reference root):
 *   orc_hash_keys        GPT-FAST/model.py:403-413    sign of <key, plane>, big-endian pack
 *   orc_value_norm       GPT-FAST/model.py:450        ||v||_2 in fp32
 *   orc_soft_hash        GPT-FAST/model.py:392-401    tanh / sqrt(D), protos, softmax over R
 *   orc_score            GPT-FAST/kernels/soft_hash_collision.cu:25-54   collision score
 *   orc_select_list      GPT-FAST/kernels/sparse.py:57-95   top-M + sink/window list
 *   orc_sparse_attention GPT-FAST/kernels/sparse.py:102-235 chunked online softmax + merge
 *
 * Parallelised over independent rows with OpenMP (the reference's CPU path gets its threads
 * from torch's intra-op pool; here the same cores are used explicitly).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = ((uint32_t)h) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline float f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ffu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) {
            u = sign;
        } else { /* subnormal */
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            man &= 0x3ffu;
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        u = sign | 0x7f800000u | (man << 13);
    } else {
        u = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* dtype tags shared by every entry point: 0 = fp32, 1 = bf16, 2 = fp16 */
static inline float load_elem(const void* base, int dtype, int64_t i) {
    if (dtype == 0) return ((const float*)base)[i];
    if (dtype == 1) return bf16_to_f32(((const uint16_t*)base)[i]);
    return f16_to_f32(((const uint16_t*)base)[i]);
}

/* keys [N, D] (row stride D), planes [L*P, D]; codes [N, L] as int16.
 * exact != 0: accumulate in fp64 (decides the true sign for 16-bit inputs);
 * exact == 0: accumulate in fp32 in ascending d. */
void orc_hash_keys(const void* keys, int key_dtype, const void* planes, int plane_dtype,
                   int64_t N, int D, int L, int P, int exact, int16_t* codes) {
    float* pl = (float*)malloc(sizeof(float) * (size_t)L * P * D);
    for (int64_t i = 0; i < (int64_t)L * P * D; ++i) pl[i] = load_elem(planes, plane_dtype, i);
#pragma omp parallel
    {
        float* kr = (float*)malloc(sizeof(float) * D);
#pragma omp for schedule(static)
        for (int64_t n = 0; n < N; ++n) {
            for (int d = 0; d < D; ++d) kr[d] = load_elem(keys, key_dtype, n * D + d);
            for (int l = 0; l < L; ++l) {
                int code = 0;
                for (int p = 0; p < P; ++p) {
                    const float* pp = pl + ((size_t)l * P + p) * D;
                    int bit;
                    if (exact) {
                        double s = 0.0;
                        for (int d = 0; d < D; ++d) s += (double)kr[d] * (double)pp[d];
                        bit = s >= 0.0;
                    } else {
                        float s = 0.f;
                        for (int d = 0; d < D; ++d) s += kr[d] * pp[d];
                        bit = s >= 0.f;
                    }
                    code = code * 2 + bit;
                }
                codes[n * L + l] = (int16_t)code;
            }
        }
        free(kr);
    }
    free(pl);
}

/* v [N, D] -> out [N] fp32 (the caller rounds to fp16 like the reference). */
void orc_value_norm(const void* v, int dtype, int64_t N, int D, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        float s = 0.f;
        for (int d = 0; d < D; ++d) {
            float x = load_elem(v, dtype, n * D + d);
            s += x * x;
        }
        out[n] = sqrtf(s);
    }
}

/* q [BH, D], planes [L*P, D], protos_T [P, R] -> q_probs [BH, L, R] */
void orc_soft_hash(const void* q, int q_dtype, const void* planes, int plane_dtype,
                   const float* protos_T, int64_t BH, int D, int L, int P, int R,
                   float temperature, float* q_probs) {
    float inv = 1.0f / fmaxf(sqrtf((float)D), 1e-6f);
#pragma omp parallel for schedule(static)
    for (int64_t bh = 0; bh < BH; ++bh) {
        float t[64];
        for (int l = 0; l < L; ++l) {
            for (int p = 0; p < P; ++p) {
                float s = 0.f;
                for (int d = 0; d < D; ++d)
                    s += load_elem(q, q_dtype, bh * D + d) *
                         load_elem(planes, plane_dtype, ((int64_t)l * P + p) * D + d);
                t[p] = tanhf(s) * inv;
            }
            float* row = q_probs + ((size_t)bh * L + l) * R;
            float mx = -INFINITY;
            for (int r = 0; r < R; ++r) {
                float lg = 0.f;
                for (int p = 0; p < P; ++p) lg += t[p] * protos_T[(size_t)p * R + r];
                lg /= temperature;
                row[r] = lg;
                mx = fmaxf(mx, lg);
            }
            float se = 0.f;
            for (int r = 0; r < R; ++r) {
                row[r] = expf(row[r] - mx);
                se += row[r];
            }
            for (int r = 0; r < R; ++r) row[r] /= se;
        }
    }
}

/* q_probs [B,H,L,R] fp32; codes [B,Hkv,Tcap,L] uint8; v_norm [B,Hkv,Tcap] fp16 bits;
 * allowed [B,H,T] bytes or NULL; scores [B,H,T] fp32.  Tables added in ascending l. */
void orc_score(const float* q_probs, const uint8_t* codes, const uint16_t* v_norm,
               const uint8_t* allowed, int B, int H, int Hkv, int64_t T, int64_t Tcap, int L,
               int R, float* scores) {
    int rep = H / Hkv;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b) {
        for (int h = 0; h < H; ++h) {
            int kvh = h / rep;
            const float* qp = q_probs + ((size_t)b * H + h) * L * R;
            const uint8_t* cd = codes + ((size_t)b * Hkv + kvh) * Tcap * L;
            const uint16_t* vn = v_norm + ((size_t)b * Hkv + kvh) * Tcap;
            float* out = scores + ((size_t)b * H + h) * T;
            const uint8_t* al = allowed ? allowed + ((size_t)b * H + h) * T : NULL;
            for (int64_t t = 0; t < T; ++t) {
                if (al && !al[t]) { out[t] = -INFINITY; continue; }
                float s = 0.f;
                for (int l = 0; l < L; ++l) s += qp[(size_t)l * R + cd[t * L + l]];
                out[t] = s * f16_to_f32(vn[t]);
            }
        }
    }
}

static inline uint32_t order_key(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if (u == 0x80000000u) u = 0; /* -0 == +0 */
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

static int cmp_u64_desc(const void* a, const void* b) {
    uint64_t x = *(const uint64_t*)a, y = *(const uint64_t*)b;
    return (x < y) - (x > y);
}

static int cmp_i32_asc(const void* a, const void* b) {
    int32_t x = *(const int32_t*)a, y = *(const int32_t*)b;
    return (x > y) - (x < y);
}

/* quickselect so that the k largest of a[0..n) sit in a[0..k) (any order) */
static void select_top(uint64_t* a, int64_t n, int64_t k) {
    int64_t lo = 0, hi = n - 1;
    while (lo < hi) {
        uint64_t x = a[lo], y = a[(lo + hi) / 2], z = a[hi];
        uint64_t piv = (x > y) ? ((y > z) ? y : (x > z ? z : x)) : ((x > z) ? x : (y > z ? z : y));
        int64_t i = lo, j = hi;
        while (i <= j) {
            while (a[i] > piv) ++i;
            while (a[j] < piv) --j;
            if (i <= j) { uint64_t t = a[i]; a[i] = a[j]; a[j] = t; ++i; --j; }
        }
        if (k - 1 <= j) hi = j;
        else if (k - 1 >= i) lo = i;
        else break;
    }
}

/* scores [rows, T] -> list [rows, Ktot] = [sink..., window..., heavy...]; heavy = top-M
 * by score, ties to the smallest index; order: descending score when sorted != 0, else
 * ascending index.  allowed [rows, T] or NULL: entries not allowed become -1.
 * Returns Ktot (callers size `list` with orc_list_len). */
int64_t orc_list_len(int64_t T, int sink, int window, int64_t M) {
    int64_t s = sink < 0 ? 0 : (sink > T ? T : sink);
    int64_t w = window < 0 ? 0 : (window > T ? T : window);
    int64_t nb = s;
    if (w > 0) {
        int64_t st = T - w > s ? T - w : s;
        if (st < T) nb += T - st;
    }
    if (nb == 0) nb = 1;
    return nb + (M < T ? M : T);
}

int64_t orc_select_list(const float* scores, const uint8_t* allowed, int64_t rows, int64_t T,
                        int sink, int window, int64_t M, int sorted, int32_t* list,
                        int32_t* list_len) {
    int64_t Ktot = orc_list_len(T, sink, window, M);
    int64_t Me = M < T ? M : T;
    int64_t s = sink < 0 ? 0 : (sink > T ? T : sink);
    int64_t w = window < 0 ? 0 : (window > T ? T : window);
#pragma omp parallel
    {
        uint64_t* keys = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)(T > 0 ? T : 1));
#pragma omp for schedule(dynamic, 1)
        for (int64_t r = 0; r < rows; ++r) {
            const float* sc = scores + (size_t)r * T;
            const uint8_t* al = allowed ? allowed + (size_t)r * T : NULL;
            int32_t* out = list + (size_t)r * Ktot;
            int64_t n = 0;
            for (int64_t i = 0; i < s; ++i) out[n++] = (int32_t)i;
            if (w > 0) {
                int64_t st = T - w > s ? T - w : s;
                for (int64_t i = st; i < T; ++i) out[n++] = (int32_t)i;
            }
            if (n == 0) out[n++] = (int32_t)(T - 1);
            for (int64_t i = 0; i < n; ++i)
                if (al && !al[out[i]]) out[i] = -1;
            if (Me > 0) {
                for (int64_t t = 0; t < T; ++t)
                    keys[t] = ((uint64_t)order_key(sc[t]) << 32) | (uint32_t)(0xffffffffu - (uint32_t)t);
                select_top(keys, T, Me);
                if (sorted) {
                    qsort(keys, (size_t)Me, sizeof(uint64_t), cmp_u64_desc);
                    for (int64_t i = 0; i < Me; ++i)
                        out[n + i] = (int32_t)(0xffffffffu - (uint32_t)(keys[i] & 0xffffffffu));
                } else {
                    for (int64_t i = 0; i < Me; ++i)
                        out[n + i] = (int32_t)(0xffffffffu - (uint32_t)(keys[i] & 0xffffffffu));
                    qsort(out + n, (size_t)Me, sizeof(int32_t), cmp_i32_asc);
                }
                for (int64_t i = 0; i < Me; ++i)
                    if (al && !al[out[n + i]]) out[n + i] = -1;
            }
            list_len[r] = (int32_t)Ktot;
        }
        free(keys);
    }
    return Ktot;
}

/* q [B,H,D], k/v [B,Hkv,Tcap,D] (kv_dtype), list [B,H,Ktot], len [B,H] -> out [B,H,D] fp32.
 * Chunks of block_seq entries, blocks of 16 inside a chunk, log-sum-exp merge. */
void orc_sparse_attention(const void* q, int q_dtype, const void* k, const void* v, int kv_dtype,
                          const int32_t* list, const int32_t* len, int B, int H, int Hkv,
                          int64_t Tcap, int D, int64_t Ktot, int block_seq, float* out) {
    int rep = H / Hkv;
    float scale = 1.0f / sqrtf((float)D);
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int b = 0; b < B; ++b) {
        for (int h = 0; h < H; ++h) {
            float qv[256], acc[256], tot[256];
            int kvh = h / rep;
            size_t kvbase = ((size_t)b * Hkv + kvh) * Tcap * D;
            const int32_t* lst = list + ((size_t)b * H + h) * Ktot;
            int n = len[(size_t)b * H + h];
            for (int d = 0; d < D; ++d) qv[d] = load_elem(q, q_dtype, ((int64_t)b * H + h) * D + d);
            float gm = -INFINITY, gs = 0.f;
            for (int d = 0; d < D; ++d) tot[d] = 0.f;
            for (int c0 = 0; c0 < n; c0 += block_seq) {
                int c1 = c0 + block_seq < n ? c0 + block_seq : n;
                float m = -INFINITY, se = 0.f;
                for (int d = 0; d < D; ++d) acc[d] = 0.f;
                for (int s0 = c0; s0 < c1; s0 += 16) {
                    int s1 = s0 + 16 < c1 ? s0 + 16 : c1;
                    float att[16];
                    float bm = -INFINITY;
                    for (int j = s0; j < s1; ++j) {
                        int idx = lst[j];
                        if (idx < 0) { att[j - s0] = -INFINITY; continue; }
                        float dot = 0.f;
                        for (int d = 0; d < D; ++d)
                            dot += qv[d] * load_elem(k, kv_dtype, (int64_t)(kvbase + (size_t)idx * D + d));
                        att[j - s0] = dot * scale;
                        bm = fmaxf(bm, att[j - s0]);
                    }
                    if (bm == -INFINITY) continue;
                    float nm = fmaxf(bm, m);
                    float resc = expf(m - nm);
                    for (int d = 0; d < D; ++d) acc[d] *= resc;
                    se *= resc;
                    for (int j = s0; j < s1; ++j) {
                        int idx = lst[j];
                        if (idx < 0) continue;
                        float p = expf(att[j - s0] - nm);
                        se += p;
                        for (int d = 0; d < D; ++d)
                            acc[d] += p * load_elem(v, kv_dtype, (int64_t)(kvbase + (size_t)idx * D + d));
                    }
                    m = nm;
                }
                if (se > 0.f) {
                    float lse = m + logf(se);
                    float nm = fmaxf(lse, gm);
                    float old = expf(gm - nm), wgt = expf(lse - nm);
                    for (int d = 0; d < D; ++d) tot[d] = tot[d] * old + wgt * (acc[d] / se);
                    gs = gs * old + wgt;
                    gm = nm;
                }
            }
            float* o = out + ((size_t)b * H + h) * D;
            for (int d = 0; d < D; ++d) o[d] = gs > 0.f ? tot[d] / gs : 0.f;
        }
    }
}
