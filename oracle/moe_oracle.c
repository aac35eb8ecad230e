/*
 * CPU oracle for the W4A16 MoE layer path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a plain-C restatement of the arithmetic of glmserve's CPU float32
 * reference forward for one MoE layer.  It is the checker the CUDA path is compared
 * with; nothing in the shipped library may call it.  Every function names the
 * reference lines it follows.  Parity status: PINNED - the restatement is compared
 * bit for bit with the reference's own GLM52Model::moe_mlp (built from the reference
 * sources by oracle/Makefile into oracle/_ref/) and with golden vectors that the
 * reference produced (tests/golden/).
 *
 * Numeric contract (must be compiled without FMA contraction and without fast-math,
 * like the reference's "-O2" x86-64 build):
 *   - dot products: fp32, ascending index, product and sum rounded separately
 *   - silu(a) = a / (1 + expf(-a)), sigmoid(a) = 1 / (1 + expf(-a))
 *   - int4: two values per byte, low nibble = even column, zero point 8, per-group scale
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>
#include <unistd.h>

#define ORC_API __attribute__((visibility("default")))

/* Minimal pthread work-sharing loop (indices handed out one at a time).  Threads only
 * split independent (expert) or (row) work; no floating-point sum crosses a thread, so
 * results do not depend on the thread count. */
typedef void (*orc_body_fn)(int64_t i, void* ctx);
typedef struct { orc_body_fn fn; void* ctx; int64_t n; int64_t next; pthread_mutex_t mu; } orc_pf_t;
static void* orc_pf_worker(void* p) {
    orc_pf_t* pf = (orc_pf_t*)p;
    for (;;) {
        pthread_mutex_lock(&pf->mu);
        int64_t i = pf->next++;
        pthread_mutex_unlock(&pf->mu);
        if (i >= pf->n) break;
        pf->fn(i, pf->ctx);
    }
    return NULL;
}
static void orc_parallel_for(int64_t n, int nthreads, orc_body_fn fn, void* ctx) {
    if (nthreads > n) nthreads = (int)n;
    if (nthreads <= 1) { for (int64_t i = 0; i < n; ++i) fn(i, ctx); return; }
    orc_pf_t pf; pf.fn = fn; pf.ctx = ctx; pf.n = n; pf.next = 0;
    pthread_mutex_init(&pf.mu, NULL);
    pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)nthreads);
    int started = 0;
    for (int t = 0; t < nthreads - 1; ++t)
        if (pthread_create(&th[started], NULL, orc_pf_worker, &pf) == 0) ++started;
    orc_pf_worker(&pf);
    for (int t = 0; t < started; ++t) pthread_join(th[t], NULL);
    free(th);
    pthread_mutex_destroy(&pf.mu);
}

/* src/model_glm52.cpp:95-96 */
static inline float orc_silu(float x) { return x / (1.0f + expf(-x)); }
static inline float orc_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

/* src/tensor.cpp:53-63 - flat index i over [out, in]; scale index i / group. */
ORC_API void orc_dequant_int4(const uint8_t* packed, const float* scales, int64_t count,
                              int64_t group, float* out) {
    for (int64_t i = 0; i < count; ++i) {
        uint8_t byte = packed[i >> 1];
        int q = (i & 1) ? (byte >> 4) : (byte & 0x0F);
        out[i] = (float)(q - 8) * scales[i / group];
    }
}

/* src/model_glm52.cpp:42-58 - y[n,out] = x[n,in] W[out,in]^T (+ bias). */
ORC_API void orc_linear(const float* w, const float* bias, const float* x, float* y,
                        int64_t n, int64_t in, int64_t out) {
    for (int64_t t = 0; t < n; ++t) {
        const float* xt = x + t * in;
        for (int64_t o = 0; o < out; ++o) {
            const float* wo = w + o * in;
            float acc = 0.0f;
            for (int64_t i = 0; i < in; ++i) acc += xt[i] * wo[i];
            y[t * out + o] = bias ? acc + bias[o] : acc;
        }
    }
}

/* src/model_glm52.cpp:61-71 - double sum of squares, float inverse, x*inv*w. */
ORC_API void orc_rmsnorm_rows(const float* x, const float* w, float* out, int64_t n, int64_t dim,
                              float eps) {
    for (int64_t r = 0; r < n; ++r) {
        const float* xr = x + r * dim;
        double ss = 0.0;
        for (int64_t i = 0; i < dim; ++i) ss += (double)xr[i] * xr[i];
        float inv = (float)(1.0 / sqrt(ss / dim + eps));
        for (int64_t i = 0; i < dim; ++i) out[r * dim + i] = xr[i] * inv * w[i];
    }
}

/*
 * src/model_glm52.cpp:1113-1129 - sigmoid score, selection by score + bias, weight = the
 * un-biased score, sum in selection order, optional normalisation, routed scale.
 * The reference orders with std::partial_sort, whose result on exactly equal keys is
 * unspecified; this restatement resolves ties to the smaller expert id, which is what
 * the reference's GPU kernel (cuda/moe_router.cu:9-16) and its numpy twin
 * (tools/make_tiny_checkpoint.py:207) do.  Returns the number of tokens whose first
 * topk+1 keys contain an exact tie (0 means the ordering is unambiguous).
 */
ORC_API int orc_router(const float* logits, const float* e_bias, int n, int E, int topk,
                       int norm_topk, float routed_scale, int* topk_ids, float* topk_w) {
    int ties = 0;
    float* score = (float*)malloc(sizeof(float) * (size_t)E * 2);
    float* choose = score + E;
    for (int t = 0; t < n; ++t) {
        const float* lt = logits + (size_t)t * E;
        for (int e = 0; e < E; ++e) {
            score[e] = orc_sigmoid(lt[e]);
            choose[e] = score[e] + (e_bias ? e_bias[e] : 0.0f);
        }
        float prev = 0.0f;
        int tie = 0;
        float w[64];
        float wsum = 0.0f;
        for (int k = 0; k <= topk && k < E; ++k) {
            int be = -1;
            float bc = 0.0f;
            for (int e = 0; e < E; ++e) {
                int taken = 0;
                for (int j = 0; j < k && j < topk; ++j) taken |= (topk_ids[(size_t)t * topk + j] == e);
                if (taken) continue;
                if (be < 0 || choose[e] > bc) { be = e; bc = choose[e]; }
            }
            if (k > 0 && be >= 0 && bc == prev) tie = 1;
            prev = bc;
            if (k < topk) {
                topk_ids[(size_t)t * topk + k] = be;
                w[k] = score[be];
                wsum += w[k];
            }
        }
        ties += tie;
        if (norm_topk && wsum > 0.0f)
            for (int k = 0; k < topk; ++k) w[k] /= wsum;
        for (int k = 0; k < topk; ++k) topk_w[(size_t)t * topk + k] = w[k] * routed_scale;
    }
    free(score);
    return ties;
}

/* cuda/moe_dispatch.cu:24-38 - stable counting sort of flat (token, slot) pairs by expert. */
ORC_API void orc_dispatch(const int* topk_ids, int n, int topk, int E, int* expert_offsets,
                          int* sorted_token_ids, int* sorted_row) {
    int total = n * topk;
    for (int e = 0; e <= E; ++e) expert_offsets[e] = 0;
    for (int i = 0; i < total; ++i) expert_offsets[topk_ids[i] + 1]++;
    for (int e = 0; e < E; ++e) expert_offsets[e + 1] += expert_offsets[e];
    int* cursor = (int*)malloc(sizeof(int) * (size_t)(E > 0 ? E : 1));
    for (int e = 0; e < E; ++e) cursor[e] = expert_offsets[e];
    for (int t = 0; t < n; ++t)
        for (int k = 0; k < topk; ++k) {
            int dst = cursor[topk_ids[t * topk + k]]++;
            sorted_token_ids[dst] = t;
            sorted_row[dst] = k;
        }
    free(cursor);
}

/* One int4 row -> fp32, the per-row form of src/tensor.cpp:53-63. */
static void dequant_row(const uint8_t* qrow, const float* srow, int64_t in, int64_t group,
                        float* out) {
    for (int64_t i = 0; i < in; ++i) {
        uint8_t byte = qrow[i >> 1];
        int q = (i & 1) ? (byte >> 4) : (byte & 0x0F);
        out[i] = (float)(q - 8) * srow[i / group];
    }
}

static inline float dot_seq(const float* x, const float* w, int64_t in) {
    float acc = 0.0f;
    for (int64_t i = 0; i < in; ++i) acc += x[i] * w[i];
    return acc;
}

/*
 * cuda/int4_gemm.cu:15-48 / src/model_glm52.cpp:42-58 on dequantised weights:
 * y[t,o] = sum_i W[o,i] x[t,i] (+ bias[o]).  Rows are dequantised one at a time so a
 * GLM-scale matrix never exists in fp32; per (t,o) the arithmetic and its order are
 * those of linear_forward.
 */
typedef struct { const float* x; const uint8_t* qW; const float* scales; const float* bias;
                 float* y; int64_t n, in, out, group, rows_per; } orc_gemm_ctx;
static void orc_gemm_body(int64_t blk, void* p) {
    orc_gemm_ctx* c = (orc_gemm_ctx*)p;
    const int64_t qs = (c->in + 1) / 2, ng = (c->in + c->group - 1) / c->group;
    float* wrow = (float*)malloc(sizeof(float) * (size_t)c->in);
    int64_t o1 = (blk + 1) * c->rows_per < c->out ? (blk + 1) * c->rows_per : c->out;
    for (int64_t o = blk * c->rows_per; o < o1; ++o) {
        dequant_row(c->qW + o * qs, c->scales + o * ng, c->in, c->group, wrow);
        for (int64_t t = 0; t < c->n; ++t) {
            float acc = dot_seq(c->x + t * c->in, wrow, c->in);
            c->y[t * c->out + o] = c->bias ? acc + c->bias[o] : acc;
        }
    }
    free(wrow);
}
ORC_API void orc_gemm_w4a16(const float* x, const uint8_t* qW, const float* scales,
                            const float* bias, float* y, int64_t n, int64_t in, int64_t out,
                            int64_t group, int nthreads) {
    orc_gemm_ctx c = {x, qW, scales, bias, y, n, in, out, group, 16};
    orc_parallel_for((out + c.rows_per - 1) / c.rows_per, nthreads, orc_gemm_body, &c);
}

/* Gate/up + SwiGLU + down of one expert over a list of token rows, unweighted.
 * src/model_glm52.cpp:1133-1140 (routed) and :1144-1150 (shared). */
static void expert_rows(const float* x, int64_t H, int64_t I, int64_t group, const uint8_t* gq,
                        const float* gs, const uint8_t* uq, const float* us, const uint8_t* dq,
                        const float* ds, const int* tok, int cnt, float* y /* [cnt,H] */) {
    if (cnt <= 0) return;
    const int64_t qh = (H + 1) / 2, ngh = (H + group - 1) / group;
    const int64_t qi = (I + 1) / 2, ngi = (I + group - 1) / group;
    float* wrow = (float*)malloc(sizeof(float) * (size_t)(H > I ? H : I));
    float* g = (float*)malloc(sizeof(float) * (size_t)cnt * I * 2);
    float* u = g + (size_t)cnt * I;
    for (int64_t r = 0; r < I; ++r) {
        dequant_row(gq + r * qh, gs + r * ngh, H, group, wrow);
        for (int j = 0; j < cnt; ++j) g[(size_t)j * I + r] = dot_seq(x + (size_t)tok[j] * H, wrow, H);
        dequant_row(uq + r * qh, us + r * ngh, H, group, wrow);
        for (int j = 0; j < cnt; ++j) u[(size_t)j * I + r] = dot_seq(x + (size_t)tok[j] * H, wrow, H);
    }
    for (int64_t i = 0; i < (int64_t)cnt * I; ++i) g[i] = orc_silu(g[i]) * u[i];
    for (int64_t o = 0; o < H; ++o) {
        dequant_row(dq + o * qi, ds + o * ngi, I, group, wrow);
        for (int j = 0; j < cnt; ++j) y[(size_t)j * H + o] = dot_seq(g + (size_t)j * I, wrow, I);
    }
    free(g);
    free(wrow);
}

typedef struct { const float* x; const uint8_t* gate_q; const float* gate_sc; const uint8_t* up_q;
                 const float* up_sc; const uint8_t* down_q; const float* down_sc; const int* offs;
                 const int* stok; float* y; int H, I, group; } orc_exp_ctx;
static void orc_exp_body(int64_t e, void* p) {
    orc_exp_ctx* c = (orc_exp_ctx*)p;
    const int64_t H = c->H, I = c->I, group = c->group;
    const int64_t qh = (H + 1) / 2, ngh = (H + group - 1) / group;
    const int64_t qi = (I + 1) / 2, ngi = (I + group - 1) / group;
    int b = c->offs[e], cnt = c->offs[e + 1] - c->offs[e];
    expert_rows(c->x, H, I, group, c->gate_q + (size_t)e * I * qh, c->gate_sc + (size_t)e * I * ngh,
                c->up_q + (size_t)e * I * qh, c->up_sc + (size_t)e * I * ngh,
                c->down_q + (size_t)e * H * qi, c->down_sc + (size_t)e * H * ngi, c->stok + b, cnt,
                c->y + (size_t)b * H);
}

/*
 * Routed experts given a routing decision: the body of cuda/moe_expert.cu:132-244
 * (moe_expert_ffn_w4a16) with the CPU arithmetic of src/model_glm52.cpp:1131-1142.
 * out[t,:] = sum_k w[t,k] * expert_{id[t,k]}(x_t), slots added in order k = 0..topk-1
 * starting from 0.  Work is done expert-major (each int4 row is dequantised once per
 * expert) and the per-slot rows are combined afterwards in slot order, which gives the
 * same bits as the reference's token-major loop.  y_slots (nullable) receives the
 * unweighted per-slot rows in dispatch order [n*topk, H].
 */
ORC_API void orc_moe_experts_w4(const float* x, const int* topk_ids, const float* topk_w,
                                const uint8_t* gate_q, const float* gate_sc,
                                const uint8_t* up_q, const float* up_sc, const uint8_t* down_q,
                                const float* down_sc, int n, int topk, int H, int I, int E,
                                int group, float* out, float* y_slots, int nthreads) {
    const int P = n * topk;
    int* offs = (int*)malloc(sizeof(int) * (size_t)(E + 1));
    int* stok = (int*)malloc(sizeof(int) * (size_t)(P > 0 ? P : 1) * 2);
    int* srow = stok + (P > 0 ? P : 1);
    orc_dispatch(topk_ids, n, topk, E, offs, stok, srow);
    float* y = y_slots ? y_slots : (float*)malloc(sizeof(float) * (size_t)(P > 0 ? P : 1) * H);
    orc_exp_ctx c = {x, gate_q, gate_sc, up_q, up_sc, down_q, down_sc, offs, stok, y, H, I, group};
    orc_parallel_for(E, nthreads, orc_exp_body, &c);
    /* position of flat slot (t,k) in dispatch order */
    int* pos = (int*)malloc(sizeof(int) * (size_t)(P > 0 ? P : 1));
    for (int r = 0; r < P; ++r) pos[stok[r] * topk + srow[r]] = r;
    for (int t = 0; t < n; ++t) {
        float* ot = out + (size_t)t * H;
        for (int i = 0; i < H; ++i) ot[i] = 0.0f;
        for (int k = 0; k < topk; ++k) {
            const float wk = topk_w[t * topk + k];
            const float* yr = y + (size_t)pos[t * topk + k] * H;
            for (int i = 0; i < H; ++i) ot[i] += wk * yr[i];
        }
    }
    free(pos);
    if (!y_slots) free(y);
    free(stok);
    free(offs);
}

typedef struct { const float* w; const float* x; float* y; int H, E; } orc_lin_ctx;
static void orc_lin_body(int64_t t, void* p) {
    orc_lin_ctx* c = (orc_lin_ctx*)p;
    orc_linear(c->w, NULL, c->x + (size_t)t * c->H, c->y + (size_t)t * c->E, 1, c->H, c->E);
}

/*
 * Whole layer, src/model_glm52.cpp:1096-1154: router logits (or the caller's, when
 * logits_in is given), routing, routed experts in slot order, shared expert added last
 * with weight 1.  Outputs logits_out [n,E], ids_out/w_out [n,topk] and out [n,H]; any
 * of the first three may be NULL.  The shared expert is optional (sg_q == NULL).
 */
ORC_API int orc_moe_layer_w4(const float* x, int n, int H, int I, int Is, int E, int topk,
                             int group, const float* router_w, const float* e_bias,
                             int norm_topk, float routed_scale, const uint8_t* gate_q,
                             const float* gate_sc, const uint8_t* up_q, const float* up_sc,
                             const uint8_t* down_q, const float* down_sc, const uint8_t* sg_q,
                             const float* sg_sc, const uint8_t* su_q, const float* su_sc,
                             const uint8_t* sd_q, const float* sd_sc, const float* logits_in,
                             float* logits_out, int* ids_out, float* w_out, float* out,
                             int nthreads) {
    float* logits = (float*)malloc(sizeof(float) * (size_t)n * E);
    int* ids = (int*)malloc(sizeof(int) * (size_t)n * topk);
    float* w = (float*)malloc(sizeof(float) * (size_t)n * topk);
    if (logits_in) {
        memcpy(logits, logits_in, sizeof(float) * (size_t)n * E);
    } else {
        orc_lin_ctx lc = {router_w, x, logits, H, E};
        orc_parallel_for(n, nthreads, orc_lin_body, &lc);
    }
    int ties = orc_router(logits, e_bias, n, E, topk, norm_topk, routed_scale, ids, w);
    orc_moe_experts_w4(x, ids, w, gate_q, gate_sc, up_q, up_sc, down_q, down_sc, n, topk, H, I,
                       E, group, out, NULL, nthreads);
    if (sg_q) {
        /* shared expert: rows of the three matrices spread over threads; per (t,row)
         * arithmetic unchanged. */
        float* g = (float*)malloc(sizeof(float) * (size_t)n * Is * 2);
        float* u = g + (size_t)n * Is;
        float* ys = (float*)malloc(sizeof(float) * (size_t)n * H);
        orc_gemm_w4a16(x, sg_q, sg_sc, NULL, g, n, H, Is, group, nthreads);
        orc_gemm_w4a16(x, su_q, su_sc, NULL, u, n, H, Is, group, nthreads);
        for (int64_t i = 0; i < (int64_t)n * Is; ++i) g[i] = orc_silu(g[i]) * u[i];
        orc_gemm_w4a16(g, sd_q, sd_sc, NULL, ys, n, Is, H, group, nthreads);
        for (int64_t i = 0; i < (int64_t)n * H; ++i) out[i] += ys[i];
        free(ys);
        free(g);
    }
    if (logits_out) memcpy(logits_out, logits, sizeof(float) * (size_t)n * E);
    if (ids_out) memcpy(ids_out, ids, sizeof(int) * (size_t)n * topk);
    if (w_out) memcpy(w_out, w, sizeof(float) * (size_t)n * topk);
    free(w);
    free(ids);
    free(logits);
    return ties;
}

/* Pre-norm + MoE + residual of one layer, src/model_glm52.cpp:1181-1187:
 * h += moe(rmsnorm(h)).  Used for the 8-layer speculative-verify block. */
ORC_API int orc_moe_block_layer_w4(float* hidden, const float* norm_w, float eps, int n, int H,
                                   int I, int Is, int E, int topk, int group,
                                   const float* router_w, const float* e_bias, int norm_topk,
                                   float routed_scale, const uint8_t* gate_q,
                                   const float* gate_sc, const uint8_t* up_q, const float* up_sc,
                                   const uint8_t* down_q, const float* down_sc,
                                   const uint8_t* sg_q, const float* sg_sc, const uint8_t* su_q,
                                   const float* su_sc, const uint8_t* sd_q, const float* sd_sc,
                                   const float* logits_in, int* ids_out, int nthreads) {
    float* normed = (float*)malloc(sizeof(float) * (size_t)n * H * 2);
    float* mlp = normed + (size_t)n * H;
    orc_rmsnorm_rows(hidden, norm_w, normed, n, H, eps);
    int ties = orc_moe_layer_w4(normed, n, H, I, Is, E, topk, group, router_w, e_bias, norm_topk,
                                routed_scale, gate_q, gate_sc, up_q, up_sc, down_q, down_sc, sg_q,
                                sg_sc, su_q, su_sc, sd_q, sd_sc, logits_in, NULL, ids_out, NULL, mlp,
                                nthreads);
    for (int64_t i = 0; i < (int64_t)n * H; ++i) hidden[i] += mlp[i];
    free(normed);
    return ties;
}

ORC_API int orc_max_threads(void) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}
