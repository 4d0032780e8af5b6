/*
 * CPU oracle for the attention + Gated-DeltaNet hot path.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the product library links, loads or
 * calls this file; it exists so that the parity tests, the smoke check and
 * the bench's CPU-baseline leg have an independent statement of the
 * arithmetic. Every function is a plain-C restatement (own code, fp32) of the
 * reference routine named in its comment; file:line citations are paths inside
 * the TinyTitan source tree.
 *
 * Parity status: PINNED. The delta-rule restatements are checked against the
 * reference's own C kernels compiled from their sources (oracle/_ref) and
 * against the reference's seeded known-answer cases
 * (tests/TinyTitan/CPUEngine/CPUBatchedPrefillTests.swift:165-324); the
 * chunk algebra against benchmark/gdn_chunked_scan.py run in-place; the
 * attention restatements have no reference binary that can run here (Swift /
 * Metal), so they are pinned by their two independent statements agreeing
 * (materialised softmax vs split/merge form) and by the committed vectors.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>
#include <unistd.h>

#define TT_EXPORT __attribute__((visibility("default")))

/* Minimal parallel-for over pthreads (no OpenMP runtime in this image):      */
/* indices [0,n) are handed out one at a time from a shared counter.         */
typedef void (*oracle_body_fn)(int index, void *ctx);
typedef struct { oracle_body_fn fn; void *ctx; int n; int next; pthread_mutex_t mu; } oracle_pf;
static void *oracle_pf_worker(void *p) {
    oracle_pf *pf = (oracle_pf *)p;
    for (;;) {
        pthread_mutex_lock(&pf->mu);
        const int i = pf->next++;
        pthread_mutex_unlock(&pf->mu);
        if (i >= pf->n) break;
        pf->fn(i, pf->ctx);
    }
    return NULL;
}
static void oracle_parallel_for(int n, int threads, oracle_body_fn fn, void *ctx) {
    if (threads <= 1 || n <= 1) { for (int i = 0; i < n; ++i) fn(i, ctx); return; }
    if (threads > n) threads = n;
    if (threads > 256) threads = 256;
    oracle_pf pf; pf.fn = fn; pf.ctx = ctx; pf.n = n; pf.next = 0;
    pthread_mutex_init(&pf.mu, NULL);
    pthread_t tid[256];
    int started = 0;
    for (int t = 0; t < threads - 1; ++t)
        if (pthread_create(&tid[started], NULL, oracle_pf_worker, &pf) == 0) ++started;
    oracle_pf_worker(&pf);
    for (int t = 0; t < started; ++t) pthread_join(tid[t], NULL);
    pthread_mutex_destroy(&pf.mu);
}

/* ------------------------------------------------------------------------ */
/* Decode attention, materialised softmax.                                   */
/* Follows sources/TinyTitanValidation/Support/Reference/Attention/          */
/* Attention.swift:14-114: per q head, all scores, window start              */
/* kvStart = seqLen > window ? seqLen - window : 0, stable softmax, then the  */
/* weighted sum of V. Layouts: q [Hq,hd], k/v [S,Hkv,hd], out [Hq,hd].       */
/* window < 0 means "no window". An empty range leaves the row zero          */
/* (Attention.swift:70-73).                                                  */
/* ------------------------------------------------------------------------ */
TT_EXPORT void tt_oracle_attn_decode(const float *q, const float *k, const float *v,
                                     int head_dim, int n_q_heads, int n_kv_heads,
                                     int seq_len, int window, float scale, float *out) {
    const int group = n_q_heads / n_kv_heads;
    int kv_start = 0;
    if (window >= 0 && seq_len > window) kv_start = seq_len - window;
    const int n = seq_len - kv_start;
    float *scores = (float *)malloc(sizeof(float) * (size_t)(n > 0 ? n : 1));
    for (int h = 0; h < n_q_heads; ++h) {
        float *o = out + (size_t)h * head_dim;
        for (int d = 0; d < head_dim; ++d) o[d] = 0.0f;
        if (n <= 0) continue;
        const int kvh = h / group;
        const float *qr = q + (size_t)h * head_dim;
        for (int p = kv_start; p < seq_len; ++p) {
            const float *kr = k + ((size_t)p * n_kv_heads + kvh) * head_dim;
            float dot = 0.0f;
            for (int d = 0; d < head_dim; ++d) dot += qr[d] * kr[d];
            scores[p - kv_start] = dot * scale;
        }
        float mx = scores[0];
        for (int i = 1; i < n; ++i) if (scores[i] > mx) mx = scores[i];
        float sum = 0.0f;
        for (int i = 0; i < n; ++i) { scores[i] = expf(scores[i] - mx); sum += scores[i]; }
        const float inv = 1.0f / sum;
        for (int i = 0; i < n; ++i) scores[i] *= inv;
        for (int d = 0; d < head_dim; ++d) {
            float acc = 0.0f;
            for (int i = 0; i < n; ++i)
                acc += scores[i] * v[((size_t)(kv_start + i) * n_kv_heads + kvh) * head_dim + d];
            o[d] = acc;
        }
    }
    free(scores);
}

/* ------------------------------------------------------------------------ */
/* Split-KV pass 1: one (q head, chunk) partial, unnormalised (m, d, o[hd]). */
/* Follows sources/TinyTitanCore/Metal/Attention/attention.metal:162-269:    */
/* keys [p_start, p_end), keep[p]==0 skips the key, physical row             */
/* p % ring_capacity when ring_capacity != 0 (:78-83), online softmax in     */
/* fp32. An empty chunk is (-inf, 0, 0) (:225-227).                          */
/* K/V rows are `kv_stride` floats apart (>= Hkv*hd).                        */
/* ------------------------------------------------------------------------ */
TT_EXPORT void tt_oracle_attn_partial(const float *q_row, const float *k, const float *v,
                                      int head_dim, int n_kv_heads, int kv_head,
                                      size_t kv_stride, int p_start, int p_end,
                                      float scale, const uint8_t *keep, int ring_capacity,
                                      float *m_out, float *d_out, float *o_out) {
    (void)n_kv_heads;
    float m_run = -INFINITY, d_run = 0.0f;
    for (int d = 0; d < head_dim; ++d) o_out[d] = 0.0f;
    for (int p = p_start; p < p_end; ++p) {
        if (keep != NULL && keep[p] == 0) continue;
        const size_t phys = ring_capacity ? (size_t)(p % ring_capacity) : (size_t)p;
        const float *kr = k + phys * kv_stride + (size_t)kv_head * head_dim;
        const float *vr = v + phys * kv_stride + (size_t)kv_head * head_dim;
        float s = 0.0f;
        for (int d = 0; d < head_dim; ++d) s = fmaf(q_row[d], kr[d], s);
        s *= scale;
        const float m_new = s > m_run ? s : m_run;
        const float alpha = expf(m_run - m_new);
        const float pe = expf(s - m_new);
        d_run = d_run * alpha + pe;
        for (int d = 0; d < head_dim; ++d) o_out[d] = o_out[d] * alpha + pe * vr[d];
        m_run = m_new;
    }
    *m_out = m_run;
    *d_out = d_run;
}

/* Pass 2 (attention.metal:395-437): M = max m_c; all -inf -> zeros;          */
/* D = sum d_c e^{m_c-M}; out = (sum o_c e^{m_c-M}) * (D>0 ? 1/D : 0).        */
TT_EXPORT void tt_oracle_attn_combine(const float *m, const float *d, const float *o,
                                      int n_chunks, int head_dim, float *out) {
    float mg = -INFINITY;
    for (int c = 0; c < n_chunks; ++c) if (m[c] > mg) mg = m[c];
    if (mg == -INFINITY) {
        for (int i = 0; i < head_dim; ++i) out[i] = 0.0f;
        return;
    }
    float D = 0.0f;
    for (int c = 0; c < n_chunks; ++c) D += d[c] * expf(m[c] - mg);
    const float inv = D > 0.0f ? 1.0f / D : 0.0f;
    for (int i = 0; i < head_dim; ++i) {
        float acc = 0.0f;
        for (int c = 0; c < n_chunks; ++c) acc += o[(size_t)c * head_dim + i] * expf(m[c] - mg);
        out[i] = acc * inv;
    }
}

/* The two passes together with the reference's split geometry               */
/* (sources/TinyTitan/Kernels/Attention/Attention.swift:196-227:             */
/* NC = max(1, min(n_chunks_req, effLen)), chunkLen = ceil(effLen / NC)).    */
TT_EXPORT void tt_oracle_attn_decode_split(const float *q, const float *k, const float *v,
                                           int head_dim, int n_q_heads, int n_kv_heads,
                                           size_t kv_stride, int seq_len, int kv_start,
                                           float scale, const uint8_t *keep,
                                           int ring_capacity, int n_chunks_req, float *out) {
    const int group = n_q_heads / n_kv_heads;
    int eff = seq_len - kv_start;
    if (eff < 1) eff = 1;
    int nc = n_chunks_req < eff ? n_chunks_req : eff;
    if (nc < 1) nc = 1;
    const int chunk_len = (eff + nc - 1) / nc;
    float *m = (float *)malloc(sizeof(float) * (size_t)nc);
    float *d = (float *)malloc(sizeof(float) * (size_t)nc);
    float *o = (float *)malloc(sizeof(float) * (size_t)nc * head_dim);
    for (int h = 0; h < n_q_heads; ++h) {
        for (int c = 0; c < nc; ++c) {
            int ps = kv_start + c * chunk_len;
            int pe = ps + chunk_len;
            if (pe > seq_len) pe = seq_len;
            tt_oracle_attn_partial(q + (size_t)h * head_dim, k, v, head_dim, n_kv_heads,
                                   h / group, kv_stride, ps, pe, scale, keep, ring_capacity,
                                   m + c, d + c, o + (size_t)c * head_dim);
        }
        tt_oracle_attn_combine(m, d, o, nc, head_dim, out + (size_t)h * head_dim);
    }
    free(m); free(d); free(o);
}

/* ------------------------------------------------------------------------ */
/* Causal prefill attention with element strides.                            */
/* Follows sources/TinyTitanValidation/Support/Reference/Attention/          */
/* PrefillAttentionRef.swift:59-101: abs_q = start + t;                      */
/* first = window==0 ? 0 : max(0, abs_q+1-window); last = min(kvValid,       */
/* abs_q+1); out = softmax(scale*q.k) v, denom>0 ? acc/denom : 0.            */
/* out is tight [T, Hq, hd].                                                 */
/* ------------------------------------------------------------------------ */
typedef struct {
    const float *q, *k, *v; size_t q_stride, kv_stride;
    int head_dim, q_heads, kv_heads, start, kv_valid, window; float scale; float *out;
} oracle_prefill_ctx;

static void oracle_prefill_row(int t, void *p) {
    const oracle_prefill_ctx *c = (const oracle_prefill_ctx *)p;
    const int per = c->q_heads / c->kv_heads, head_dim = c->head_dim;
    const int abs_q = c->start + t;
    int first = 0;
    if (c->window != 0) { first = abs_q + 1 - c->window; if (first < 0) first = 0; }
    const int last = abs_q + 1 < c->kv_valid ? abs_q + 1 : c->kv_valid;
    const int n = last - first;
    float *scores = (float *)malloc(sizeof(float) * (size_t)(n > 0 ? n : 1));
    for (int h = 0; h < c->q_heads; ++h) {
        const int kvh = h / per;
        const float *qr = c->q + (size_t)t * c->q_stride + (size_t)h * head_dim;
        float *o = c->out + ((size_t)t * c->q_heads + h) * head_dim;
        float mx = -INFINITY;
        for (int key = first; key < last; ++key) {
            const float *kr = c->k + (size_t)key * c->kv_stride + (size_t)kvh * head_dim;
            float s = 0.0f;
            for (int d = 0; d < head_dim; ++d) s += qr[d] * kr[d];
            s *= c->scale;
            scores[key - first] = s;
            if (s > mx) mx = s;
        }
        float denom = 0.0f;
        for (int i = 0; i < n; ++i) { scores[i] = expf(scores[i] - mx); denom += scores[i]; }
        for (int d = 0; d < head_dim; ++d) {
            float acc = 0.0f;
            for (int i = 0; i < n; ++i)
                acc += scores[i] * c->v[(size_t)(first + i) * c->kv_stride + (size_t)kvh * head_dim + d];
            o[d] = denom > 0.0f ? acc / denom : 0.0f;
        }
    }
    free(scores);
}

TT_EXPORT void tt_oracle_attn_prefill(const float *q, const float *k, const float *v,
                                      size_t q_stride, size_t kv_stride,
                                      int head_dim, int q_heads, int kv_heads,
                                      int start, int chunk, int kv_valid, int window,
                                      float scale, int threads, float *out) {
    oracle_prefill_ctx c = {q, k, v, q_stride, kv_stride, head_dim, q_heads, kv_heads,
                            start, kv_valid, window, scale, out};
    oracle_parallel_for(chunk, threads, oracle_prefill_row, &c);
}

/* ------------------------------------------------------------------------ */
/* CPU-engine decode attention (the timed CPU baseline for decode).          */
/* Follows sources/TinyTitan/CPUEngine/CPUQwen35.swift:313-348 and           */
/* CPUTensorOps.swift:103-113: fp32 KV [pos][Hkv*hd], per head scores,       */
/* softmaxInPlace (peak, exp, sum, scale by 1/total), weight==0 skipped.     */
/* `threads` > 1 spreads the heads over OpenMP threads (the reference runs   */
/* this loop on one thread).                                                 */
/* ------------------------------------------------------------------------ */
typedef struct {
    const float *query, *keys, *values; int heads, kv_heads, dim, cached; float scale; float *out;
} oracle_cpuattn_ctx;

static void oracle_cpuattn_head(int head, void *p) {
    const oracle_cpuattn_ctx *c = (const oracle_cpuattn_ctx *)p;
    const int group = c->heads / c->kv_heads, dim = c->dim, cached = c->cached, kv_heads = c->kv_heads;
    float *scores = (float *)malloc(sizeof(float) * (size_t)(cached > 0 ? cached : 1));
    const int kvh = head / group;
    const size_t qb = (size_t)head * dim;
    for (int i = 0; i < dim; ++i) c->out[qb + i] = 0.0f;
    for (int step = 0; step < cached; ++step) {
        const size_t base = (size_t)step * kv_heads * dim + (size_t)kvh * dim;
        float total = 0.0f;
        for (int i = 0; i < dim; ++i) total += c->keys[base + i] * c->query[qb + i];
        scores[step] = total * c->scale;
    }
    if (cached > 0) {
        float peak = scores[0];
        for (int i = 1; i < cached; ++i) if (scores[i] > peak) peak = scores[i];
        float total = 0.0f;
        for (int i = 0; i < cached; ++i) { scores[i] = expf(scores[i] - peak); total += scores[i]; }
        const float inv = 1.0f / total;
        for (int i = 0; i < cached; ++i) scores[i] *= inv;
    }
    for (int step = 0; step < cached; ++step) {
        const float w = scores[step];
        if (w == 0.0f) continue;
        const size_t base = (size_t)step * kv_heads * dim + (size_t)kvh * dim;
        for (int i = 0; i < dim; ++i) c->out[qb + i] += w * c->values[base + i];
    }
    free(scores);
}

TT_EXPORT void tt_oracle_cpu_engine_attention(const float *query, const float *keys,
                                              const float *values, int heads, int kv_heads,
                                              int dim, int cached, float scale,
                                              int threads, float *out) {
    oracle_cpuattn_ctx c = {query, keys, values, heads, kv_heads, dim, cached, scale, out};
    oracle_parallel_for(heads, threads, oracle_cpuattn_head, &c);
}

/* Many independent sessions of the same decode attention: (session, head)   */
/* pairs over threads. Session s has `cached[s]` rows starting at row        */
/* `row_base[s]` of the shared fp32 key/value stores.                         */
typedef struct {
    const float *query, *keys, *values; const int *cached; const long long *row_base;
    int heads, kv_heads, dim; float scale; float *out;
} oracle_cpuattn_batch_ctx;

static void oracle_cpuattn_batch_item(int idx, void *p) {
    const oracle_cpuattn_batch_ctx *b = (const oracle_cpuattn_batch_ctx *)p;
    const int s = idx / b->heads, head = idx % b->heads;
    oracle_cpuattn_ctx c = {b->query + (size_t)s * b->heads * b->dim,
                            b->keys + (size_t)b->row_base[s] * b->kv_heads * b->dim,
                            b->values + (size_t)b->row_base[s] * b->kv_heads * b->dim,
                            b->heads, b->kv_heads, b->dim, b->cached[s], b->scale,
                            b->out + (size_t)s * b->heads * b->dim};
    oracle_cpuattn_head(head, &c);
}

TT_EXPORT void tt_oracle_cpu_engine_attention_sessions(const float *query, const float *keys,
                                                       const float *values, const int *cached,
                                                       const long long *row_base, int sessions,
                                                       int heads, int kv_heads, int dim,
                                                       float scale, int threads, float *out) {
    oracle_cpuattn_batch_ctx b = {query, keys, values, cached, row_base, heads, kv_heads, dim, scale, out};
    oracle_parallel_for(sessions * heads, threads, oracle_cpuattn_batch_item, &b);
}

/* Plain row-major GEMM used where the reference calls its BLAS wrapper       */
/* (sources/TinyTitanKernelsC/include/tinytitan_kernels.h:76-78):             */
/* out[rows,cols] = a[rows,inner] * (tb ? b[cols,inner]^T : b[inner,cols]).   */
static void oracle_sgemm(int tb, int rows, int cols, int inner,
                         const float *a, const float *b, float *out) {
    if (tb) {
        for (int i = 0; i < rows; ++i)
            for (int j = 0; j < cols; ++j) {
                float acc = 0.0f;
                const float *ar = a + (size_t)i * inner, *br = b + (size_t)j * inner;
                for (int l = 0; l < inner; ++l) acc += ar[l] * br[l];
                out[(size_t)i * cols + j] = acc;
            }
    } else {
        for (int i = 0; i < rows; ++i) {
            float *orow = out + (size_t)i * cols;
            for (int j = 0; j < cols; ++j) orow[j] = 0.0f;
            for (int l = 0; l < inner; ++l) {
                const float av = a[(size_t)i * inner + l];
                const float *br = b + (size_t)l * cols;
                for (int j = 0; j < cols; ++j) orow[j] += av * br[j];
            }
        }
    }
}

/* ------------------------------------------------------------------------ */
/* CPU-engine batched prefill attention for one head (the timed CPU          */
/* baseline for prefill). Follows                                            */
/* sources/TinyTitan/CPUEngine/CPUQwen35+BatchAttention.swift:119-178:       */
/* gather the head, scores = Q K^T, per-row column limit base+row, softmax,  */
/* zero the tail, result = P V. query [tokens, heads*dim]; caches            */
/* [positions, kv_heads*dim]; result [tokens, dim].                          */
/* ------------------------------------------------------------------------ */
TT_EXPORT int tt_oracle_cpu_engine_attention_head(const float *query, int tokens, int heads,
                                                  int head, int dim, const float *cached_keys,
                                                  const float *cached_values, int positions,
                                                  int kv_heads, int kv_head, int base_position,
                                                  float scale, float *result) {
    const size_t kw = (size_t)kv_heads * dim;
    float *qh = (float *)malloc(sizeof(float) * (size_t)tokens * dim);
    float *kh = (float *)malloc(sizeof(float) * (size_t)positions * dim);
    float *vh = (float *)malloc(sizeof(float) * (size_t)positions * dim);
    float *scores = (float *)malloc(sizeof(float) * (size_t)tokens * positions);
    if (!qh || !kh || !vh || !scores) { free(qh); free(kh); free(vh); free(scores); return 1; }
    for (int r = 0; r < tokens; ++r)
        memcpy(qh + (size_t)r * dim, query + (size_t)r * heads * dim + (size_t)head * dim,
               sizeof(float) * (size_t)dim);
    for (int p = 0; p < positions; ++p) {
        memcpy(kh + (size_t)p * dim, cached_keys + p * kw + (size_t)kv_head * dim, sizeof(float) * (size_t)dim);
        memcpy(vh + (size_t)p * dim, cached_values + p * kw + (size_t)kv_head * dim, sizeof(float) * (size_t)dim);
    }
    oracle_sgemm(1, tokens, positions, dim, qh, kh, scores);
    int rc = 0;
    for (int r = 0; r < tokens; ++r) {
        const int limit = base_position + r;
        if (limit >= positions) { rc = 2; break; }
        float *row = scores + (size_t)r * positions;
        float peak = -INFINITY;
        for (int c = 0; c <= limit; ++c) { row[c] *= scale; if (row[c] > peak) peak = row[c]; }
        float total = 0.0f;
        for (int c = 0; c <= limit; ++c) { row[c] = expf(row[c] - peak); total += row[c]; }
        const float norm = 1.0f / total;
        for (int c = 0; c <= limit; ++c) row[c] *= norm;
        for (int c = limit + 1; c < positions; ++c) row[c] = 0.0f;
    }
    if (rc == 0) oracle_sgemm(0, tokens, dim, positions, scores, vh, result);
    free(qh); free(kh); free(vh); free(scores);
    return rc;
}

/* All heads of the batched prefill attention, heads over OpenMP threads;    */
/* result [tokens, heads*dim].                                               */
typedef struct {
    const float *query, *ck, *cv; int tokens, heads, dim, positions, kv_heads, base_position;
    float scale; float *result; int rc;
} oracle_attnbatch_ctx;

static void oracle_attnbatch_head(int head, void *p) {
    oracle_attnbatch_ctx *c = (oracle_attnbatch_ctx *)p;
    const int group = c->heads / c->kv_heads;
    float *tmp = (float *)malloc(sizeof(float) * (size_t)c->tokens * c->dim);
    int rc = tt_oracle_cpu_engine_attention_head(c->query, c->tokens, c->heads, head, c->dim, c->ck,
                                                 c->cv, c->positions, c->kv_heads, head / group,
                                                 c->base_position, c->scale, tmp);
    if (rc == 0) {
        for (int r = 0; r < c->tokens; ++r)
            memcpy(c->result + (size_t)r * c->heads * c->dim + (size_t)head * c->dim,
                   tmp + (size_t)r * c->dim, sizeof(float) * (size_t)c->dim);
    } else {
        __atomic_store_n(&c->rc, rc, __ATOMIC_RELAXED);
    }
    free(tmp);
}

TT_EXPORT int tt_oracle_cpu_engine_attention_batch(const float *query, int tokens, int heads,
                                                   int dim, const float *cached_keys,
                                                   const float *cached_values, int positions,
                                                   int kv_heads, int base_position, float scale,
                                                   int threads, float *result) {
    oracle_attnbatch_ctx c = {query, cached_keys, cached_values, tokens, heads, dim, positions,
                              kv_heads, base_position, scale, result, 0};
    oracle_parallel_for(heads, threads, oracle_attnbatch_head, &c);
    return c.rc;
}

/* ------------------------------------------------------------------------ */
/* Gated delta rule, one token, all heads (CPU-engine form).                 */
/* Follows sources/TinyTitanKernelsC/delta_rule.c:26-90 (scalar branch):     */
/* beta = sigmoid(b), decay = exp(-exp(decayLog) * softplus(a + decayBias))  */
/* with softplus(x) = log1p(exp(-|x|)) + max(x, 0) (:22-24), key head        */
/* = head / (heads/keyHeads); row *= decay; stored = row.k;                  */
/* corr = (v - stored)*beta; row += k*corr; readout = (row.q) * inverse.     */
/* ------------------------------------------------------------------------ */
static float oracle_softplus_c(float x) { return log1pf(expf(-fabsf(x))) + fmaxf(x, 0.0f); }

TT_EXPORT void tt_oracle_delta_rule(const float *query, const float *key, const float *value,
                                    const float *a, const float *b, const float *decay_log,
                                    const float *decay_bias, size_t heads, size_t key_heads,
                                    size_t dk, size_t dv, float inverse, float *state,
                                    float *readout) {
    if (heads == 0 || key_heads == 0 || dk == 0 || dv == 0 || heads % key_heads != 0) return;
    const size_t repeats = heads / key_heads;
    for (size_t head = 0; head < heads; ++head) {
        const float beta = 1.0f / (1.0f + expf(-b[head]));
        const float decay = expf(-expf(decay_log[head]) * oracle_softplus_c(a[head] + decay_bias[head]));
        const float *kr = key + (head / repeats) * dk;
        const float *qr = query + (head / repeats) * dk;
        for (size_t i = 0; i < dv; ++i) {
            float *row = state + (head * dv + i) * dk;
            float stored = 0.0f;
            for (size_t c = 0; c < dk; ++c) { row[c] *= decay; stored += row[c] * kr[c]; }
            const float corr = (value[head * dv + i] - stored) * beta;
            float sum = 0.0f;
            for (size_t c = 0; c < dk; ++c) { row[c] += kr[c] * corr; sum += row[c] * qr[c]; }
            readout[head * dv + i] = sum * inverse;
        }
    }
}

/* ------------------------------------------------------------------------ */
/* Gated delta rule, GPU-kernel form, `rows` tokens sequentially.            */
/* Follows sources/TinyTitanCore/Metal/GDN/gdn.metal:529-669 and             */
/* sources/TinyTitanValidation/Support/Reference/GDN/GDNReference.swift:     */
/* 84-107: conv_out row = [q: Hk*Dk | k: Hk*Dk | v: Hv*Dv], a/b [rows,Hv],   */
/* softplus(x) = x>20 ? x : log(1+exp(x)) (gdn.metal:134-138),               */
/* g = a_preexp ? exp(A*sp) : exp(-exp(A_log)*sp) (:151-157),                */
/* hk = v_tiled ? h % Hk : h / (Hv/Hk) (:144-149); y = row.q * readout_scale */
/* All inputs are fp32 here; the caller rounds them to the storage types     */
/* first and rounds y afterwards (GDNReference.swift:105). checkpoint, when  */
/* non-NULL, receives the state after row 0 (gdn.metal:658-663).             */
/* ------------------------------------------------------------------------ */
TT_EXPORT void tt_oracle_gdn_step_rows(const float *conv_out, size_t row_stride,
                                       const float *a, const float *b, const float *a_log,
                                       const float *dt_bias, int hk_heads, int hv_heads,
                                       int dk, int dv, int rows, int a_preexp, int v_tiled,
                                       float readout_scale, float *state, float *checkpoint,
                                       float *y) {
    for (int t = 0; t < rows; ++t) {
        const float *row_in = conv_out + (size_t)t * row_stride;
        for (int h = 0; h < hv_heads; ++h) {
            const int hk = v_tiled ? h % hk_heads : h / (hv_heads / hk_heads);
            const float *q = row_in + (size_t)hk * dk;
            const float *k = row_in + (size_t)hk_heads * dk + (size_t)hk * dk;
            const float *v = row_in + (size_t)2 * hk_heads * dk + (size_t)h * dv;
            const float x = a[(size_t)t * hv_heads + h] + dt_bias[h];
            const float sp = x > 20.0f ? x : logf(1.0f + expf(x));
            const float g = a_preexp ? expf(a_log[h] * sp) : expf(-expf(a_log[h]) * sp);
            const float beta = 1.0f / (1.0f + expf(-b[(size_t)t * hv_heads + h]));
            for (int i = 0; i < dv; ++i) {
                float *srow = state + ((size_t)h * dv + i) * dk;
                float kv = 0.0f;
                for (int c = 0; c < dk; ++c) { srow[c] *= g; kv += srow[c] * k[c]; }
                const float delta = (v[i] - kv) * beta;
                float o = 0.0f;
                for (int c = 0; c < dk; ++c) { srow[c] += k[c] * delta; o += srow[c] * q[c]; }
                y[(size_t)t * hv_heads * dv + (size_t)h * dv + i] = o * readout_scale;
            }
        }
        if (t == 0 && checkpoint != NULL)
            memcpy(checkpoint, state, sizeof(float) * (size_t)hv_heads * dv * dk);
    }
}

/* ------------------------------------------------------------------------ */
/* Chunked delta rule, one head, `tokens` tokens, alpha/beta precomputed.    */
/* Follows sources/TinyTitanKernelsC/gdn_chunk.c:72-195 and the algebra of   */
/* benchmark/gdn_chunked_scan.py:70-97: gather [K;Q]; A_t = prod alpha;      */
/* products = S0 [K;Q]^T; gram = K [K;Q]^T; triangular pass with the decay   */
/* ratio formed as a backward product of alphas (never A_t/A_s, :141-147);   */
/* state = A_C S0 + sum_s (A_C/A_s) c_s k_s^T.                               */
/* Returns 0, or 1 when scratch could not be allocated.                      */
/* ------------------------------------------------------------------------ */
TT_EXPORT int tt_oracle_delta_rule_chunk(const float *queries, size_t q_stride,
                                         const float *keys, size_t k_stride,
                                         const float *values, size_t v_stride,
                                         const float *alphas, size_t a_stride,
                                         const float *betas, size_t b_stride,
                                         size_t tokens, size_t dk, size_t dv,
                                         float *state, float *readouts, size_t r_stride) {
    if (tokens == 0 || dk == 0 || dv == 0) return 0;
    const size_t C = tokens, C2 = 2 * tokens;
    float *kq = (float *)malloc(sizeof(float) * C2 * dk);
    float *prod = (float *)malloc(sizeof(float) * dv * C2);
    float *gram = (float *)malloc(sizeof(float) * C * C2);
    float *corr = (float *)malloc(sizeof(float) * C * dv);
    float *wgt = (float *)malloc(sizeof(float) * dv * C);
    float *upd = (float *)malloc(sizeof(float) * dv * dk);
    float *cum = (float *)malloc(sizeof(float) * C);
    if (!kq || !prod || !gram || !corr || !wgt || !upd || !cum) {
        free(kq); free(prod); free(gram); free(corr); free(wgt); free(upd); free(cum);
        return 1;
    }
    for (size_t t = 0; t < C; ++t) {
        memcpy(kq + t * dk, keys + t * k_stride, sizeof(float) * dk);
        memcpy(kq + (C + t) * dk, queries + t * q_stride, sizeof(float) * dk);
    }
    float run = 1.0f;
    for (size_t t = 0; t < C; ++t) { run *= alphas[t * a_stride]; cum[t] = run; }
    oracle_sgemm(1, (int)dv, (int)C2, (int)dk, state, kq, prod);
    oracle_sgemm(1, (int)C, (int)C2, (int)dk, kq, kq, gram);
    for (size_t t = 0; t < C; ++t) {
        const float prev = t > 0 ? cum[t - 1] : 1.0f;
        const float alpha = alphas[t * a_stride], beta = betas[t * b_stride];
        if (t > 0)
            for (size_t i = 0; i < dv; ++i) { prod[i * C2 + t] *= prev; prod[i * C2 + C + t] *= prev; }
        float w = 1.0f;
        for (size_t s = t; s-- > 0;) {
            if (s + 1 < t) w *= alphas[(s + 1) * a_stride];
            const float kw = w * gram[s * C2 + t], qw = w * gram[s * C2 + C + t];
            const float *cs = corr + s * dv;
            for (size_t i = 0; i < dv; ++i) { prod[i * C2 + t] += kw * cs[i]; prod[i * C2 + C + t] += qw * cs[i]; }
        }
        const float kqd = gram[t * C2 + C + t];
        for (size_t i = 0; i < dv; ++i) {
            const float c = beta * (values[t * v_stride + i] - alpha * prod[i * C2 + t]);
            corr[t * dv + i] = c;
            readouts[t * r_stride + i] = alpha * prod[i * C2 + C + t] + c * kqd;
        }
    }
    float w = 1.0f;
    for (size_t s = C; s-- > 0;) {
        if (s + 1 < C) w *= alphas[(s + 1) * a_stride];
        for (size_t i = 0; i < dv; ++i) wgt[i * C + s] = w * corr[s * dv + i];
    }
    oracle_sgemm(0, (int)dv, (int)dk, (int)C, wgt, kq, upd);
    const float last = cum[C - 1];
    for (size_t i = 0; i < dv * dk; ++i) state[i] = last * state[i] + upd[i];
    free(kq); free(prod); free(gram); free(corr); free(wgt); free(upd); free(cum);
    return 0;
}

/* ------------------------------------------------------------------------ */
/* Driver shaped like the reference's batched CPU GDN                        */
/* (sources/TinyTitan/CPUEngine/CPUQwen35+BatchGDN.swift:192-253): heads are */
/* split over threads, each head walks the prompt in chunks of `chunk`       */
/* tokens through `chunk_fn` (the oracle's or the compiled reference's       */
/* chunk kernel). q/k [T, Hk*dk], v [T, Hv*dv], alpha/beta [T, Hv],          */
/* state [Hv, dv, dk], y [T, Hv*dv]; head h reads key head h/(Hv/Hk).        */
/* ------------------------------------------------------------------------ */
typedef int (*tt_chunk_fn)(const float *, size_t, const float *, size_t, const float *, size_t,
                           const float *, size_t, const float *, size_t, size_t, size_t, size_t,
                           float *, float *, size_t);

typedef struct {
    tt_chunk_fn fn; const float *q, *k, *v, *alpha, *beta;
    int tokens, hk_heads, hv_heads, dk, dv, chunk; float *state, *y; int rc;
} oracle_scan_ctx;

static void oracle_scan_head(int h, void *p) {
    oracle_scan_ctx *c = (oracle_scan_ctx *)p;
    const int rep = c->hv_heads / c->hk_heads, hk = h / rep;
    const size_t kw = (size_t)c->hk_heads * c->dk, vw = (size_t)c->hv_heads * c->dv;
    for (int t0 = 0; t0 < c->tokens; t0 += c->chunk) {
        const int n = c->tokens - t0 < c->chunk ? c->tokens - t0 : c->chunk;
        int rc = c->fn(c->q + (size_t)t0 * kw + (size_t)hk * c->dk, kw,
                       c->k + (size_t)t0 * kw + (size_t)hk * c->dk, kw,
                       c->v + (size_t)t0 * vw + (size_t)h * c->dv, vw,
                       c->alpha + (size_t)t0 * c->hv_heads + h, (size_t)c->hv_heads,
                       c->beta + (size_t)t0 * c->hv_heads + h, (size_t)c->hv_heads,
                       (size_t)n, (size_t)c->dk, (size_t)c->dv,
                       c->state + (size_t)h * c->dv * c->dk,
                       c->y + (size_t)t0 * vw + (size_t)h * c->dv, vw);
        if (rc != 0) __atomic_store_n(&c->rc, rc, __ATOMIC_RELAXED);
    }
}

TT_EXPORT int tt_oracle_gdn_scan_heads(tt_chunk_fn chunk_fn, const float *q, const float *k,
                                       const float *v, const float *alpha, const float *beta,
                                       int tokens, int hk_heads, int hv_heads, int dk, int dv,
                                       int chunk, int threads, float *state, float *y) {
    oracle_scan_ctx c = {chunk_fn != NULL ? chunk_fn : tt_oracle_delta_rule_chunk, q, k, v, alpha,
                         beta, tokens, hk_heads, hv_heads, dk, dv, chunk, state, y, 0};
    oracle_parallel_for(hv_heads, threads, oracle_scan_head, &c);
    return c.rc;
}

/* One-token rule over many independent sessions, (session, head) pairs over */
/* threads, through `rule_fn` shaped like tinytitan_delta_rule_range         */
/* (tinytitan_kernels.h:104-121); NULL selects the oracle's own rule.        */
typedef void (*tt_rule_range_fn)(const float *, const float *, const float *, const float *,
                                 const float *, const float *, const float *, size_t, size_t,
                                 size_t, size_t, float, size_t, size_t, float *, float *);

static void oracle_delta_rule_head(const float *query, const float *key, const float *value,
                                   const float *a, const float *b, const float *decay_log,
                                   const float *decay_bias, size_t heads, size_t key_heads,
                                   size_t dk, size_t dv, float inverse, size_t first, size_t count,
                                   float *state, float *readout) {
    const size_t repeats = heads / key_heads;
    for (size_t head = first; head < first + count; ++head) {
        const float beta = 1.0f / (1.0f + expf(-b[head]));
        const float decay = expf(-expf(decay_log[head]) * oracle_softplus_c(a[head] + decay_bias[head]));
        const float *kr = key + (head / repeats) * dk;
        const float *qr = query + (head / repeats) * dk;
        for (size_t i = 0; i < dv; ++i) {
            float *row = state + (head * dv + i) * dk;
            float stored = 0.0f;
            for (size_t c = 0; c < dk; ++c) { row[c] *= decay; stored += row[c] * kr[c]; }
            const float corr = (value[head * dv + i] - stored) * beta;
            float sum = 0.0f;
            for (size_t c = 0; c < dk; ++c) { row[c] += kr[c] * corr; sum += row[c] * qr[c]; }
            readout[head * dv + i] = sum * inverse;
        }
    }
}

typedef struct {
    tt_rule_range_fn fn; const float *query, *key, *value, *a, *b, *decay_log, *decay_bias;
    int heads, key_heads, dk, dv; float inverse; float *state, *readout;
} oracle_rule_ctx;

static void oracle_rule_item(int idx, void *p) {
    const oracle_rule_ctx *c = (const oracle_rule_ctx *)p;
    const int s = idx / c->heads, h = idx % c->heads;
    c->fn(c->query + (size_t)s * c->key_heads * c->dk, c->key + (size_t)s * c->key_heads * c->dk,
          c->value + (size_t)s * c->heads * c->dv, c->a + (size_t)s * c->heads,
          c->b + (size_t)s * c->heads, c->decay_log, c->decay_bias, (size_t)c->heads,
          (size_t)c->key_heads, (size_t)c->dk, (size_t)c->dv, c->inverse, (size_t)h, 1,
          c->state + (size_t)s * c->heads * c->dv * c->dk, c->readout + (size_t)s * c->heads * c->dv);
}

TT_EXPORT void tt_oracle_delta_rule_sessions(tt_rule_range_fn rule_fn, const float *query,
                                             const float *key, const float *value, const float *a,
                                             const float *b, const float *decay_log,
                                             const float *decay_bias, int sessions, int heads,
                                             int key_heads, int dk, int dv, float inverse,
                                             int threads, float *state, float *readout) {
    oracle_rule_ctx c = {rule_fn != NULL ? rule_fn : oracle_delta_rule_head, query, key, value, a, b,
                         decay_log, decay_bias, heads, key_heads, dk, dv, inverse, state, readout};
    oracle_parallel_for(sessions * heads, threads, oracle_rule_item, &c);
}

TT_EXPORT int tt_oracle_max_threads(void) {
    const long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}
