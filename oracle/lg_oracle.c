/* lg_oracle.c -- TEST INFRASTRUCTURE: a CPU restatement of the little-gemma decode step.
 *
 * Scalar f32, sums in index order, one position at a time.  It exists to check the CUDA
 * backend; only tests, the smoke check and the CPU-baseline leg of the benchmark may load it.
 * Its own correctness is pinned by comparing it, bit for bit, with the compiled reference CPU
 * backend (oracle/_ref) on seeded models and by golden vectors generated from that backend
 * (tests/golden).  Each routine names the reference lines whose arithmetic it restates.
 */
#ifdef _OPENMP
#include <omp.h>
#endif
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
#include "lg_host.h"

/* The host set-up code calls into a backend; this library is a host-memory backend. */
const int model_kv_host = 1;
int (*model_pick)(const float *, int) = NULL;
int  mtp_draft_device(struct mtp *t, const struct model *m, const struct kvcache *kv, int a, int b)
{ (void)t; (void)m; (void)kv; (void)a; (void)b; return -1; }
int  mtp_draft_chain_device(struct mtp *t, const struct model *m, const struct kvcache *kv, int a, int b)
{ (void)t; (void)m; (void)kv; (void)a; (void)b; return -1; }
void mtp_free_device(struct mtp *t) { (void)t; }

float lg_half_to_float(uint16_t h);

/* f32 -> f16, round to nearest even (what cvt.rn.f16.f32 does; reference
 * src/cpu/model-cpu.c:185-200 reaches the same bits by a scaling trick). */
static uint16_t half_of(float f) {
    uint32_t x; memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u, a = x & 0x7FFFFFFFu;
    if (a > 0x7F800000u) return (uint16_t)(sign | 0x7E00u);
    if (a >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);          /* rounds to inf */
    if (a < 0x33000001u) return (uint16_t)sign;                        /* below half the smallest subnormal */
    uint32_t e = a >> 23, mant = (a & 0x7FFFFFu) | 0x800000u;
    int shift = e >= 113 ? 13 : (int)(126 - e);                       /* subnormal halves shift further */
    uint32_t keep = mant >> shift, rem = mant & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (keep & 1))) keep++;
    uint32_t out = e >= 113 ? ((e - 112) << 10) + (keep - 0x400u) : keep;
    return (uint16_t)(sign | out);
}

struct orc {
    struct gguf_context *g;
    struct model m;
    struct mtp *head;
    int max_seq, mtp_n, kv_f16_all;
    int *seq, *kvdim, *round16;           /* per layer; seq 0 = borrows */
    float **k, **v;                        /* rows kept as f32 (already rounded through f16 where stored so) */
    float *logits, *trace;                 /* trace: hidden after each layer of the last forward */
};

/* ---- small math (reference src/cpu/model-cpu.c:78-119) ---- */
static void rms(float *o, const float *x, const float *w, int n, float eps) {
    float ss = 0.0f;
    for (int i = 0; i < n; i++) ss += x[i] * x[i];
    float s = 1.0f / sqrtf(ss / (float)n + eps);
    if (w) for (int i = 0; i < n; i++) o[i] = x[i] * s * w[i];
    else   for (int i = 0; i < n; i++) o[i] = x[i] * s;
}
static void rope(float *v, int d, int pos, float base, const float *div) {
    int half = d / 2;
    for (int i = 0; i < half; i++) {
        float ang = (float)pos * powf(base, -2.0f * (float)i / (float)d) / (div ? div[i] : 1.0f);
        float c = cosf(ang), s = sinf(ang), a = v[i], b = v[i + half];
        v[i] = a * c - b * s;
        v[i + half] = a * s + b * c;
    }
}
static float gelu_tanh(float x) {
    return 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}
static void softmax_inplace(float *x, int n) {
    float mx = x[0], sum = 0.0f;
    for (int i = 1; i < n; i++) if (x[i] > mx) mx = x[i];
    for (int i = 0; i < n; i++) { x[i] = expf(x[i] - mx); sum += x[i]; }
    for (int i = 0; i < n; i++) x[i] /= sum;
}
/* out = W x, each row decoded then summed in index order (model-cpu.c:147-164) */
static void matvec(float *out, const struct gguf_tensor *t, const float *x, int k, int rows) {
    size_t rb = ggml_nbytes(t->type, k);
    #pragma omp parallel
    {
        float *w = malloc((size_t)k * sizeof(float));
        #pragma omp for schedule(static)
        for (int r = 0; r < rows; r++) {
            dequantize_into(t->type, (const uint8_t *)t->data + (size_t)r * rb, w, k);
            float s = 0.0f;
            for (int j = 0; j < k; j++) s += w[j] * x[j];
            out[r] = s;
        }
        free(w);
    }
}
static const struct gguf_tensor *T(const struct gguf_context *g, int L, const char *leaf) {
    char n[96];
    if (L >= 0) snprintf(n, sizeof n, "blk.%d.%s", L, leaf); else snprintf(n, sizeof n, "%s", leaf);
    return gguf_find_tensor(g, n);
}
static const float *F(const struct gguf_context *g, int L, const char *leaf) {
    const struct gguf_tensor *t = T(g, L, leaf);
    return t ? (const float *)t->data : NULL;
}
static int kv_owner(const struct model *m, int L) {                  /* model-cpu.c:175-179 */
    if (L < m->cfg.n_kv_start) return L;
    return m->cfg.n_kv_start - (m->is_local[L] ? 2 : 1);
}

/* softmax(q.K) V over positions [t0, t1] of one cache, scale 1.0 (model-cpu.c:380-400) */
static void attend(float *out, const float *q, int n_head, int hd, int gqa, const float *K, const float *V,
                   int kvdim, int seq, int t0, int t1, float *att) {
    for (int h = 0; h < n_head; h++) {
        const float *qh = q + h * hd;
        size_t col = (size_t)(h / gqa) * hd;
        for (int t = t0; t <= t1; t++) {
            const float *kr = K + (size_t)(t % seq) * kvdim + col;
            float s = 0.0f;
            for (int i = 0; i < hd; i++) s += qh[i] * kr[i];
            att[t - t0] = s;
        }
        softmax_inplace(att, t1 - t0 + 1);
        float *o = out + h * hd;
        for (int i = 0; i < hd; i++) o[i] = 0.0f;
        for (int t = t0; t <= t1; t++) {
            const float *vr = V + (size_t)(t % seq) * kvdim + col;
            float a = att[t - t0];
            for (int i = 0; i < hd; i++) o[i] += a * vr[i];
        }
    }
}

/* One position through the decoder (model-cpu.c:267-294 PLE inputs, :301-448 layers and head,
 * :450-457 embedding scale).  logits == NULL skips the head. */
/* `row` != NULL: a media position -- the given embedding row enters as it is and the per-layer table row of
 * token 0 (padding) is used (model-cpu.c:459-465, 489-497) */
static void forward_row(struct orc *o, int tok, const float *row, int pos, float *logits) {
    struct model *m = &o->m;
    const struct config *c = &m->cfg;
    const struct gguf_context *g = o->g;
    const int ne = c->n_embd, H = c->n_head, ple = c->n_embd_per_layer;
    int qmax = 0, kvmax = 0;
    for (int L = 0; L < c->n_layer; L++) {
        if (H * m->head_dim[L] > qmax) qmax = H * m->head_dim[L];
        if (m->n_head_kv[L] * m->head_dim[L] > kvmax) kvmax = m->n_head_kv[L] * m->head_dim[L];
    }
    float *x = dequantize_row(T(g, -1, "token_embd.weight"), tok, ne);
    float *h = malloc(sizeof(float) * ne), *q = malloc(sizeof(float) * qmax), *xb = malloc(sizeof(float) * qmax);
    float *kb = malloc(sizeof(float) * kvmax), *vb = malloc(sizeof(float) * kvmax), *ob = malloc(sizeof(float) * ne);
    float *g1 = malloc(sizeof(float) * c->n_ff), *g2 = malloc(sizeof(float) * c->n_ff);
    float *att = malloc(sizeof(float) * (pos + 1)), *pg = malloc(sizeof(float) * (ple > 0 ? ple : 1));
    for (int i = 0; i < ne; i++) x[i] *= sqrtf((float)ne);
    if (row) memcpy(x, row, sizeof(float) * ne);

    float *ipl = NULL;                                            /* per-layer inputs */
    const struct gguf_tensor *pte = ple > 0 ? T(g, -1, "per_layer_token_embd.weight") : NULL;
    if (pte) {
        int total = ple * c->n_layer;
        float *trow = dequantize_row(pte, tok, total);
        ipl = malloc(sizeof(float) * total);
        for (int i = 0; i < total; i++) trow[i] *= sqrtf((float)ple);
        matvec(ipl, T(g, -1, "per_layer_model_proj.weight"), x, ne, total);
        float ps = 1.0f / sqrtf((float)ne);
        for (int i = 0; i < total; i++) ipl[i] *= ps;
        for (int L = 0; L < c->n_layer; L++)
            rms(ipl + L * ple, ipl + L * ple, F(g, -1, "per_layer_proj_norm.weight"), ple, c->rms_eps);
        float r2 = 1.0f / sqrtf(2.0f);
        for (int i = 0; i < total; i++) ipl[i] = (ipl[i] + trow[i]) * r2;
        free(trow);
    }
    const float *rdiv = F(g, -1, "rope_freqs.weight");

    for (int L = 0; L < c->n_layer; L++) {
        const int local = m->is_local[L], hd = m->head_dim[L], nkv = m->n_head_kv[L];
        const int qd = H * hd, kvd = nkv * hd;
        const float base = local ? c->rope_freq_base_swa : c->rope_freq_base;
        const float *div = local ? NULL : rdiv;

        rms(h, x, F(g, L, "attn_norm.weight"), ne, c->rms_eps);
        matvec(q, T(g, L, "attn_q.weight"), h, ne, qd);
        for (int a = 0; a < H; a++) rms(q + a * hd, q + a * hd, F(g, L, "attn_q_norm.weight"), hd, c->rms_eps);
        for (int a = 0; a < H; a++) rope(q + a * hd, hd, pos, base, div);
        int src = kv_owner(m, L);
        if (L < c->n_kv_start) {
            matvec(kb, T(g, L, "attn_k.weight"), h, ne, kvd);
            const struct gguf_tensor *wv = T(g, L, "attn_v.weight");
            if (wv) matvec(vb, wv, h, ne, kvd); else memcpy(vb, kb, sizeof(float) * kvd);
            for (int a = 0; a < nkv; a++) rms(kb + a * hd, kb + a * hd, F(g, L, "attn_k_norm.weight"), hd, c->rms_eps);
            for (int a = 0; a < nkv; a++) rms(vb + a * hd, vb + a * hd, NULL, hd, c->rms_eps);
            for (int a = 0; a < nkv; a++) rope(kb + a * hd, hd, pos, base, div);
            float *kr = o->k[L] + (size_t)(pos % o->seq[L]) * kvd, *vr = o->v[L] + (size_t)(pos % o->seq[L]) * kvd;
            for (int i = 0; i < kvd; i++) {
                kr[i] = o->round16[L] ? lg_half_to_float(half_of(kb[i])) : kb[i];
                vr[i] = o->round16[L] ? lg_half_to_float(half_of(vb[i])) : vb[i];
            }
        }
        int t0 = (local && c->sliding_window > 0 && pos - c->sliding_window + 1 > 0) ? pos - c->sliding_window + 1 : 0;
        attend(xb, q, H, hd, H / nkv, o->k[src], o->v[src], o->kvdim[src], o->seq[src], t0, pos, att);

        matvec(ob, T(g, L, "attn_output.weight"), xb, qd, ne);
        rms(ob, ob, F(g, L, "post_attention_norm.weight"), ne, c->rms_eps);
        for (int i = 0; i < ne; i++) x[i] += ob[i];

        const int nff = m->ffn_len[L];
        rms(h, x, F(g, L, "ffn_norm.weight"), ne, c->rms_eps);
        matvec(g1, T(g, L, "ffn_gate.weight"), h, ne, nff);
        matvec(g2, T(g, L, "ffn_up.weight"), h, ne, nff);
        for (int i = 0; i < nff; i++) g1[i] = gelu_tanh(g1[i]) * g2[i];
        matvec(ob, T(g, L, "ffn_down.weight"), g1, nff, ne);
        rms(ob, ob, F(g, L, "post_ffw_norm.weight"), ne, c->rms_eps);
        for (int i = 0; i < ne; i++) x[i] += ob[i];

        if (ipl) {
            matvec(pg, T(g, L, "inp_gate.weight"), x, ne, ple);
            for (int i = 0; i < ple; i++) pg[i] = gelu_tanh(pg[i]) * ipl[L * ple + i];
            matvec(ob, T(g, L, "proj.weight"), pg, ple, ne);
            rms(ob, ob, F(g, L, "post_norm.weight"), ne, c->rms_eps);
            for (int i = 0; i < ne; i++) x[i] += ob[i];
        }
        const float *os = F(g, L, "layer_output_scale.weight");
        if (os) for (int i = 0; i < ne; i++) x[i] *= os[0];
        memcpy(o->trace + (size_t)L * ne, x, sizeof(float) * ne);
    }
    if (logits) {
        rms(x, x, F(g, -1, "output_norm.weight"), ne, c->rms_eps);
        memcpy(m->last_hidden, x, sizeof(float) * ne);
        matvec(logits, T(g, -1, "token_embd.weight"), x, ne, c->n_vocab);
        if (c->logit_softcap > 0.0f)
            for (int v = 0; v < c->n_vocab; v++) logits[v] = c->logit_softcap * tanhf(logits[v] / c->logit_softcap);
    }
    free(x); free(h); free(q); free(xb); free(kb); free(vb); free(ob); free(g1); free(g2); free(att); free(pg); free(ipl);
}

static void forward(struct orc *o, int tok, int pos, float *logits) { forward_row(o, tok, NULL, pos, logits); }

static int argmax_first(const float *v, int n) {                     /* model-cpu.c:476-478 */
    int b = 0;
    for (int i = 1; i < n; i++) if (v[i] > v[b]) b = i;
    return b;
}

/* The draft head for the successor of `tok` at `pos`; attends cache positions [start, pos)
 * (reference src/mtp.c:264-356). */
static int draft(struct orc *o, int tok, int pos) {
    struct mtp *t = o->head;
    struct model *m = &o->m;
    if (!t) return -1;
    const int ni = t->n_inner, nb = t->n_bb;
    int qmax = 0;
    for (int L = 0; L < t->n_layer; L++) if (t->n_head * t->l[L].hd > qmax) qmax = t->n_head * t->l[L].hd;
    float *cat = malloc(sizeof(float) * 2 * nb), *x = malloc(sizeof(float) * ni), *h = malloc(sizeof(float) * ni);
    float *q = malloc(sizeof(float) * qmax), *xb = malloc(sizeof(float) * qmax), *ob = malloc(sizeof(float) * ni);
    float *g1 = malloc(sizeof(float) * t->n_ff), *g2 = malloc(sizeof(float) * t->n_ff);
    float *att = malloc(sizeof(float) * (pos + 1)), *lg = malloc(sizeof(float) * t->n_vocab);
    float *e = dequantize_row(T(o->g, -1, "token_embd.weight"), tok, nb);
    for (int i = 0; i < nb; i++) cat[i] = e[i] * sqrtf((float)nb);
    free(e);
    memcpy(cat + nb, m->last_hidden, sizeof(float) * nb);
    matvec(x, t->pre, cat, 2 * nb, ni);
    for (int L = 0; L < t->n_layer; L++) {
        const struct mtp_layer *b = &t->l[L];
        const int hd = b->hd, src = b->src, qd = t->n_head * hd;
        rms(h, x, b->attn_norm, ni, t->eps);
        matvec(q, b->q, h, ni, qd);
        for (int a = 0; a < t->n_head; a++) {
            rms(q + a * hd, q + a * hd, b->q_norm, hd, t->eps);
            rope(q + a * hd, hd, pos, b->local ? t->base_swa : t->base_full, NULL);
        }
        int W = m->cfg.sliding_window;
        int t0 = (b->local && W > 0 && pos - W + 1 > 0) ? pos - W + 1 : 0;
        if (pos - 1 >= t0)
            attend(xb, q, t->n_head, hd, t->n_head / m->n_head_kv[src], o->k[src], o->v[src], o->kvdim[src],
                   o->seq[src], t0, pos - 1, att);
        else memset(xb, 0, sizeof(float) * qd);
        matvec(ob, b->o, xb, qd, ni);
        rms(ob, ob, b->post_attn, ni, t->eps);
        for (int i = 0; i < ni; i++) h[i] = x[i] + ob[i];
        rms(x, h, b->ffn_norm, ni, t->eps);
        matvec(g1, b->gate, x, ni, t->n_ff);
        matvec(g2, b->up, x, ni, t->n_ff);
        for (int i = 0; i < t->n_ff; i++) g1[i] = gelu_tanh(g1[i]) * g2[i];
        matvec(ob, b->down, g1, t->n_ff, ni);
        rms(ob, ob, b->post_ffw, ni, t->eps);
        for (int i = 0; i < ni; i++) x[i] = h[i] + ob[i];
        if (b->out_scale) for (int i = 0; i < ni; i++) x[i] *= b->out_scale[0];
    }
    rms(x, x, t->out_norm, ni, t->eps);
    matvec(lg, t->head, x, ni, t->n_vocab);
    if (t->softcap > 0.0f) for (int v = 0; v < t->n_vocab; v++) lg[v] = t->softcap * tanhf(lg[v] / t->softcap);
    int best = argmax_first(lg, t->n_vocab);
    free(cat); free(x); free(h); free(q); free(xb); free(ob); free(g1); free(g2); free(att); free(lg);
    return best;
}

/* ---- flat API (same shape as oracle/ref_shim.c) ---- */

void *orc_open(const char *target, const char *head, int max_seq, int kv_f16_all) {
    struct orc *o = calloc(1, sizeof *o);
    if (!o) return NULL;
    o->g = load_gguf(target);
    if (!o->g || model_init(&o->m, o->g) != 0) { free(o); return NULL; }
    const struct config *c = &o->m.cfg;
    o->max_seq = max_seq; o->mtp_n = LG_MTP_N; o->kv_f16_all = kv_f16_all;
    o->seq = calloc(c->n_layer, sizeof(int)); o->kvdim = calloc(c->n_layer, sizeof(int));
    o->round16 = calloc(c->n_layer, sizeof(int));
    o->k = calloc(c->n_layer, sizeof(float *)); o->v = calloc(c->n_layer, sizeof(float *));
    for (int L = 0; L < c->n_layer; L++) {                           /* model-cpu.c:218-253 */
        o->kvdim[L] = o->m.n_head_kv[L] * o->m.head_dim[L];
        if (L >= c->n_kv_start) continue;
        int ring = o->m.is_local[L] && c->sliding_window > 0 && c->sliding_window < max_seq;
        o->seq[L] = ring ? c->sliding_window : max_seq;
        o->round16[L] = kv_f16_all || !o->m.is_local[L];
        o->k[L] = calloc((size_t)o->seq[L] * o->kvdim[L], sizeof(float));
        o->v[L] = calloc((size_t)o->seq[L] * o->kvdim[L], sizeof(float));
    }
    if (head && head[0]) o->head = mtp_open(head, &o->m);
    o->logits = malloc(sizeof(float) * c->n_vocab);
    o->trace = calloc((size_t)c->n_layer * c->n_embd, sizeof(float));
    return o;
}
void orc_close(void *p) {
    struct orc *o = p;
    if (!o) return;
    for (int L = 0; L < o->m.cfg.n_layer; L++) { free(o->k[L]); free(o->v[L]); }
    free(o->k); free(o->v); free(o->seq); free(o->kvdim); free(o->round16); free(o->logits); free(o->trace);
    if (o->head) mtp_free(o->head);
    model_free(&o->m);
    free_gguf(o->g);
    free(o);
}
int  orc_has_head(void *p) { return ((struct orc *)p)->head != NULL; }
int  orc_n_vocab(void *p) { return ((struct orc *)p)->m.cfg.n_vocab; }
int  orc_n_embd(void *p) { return ((struct orc *)p)->m.cfg.n_embd; }
int  orc_n_layer(void *p) { return ((struct orc *)p)->m.cfg.n_layer; }
int  orc_mtp_n(void) { return LG_MTP_N; }
/* thread count of the OpenMP runtime (set it explicitly: a launcher may have exported OMP_NUM_THREADS=1) */
int  orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n; return 1;
#endif
}
void orc_set_mtp_n(void *p, int n) { ((struct orc *)p)->mtp_n = n; }
void orc_forward(void *p, int tok, int pos, float *logits) { forward(p, tok, pos, logits); }
void orc_last_hidden(void *p, float *out) {
    struct orc *o = p; memcpy(out, o->m.last_hidden, sizeof(float) * o->m.cfg.n_embd);
}
void orc_trace(void *p, float *out) {
    struct orc *o = p; memcpy(out, o->trace, sizeof(float) * o->m.cfg.n_embd * o->m.cfg.n_layer);
}
int orc_next(void *p, int tok, int pos) {
    struct orc *o = p;
    forward(o, tok, pos, o->logits);
    return argmax_first(o->logits, o->m.cfg.n_vocab);
}
void orc_prefill(void *p, const int *toks, int n, int pos0) {
    for (int i = 0; i < n; i++) forward(p, toks[i], pos0 + i, NULL);
}
/* ids[i] >= 0: token; ids[i] < 0: row -ids[i]-1 of `rows` (model-cpu.c:489-497) */
void orc_prefill_mixed(void *p, const float *rows, const int *ids, int n, int pos0) {
    struct orc *o = p;
    for (int i = 0; i < n; i++) {
        if (ids[i] >= 0) forward(o, ids[i], pos0 + i, NULL);
        else forward_row(o, 0, rows + (size_t)(-ids[i] - 1) * o->m.cfg.n_embd, pos0 + i, NULL);
    }
}
/* verify block, sequentially: forwards stop at the first draft that fails (model-cpu.c:51-58) */
int orc_spec(void *p, const int *toks, int pos, int *out) {
    struct orc *o = p;
    int j = 0;
    do { out[j] = orc_next(o, toks[j], pos + j); j++; } while (j < o->mtp_n && out[j - 1] == toks[j]);
    return j;
}
int orc_draft(void *p, int tok, int pos) { return draft(p, tok, pos); }
int orc_kv_row(void *p, int L, int pos, float *k, float *v) {
    struct orc *o = p;
    if (L < 0 || L >= o->m.cfg.n_layer || !o->k[L]) return 0;
    size_t off = (size_t)(pos % o->seq[L]) * o->kvdim[L];
    memcpy(k, o->k[L] + off, sizeof(float) * o->kvdim[L]);
    memcpy(v, o->v[L] + off, sizeof(float) * o->kvdim[L]);
    return o->kvdim[L];
}
int orc_dequant(unsigned type, const void *src, float *out, long long n) {
    return dequantize_into(type, src, out, n) ? 0 : -1;
}
/* greedy generation; rounds follow the reference CLI (src/run.c:54-71,744-767): toks[0] is the
 * chosen token, drafts fill toks[1..]; emit the accepted drafts, continue from out[adv-1]. */
int orc_generate(void *p, const int *prompt, int n_prompt, int n_gen, int *out_toks, int mode,
                 const int *replay, int *stats) {
    struct orc *o = p;
    int g = 0, nd = 0, na = 0, N = o->mtp_n;
    if (n_prompt > 1) orc_prefill(o, prompt, n_prompt - 1, 0);
    int pos = n_prompt - 1;
    int best = orc_next(o, prompt[n_prompt - 1], pos++);
    out_toks[g++] = best;
    while (g < n_gen) {
        if (!mode) { best = orc_next(o, best, pos++); out_toks[g++] = best; continue; }
        int toks[16], out[16];
        toks[0] = best;
        for (int j = 1; j < N; j++) {
            if (mode == 2) toks[j] = replay[g + j - 1];
            else if (j == 1) { int d = draft(o, best, pos); toks[1] = d >= 0 ? d : best; }
            else toks[j] = toks[j - 1];                       /* the host draft does not chain */
        }
        int adv = orc_spec(o, toks, pos, out);
        nd += N - 1; na += adv - 1;
        for (int j = 1; j < adv && g < n_gen; j++) out_toks[g++] = toks[j];
        best = out[adv - 1];
        pos += adv;
        if (g < n_gen) out_toks[g++] = best;
    }
    if (stats) { stats[0] = nd; stats[1] = na; }
    return g;
}
