/* ref_shim.c -- TEST INFRASTRUCTURE. A flat, ctypes-friendly face over the UNMODIFIED
 * little-gemma CPU backend (src/gguf.c, src/quant.c, src/model.c, src/mtp.c,
 * src/cpu/model-cpu.c), compiled where those sources lie by oracle/Makefile into
 * oracle/_ref/.  It is the parity oracle and the timed CPU baseline; nothing the
 * product ships may link or call it.
 *
 * Only glue lives here: the reference keeps `model_pick` in its CLI (src/run.c:83), so the
 * shim defines it; the generate loop below follows src/run.c:54-71 (one MTP round) and
 * src/run.c:744-767 (emit toks[1..adv-1], continue from out[adv-1]).
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "gguf.h"
#include "quant.h"
#include "model.h"

#ifdef _OPENMP
#include <omp.h>
#endif

int (*model_pick)(const float *logits, int n) = NULL;

/* Thread count of the OpenMP runtime this image is linked against.  A launcher may have exported
 * OMP_NUM_THREADS=1 for its workers (torchrun does) before this library was loaded; the timed CPU
 * baseline sets the count it wants here and reports what the runtime then says. */
int ref_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n; return 1;
#endif
}

struct ref_session {
    struct gguf_context *ctx;
    struct model m;
    struct kvcache kv;
    struct mtp *head;
    float *logits;
};

/* kv_f16_all != 0 stores the sliding-window rings as f16 too (the CUDA backends' layout,
 * src/cuda/model-cuda.cuh:1036-1045).  The CPU forward honours kv->f16[] on both the write
 * (src/cpu/model-cpu.c:366-373) and the reads (:377,389,398), so patching the freshly
 * initialised cache needs no source edit. */
void *ref_open(const char *target, const char *head, int max_seq, int kv_f16_all) {
    struct ref_session *s = calloc(1, sizeof *s);
    if (!s) return NULL;
    s->ctx = load_gguf(target);
    if (!s->ctx || model_init(&s->m, s->ctx) != 0 || kvcache_init(&s->kv, &s->m, max_seq) != 0) {
        fprintf(stderr, "ref_open: cannot load %s\n", target);
        free(s);
        return NULL;
    }
    if (kv_f16_all)
        for (int L = 0; L < s->kv.n_layer; L++)
            if (s->kv.k[L] && !s->kv.f16[L]) {
                size_t n = (size_t)s->kv.seq[L] * s->kv.kv_dim[L];
                free(s->kv.k[L]); free(s->kv.v[L]);
                s->kv.k[L] = calloc(n, 2); s->kv.v[L] = calloc(n, 2);
                s->kv.f16[L] = 1;
            }
    if (head && head[0]) s->head = mtp_open(head, &s->m);
    s->logits = malloc((size_t)s->m.cfg.n_vocab * sizeof(float));
    return s;
}

void ref_close(void *h) {
    struct ref_session *s = h;
    if (!s) return;
    if (s->head) mtp_free(s->head);
    kvcache_free(&s->kv);
    model_free(&s->m);
    free_gguf(s->ctx);
    free(s->logits);
    free(s);
}

int ref_has_head(void *h) { return ((struct ref_session *)h)->head != NULL; }
int ref_n_vocab(void *h) { return ((struct ref_session *)h)->m.cfg.n_vocab; }
int ref_n_embd(void *h) { return ((struct ref_session *)h)->m.cfg.n_embd; }
int ref_mtp_n(void) { return LG_MTP_N; }

void ref_forward(void *h, int tok, int pos, float *logits) {
    struct ref_session *s = h;
    model_forward(&s->m, &s->kv, tok, pos, logits);
}
void ref_last_hidden(void *h, float *out) {
    struct ref_session *s = h;
    memcpy(out, s->m.last_hidden, (size_t)s->m.cfg.n_embd * sizeof(float));
}
int ref_next(void *h, int tok, int pos) {
    struct ref_session *s = h;
    return model_forward_next(&s->m, &s->kv, tok, pos);
}
void ref_prefill_mixed(void *h, const float *rows, const int *ids, int n, int pos0) {
    struct ref_session *s = h;
    model_prefill_mixed(&s->m, &s->kv, rows, ids, n, pos0);
}
void ref_prefill(void *h, const int *toks, int n, int pos0) {
    struct ref_session *s = h;
    model_prefill(&s->m, &s->kv, toks, n, pos0);
}
int ref_spec(void *h, const int *toks, int pos, int *out) {
    struct ref_session *s = h;
    return model_forward_spec(&s->m, &s->kv, toks, pos, out);
}
int ref_draft(void *h, int tok, int pos) {
    struct ref_session *s = h;
    return s->head ? mtp_draft(s->head, &s->m, &s->kv, tok, pos) : -1;
}

/* One cache row of owning layer L at position pos, widened to f32. Returns kv_dim, 0 if the
 * layer borrows its cache. */
int ref_kv_row(void *h, int L, int pos, float *k, float *v) {
    struct ref_session *s = h;
    if (L < 0 || L >= s->kv.n_layer || !s->kv.k[L]) return 0;
    int d = s->kv.kv_dim[L];
    size_t row = (size_t)(pos % s->kv.seq[L]) * d;
    if (s->kv.f16[L]) {
        dequantize_into(GGML_TYPE_F16, (const uint16_t *)s->kv.k[L] + row, k, d);
        dequantize_into(GGML_TYPE_F16, (const uint16_t *)s->kv.v[L] + row, v, d);
    } else {
        memcpy(k, (const float *)s->kv.k[L] + row, (size_t)d * 4);
        memcpy(v, (const float *)s->kv.v[L] + row, (size_t)d * 4);
    }
    return d;
}

int ref_dequant(unsigned type, const void *src, float *out, long long n) {
    return dequantize_into(type, src, out, n) ? 0 : -1;
}

/* Greedy generation fed token ids directly (the reference CLI only takes text).
 * use_mtp: 0 = plain decode, 1 = MTP rounds with the loaded head, 2 = MTP rounds with drafts
 * taken from `replay` (replay[i] is the draft offered for stream index i, i.e. position
 * n_prompt + i).  Returns tokens written to out (n_gen); stats[0]=drafts, stats[1]=accepted. */
int ref_generate(void *h, const int *prompt, int n_prompt, int n_gen, int *out_toks,
                 int use_mtp, const int *replay, int *stats) {
    struct ref_session *s = h;
    int pos = 0, g = 0, n_draft = 0, n_accept = 0;
    if (n_prompt > 1) model_prefill(&s->m, &s->kv, prompt, n_prompt - 1, 0);
    pos = n_prompt - 1;
    int best = model_forward_next(&s->m, &s->kv, prompt[n_prompt - 1], pos);
    pos++;
    out_toks[g++] = best;
    while (g < n_gen) {
        if (!use_mtp) {
            best = model_forward_next(&s->m, &s->kv, best, pos);
            pos++;
            out_toks[g++] = best;
            continue;
        }
        int toks[LG_MTP_N], out[LG_MTP_N];
        toks[0] = best;
        if (use_mtp == 2) {
            for (int j = 1; j < LG_MTP_N; j++) toks[j] = replay[g + j - 1];
        } else {
            int d = mtp_draft(s->head, &s->m, &s->kv, best, pos);
            toks[1] = d >= 0 ? d : best;
            for (int j = 2; j < LG_MTP_N; j++) {
                int dj = mtp_draft_chain(s->head, &s->m, &s->kv, toks[j - 1], pos + j - 1);
                toks[j] = dj >= 0 ? dj : toks[j - 1];
            }
        }
        int adv = model_forward_spec(&s->m, &s->kv, toks, pos, out);
        n_draft += LG_MTP_N - 1;
        n_accept += adv - 1;
        for (int j = 1; j < adv && g < n_gen; j++) out_toks[g++] = toks[j];
        best = out[adv - 1];
        pos += adv;
        if (g < n_gen) out_toks[g++] = best;
    }
    if (stats) { stats[0] = n_draft; stats[1] = n_accept; }
    return g;
}
