/* lg_session.c -- a flat session API over the model interface, for language bindings.
 *
 * Everything here goes through the same calls the reference CLI makes (src/run.c:54-71 one MTP
 * round; src/run.c:697-785 generate: prefill all but the last prompt token, model_forward_next
 * on the last, then rounds), so a binding that drives a session exercises the backend exactly
 * as `run -mtp` would.
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "lg_host.h"
#include "lg_b200.h"

/* The sampling hook lives in the caller (the reference defines it in its CLI, src/run.c:83).
 * A weak NULL default keeps the library loadable on its own; a caller's definition wins. */
__attribute__((weak)) int (*model_pick)(const float *logits, int n) = NULL;

struct lg_session {
    struct gguf_context *g;
    struct model m;
    struct kvcache kv;
    struct mtp *head;
    int mtp_n;
};

long long lgs_host_syncs(void *p) { return lg_host_syncs(&((struct lg_session *)p)->m); }

void *lgs_open(const char *target, const char *head, int max_seq, int kv_f16_all_ignored) {
    (void)kv_f16_all_ignored;                       /* the device cache is always f16 */
    struct lg_session *s = calloc(1, sizeof *s);
    if (!s) return NULL;
    s->g = load_gguf(target);
    if (!s->g) { free(s); return NULL; }
    if (model_init(&s->m, s->g) != 0) { free_gguf(s->g); free(s); return NULL; }
    if (kvcache_init(&s->kv, &s->m, max_seq) != 0) { model_free(&s->m); free_gguf(s->g); free(s); return NULL; }
    if (head && head[0]) s->head = mtp_open(head, &s->m);
    s->mtp_n = LG_MTP_N;
    lg_set_round_width(LG_MTP_N);
    return s;
}
void lgs_close(void *p) {
    struct lg_session *s = p;
    if (!s) return;
    if (s->head) mtp_free(s->head);
    kvcache_free(&s->kv);
    lg_engine_release();
    model_free(&s->m);
    free_gguf(s->g);
    free(s);
}
int  lgs_has_head(void *p) { return ((struct lg_session *)p)->head != NULL; }
int  lgs_n_vocab(void *p) { return ((struct lg_session *)p)->m.cfg.n_vocab; }
int  lgs_n_embd(void *p) { return ((struct lg_session *)p)->m.cfg.n_embd; }
int  lgs_n_layer(void *p) { return ((struct lg_session *)p)->m.cfg.n_layer; }
int  lgs_mtp_n(void) { return LG_MTP_N; }
/* verify width of the session's rounds, clamped to what the backend runs (1..8) */
void lgs_set_mtp_n(void *p, int n) {
    struct lg_session *s = p;
    s->mtp_n = n < 1 ? 1 : (n > 8 ? 8 : n);
    lg_set_round_width(s->mtp_n);
}
void *lgs_model(void *p) { return &((struct lg_session *)p)->m; }
void *lgs_kv(void *p) { return &((struct lg_session *)p)->kv; }
void *lgs_head(void *p) { return ((struct lg_session *)p)->head; }

void lgs_forward(void *p, int tok, int pos, float *logits) {
    struct lg_session *s = p; model_forward(&s->m, &s->kv, tok, pos, logits);
}
void lgs_last_hidden(void *p, float *out) { lg_last_hidden(&((struct lg_session *)p)->m, out); }
int  lgs_next(void *p, int tok, int pos) { struct lg_session *s = p; return model_forward_next(&s->m, &s->kv, tok, pos); }
void lgs_prefill(void *p, const int *toks, int n, int pos0) { struct lg_session *s = p; model_prefill(&s->m, &s->kv, toks, n, pos0); }
void lgs_prefill_mixed(void *p, const float *rows, const int *ids, int n, int pos0) {
    struct lg_session *s = p; model_prefill_mixed(&s->m, &s->kv, rows, ids, n, pos0);
}
void lgs_prefill_embd(void *p, const float *rows, int n, int pos0) { struct lg_session *s = p; model_prefill_embd(&s->m, &s->kv, rows, n, pos0); }
int  lgs_spec(void *p, const int *toks, int pos, int *out) {
    struct lg_session *s = p; return lg_forward_spec_n(&s->m, &s->kv, s->mtp_n, toks, pos, out);
}
int  lgs_draft(void *p, int tok, int pos) {
    struct lg_session *s = p; return s->head ? mtp_draft(s->head, &s->m, &s->kv, tok, pos) : -1;
}
int  lgs_draft_chain(void *p, int tok, int pos) {
    struct lg_session *s = p; return s->head ? mtp_draft_chain(s->head, &s->m, &s->kv, tok, pos) : -1;
}
int  lgs_kv_row(void *p, int L, int pos, float *k, float *v) { struct lg_session *s = p; return lg_kv_row(&s->m, &s->kv, L, pos, k, v); }
int  lgs_dequant(unsigned type, const void *src, float *out, long long n) {
    int blk = ggml_blck_size(type);
    if (!blk || n % blk) return -1;
    return lg_dequant_host((int)type, src, 1, (int)n, out);
}

/* Host-driven rounds through the reference-shaped calls -- one blocking call per draft and per
 * verify, exactly like src/run.c:54-71.  Starts from chosen token `best` at position `pos` with
 * g tokens already emitted; runs until n_gen tokens are out or n_rounds rounds are done.
 * mode 0 plain decode, 1 head drafts, 2 replayed drafts (replay[i] = draft for stream index i),
 * 3 head drafts computed through the API but replaced by the replayed ones (the acceptance
 * rate is then the table's while the head's cost is still paid). */
static int replay_at(const int *replay, int n_replay, int i) { return replay && i >= 0 && i < n_replay ? replay[i] : 0; }

int lgs_rounds_host(void *p, int best, int pos, int g, int n_gen, int n_rounds, int *out_toks, int mode,
                    const int *replay, int n_replay, int *stats) {
    struct lg_session *s = p;
    int nd = 0, na = 0, N = s->mtp_n, rounds = 0;
    if (N < 1 || N > 8) return -1;
    lg_set_round_width(N);
    if (mode == 3 && replay) {
        /* the device applies the same override when it runs a round ahead of the calls below: draft for stream index i
         * is replay[i], and the index of the first draft of a round is g = (its position) + (g - pos) */
        lg_set_replay(&s->m, replay, n_replay);
        lg_set_replay_origin(&s->m, g - pos, 1);
    } else {
        lg_set_replay_origin(&s->m, 0, 0);
    }
    while (g < n_gen && (n_rounds <= 0 || rounds < n_rounds)) {
        rounds++;
        if (!mode) { best = model_forward_next(&s->m, &s->kv, best, pos++); out_toks[g++] = best; continue; }
        int toks[8], out[8];
        toks[0] = best;
        if (mode == 1 || mode == 3) {
            int d = mtp_draft(s->head, &s->m, &s->kv, best, pos);
            toks[1] = d >= 0 ? d : best;
            if (mode == 3) toks[1] = replay_at(replay, n_replay, g);
            for (int j = 2; j < N; j++) {
                int dj = mtp_draft_chain(s->head, &s->m, &s->kv, toks[j - 1], pos + j - 1);
                toks[j] = dj >= 0 ? dj : toks[j - 1];
                if (mode == 3) toks[j] = replay_at(replay, n_replay, g + j - 1);
            }
        } else {
            for (int j = 1; j < N; j++) toks[j] = replay_at(replay, n_replay, g + j - 1);
        }
        int adv = lg_forward_spec_n(&s->m, &s->kv, N, toks, pos, out);
        nd += N - 1; na += adv - 1;
        for (int j = 1; j < adv && g < n_gen; j++) out_toks[g++] = toks[j];
        best = out[adv - 1];
        pos += adv;
        if (g < n_gen) out_toks[g++] = best;
    }
    if (stats) { stats[0] = nd; stats[1] = na; stats[2] = pos; stats[3] = best; }
    return g;
}

/* Prompt then host-driven rounds: the generate loop of src/run.c:697-785. */
int lgs_generate(void *p, const int *prompt, int n_prompt, int n_gen, int *out_toks, int mode,
                 const int *replay, int n_replay, int *stats) {
    struct lg_session *s = p;
    int st[4];
    if (n_prompt > 1) model_prefill(&s->m, &s->kv, prompt, n_prompt - 1, 0);
    int pos = n_prompt - 1;
    int best = model_forward_next(&s->m, &s->kv, prompt[n_prompt - 1], pos++);
    out_toks[0] = best;
    int g = lgs_rounds_host(p, best, pos, 1, n_gen, 0, out_toks, mode, replay, n_replay, st);
    if (stats) { stats[0] = st[0]; stats[1] = st[1]; }
    return g;
}

/* Device-resident generation: after the prompt, rounds run back to back on the device with one
 * synchronisation at the end.  Emits at least n_gen tokens (a round may overshoot). */
int lgs_generate_device(void *p, const int *prompt, int n_prompt, int n_gen, int *out_toks, int mode,
                        const int *replay, int n_replay, int *stats) {
    struct lg_session *s = p;
    int N = mode ? s->mtp_n : 1;
    if (n_prompt > 1) model_prefill(&s->m, &s->kv, prompt, n_prompt - 1, 0);
    int pos = n_prompt - 1;
    int best = model_forward_next(&s->m, &s->kv, prompt[n_prompt - 1], pos++);
    out_toks[0] = best;
    if (mode == 2) lg_set_replay(&s->m, replay, n_replay);
    lg_rounds_begin(&s->m, best, pos, 1);
    int st[4] = {0, 1, 0, 0};
    while (st[1] < n_gen) {
        int left = n_gen - st[1];
        int rounds = mode ? (left + N - 1) / N : left;       /* lower bound on rounds still needed */
        if (lg_rounds_enqueue(&s->m, &s->kv, mode == 1 || s->head ? s->head : NULL, N, mode, rounds) != 0) return -1;
        lg_rounds_collect(&s->m, NULL, 0, 0, st);
    }
    int n = st[1] - 1 < n_gen - 1 ? st[1] - 1 : n_gen - 1;
    lg_rounds_collect(&s->m, out_toks + 1, 1, n, st);
    if (stats) { stats[0] = st[2]; stats[1] = st[3]; }
    return n + 1;
}
