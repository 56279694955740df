/* lg_setup.c -- host-side set-up: hyper-parameters and per-layer geometry of the target model,
 * and opening / validating a draft head.  Independent implementation of the behaviour of the
 * little-gemma host (src/model.c:67-189 target; src/mtp.c:124-262 head):
 *   - metadata keys are prefixed with general.architecture;
 *   - head_count, head_count_kv, feed_forward_length may be scalars or per-layer i32 arrays;
 *   - n_vocab is the length of tokenizer.ggml.tokens;
 *   - head_dim[L] and n_head_kv[L] come from the attn_q / attn_k tensor shapes; a KV-borrowing
 *     layer without attn_k inherits n_head_kv from the layer it borrows from;
 *   - a draft-head block reads the target's last sliding-window owner (n_kv_start-2) when its
 *     head size equals that layer's, else the last global owner (n_kv_start-1).
 * The draft forward itself runs on the device; mtp_draft / mtp_draft_chain only dispatch.
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "lg_host.h"

extern const int model_kv_host;
int  mtp_draft_device(struct mtp *, const struct model *, const struct kvcache *, int, int);
int  mtp_draft_chain_device(struct mtp *, const struct model *, const struct kvcache *, int, int);
void mtp_free_device(struct mtp *);

static const struct gguf_meta *arch_meta(const struct gguf_context *g, const char *arch, const char *leaf) {
    char key[160];
    snprintf(key, sizeof key, "%s.%s", arch, leaf);
    return gguf_find_meta(g, key);
}
static int is_i32_array(const struct gguf_meta *kv) {
    return kv && kv->type == GGUF_TYPE_ARRAY && kv->value.arr.type == GGUF_TYPE_INT32 && kv->value.arr.n > 0;
}
/* scalar u32/i32, or element `idx` (clamped) / the maximum (idx < 0) of an i32 array */
static int arch_int(const struct gguf_context *g, const char *arch, const char *leaf, int idx, int fb) {
    const struct gguf_meta *kv = arch_meta(g, arch, leaf);
    if (!kv) return fb;
    if (is_i32_array(kv)) {
        const int32_t *a = kv->value.arr.data;
        if (idx >= 0) return a[(uint64_t)idx < kv->value.arr.n ? (uint64_t)idx : kv->value.arr.n - 1];
        int best = a[0];
        for (uint64_t i = 1; i < kv->value.arr.n; i++) if (a[i] > best) best = a[i];
        return best;
    }
    if (kv->type == GGUF_TYPE_UINT32) return (int)kv->value.u32;
    if (kv->type == GGUF_TYPE_INT32) return kv->value.i32;
    return fb;
}
static float arch_float(const struct gguf_context *g, const char *arch, const char *leaf, float fb) {
    const struct gguf_meta *kv = arch_meta(g, arch, leaf);
    return kv && kv->type == GGUF_TYPE_FLOAT32 ? kv->value.f32 : fb;
}

int config_load(struct config *c, const struct gguf_context *g) {
    memset(c, 0, sizeof *c);
    const char *arch = gguf_get_str(g, "general.architecture", "");
    if (!arch[0]) { fprintf(stderr, "config: general.architecture is missing\n"); return -1; }
    snprintf(c->arch, sizeof c->arch, "%s", arch);
    c->n_layer   = arch_int(g, arch, "block_count", 0, 0);
    c->n_embd    = arch_int(g, arch, "embedding_length", 0, 0);
    c->n_head    = arch_int(g, arch, "attention.head_count", 0, 0);
    c->n_head_kv = arch_int(g, arch, "attention.head_count_kv", 0, c->n_head);
    c->n_ff      = arch_int(g, arch, "feed_forward_length", -1, 0);
    c->n_ctx     = arch_int(g, arch, "context_length", 0, 0);
    c->sliding_window   = arch_int(g, arch, "attention.sliding_window", 0, 0);
    c->n_embd_per_layer = arch_int(g, arch, "embedding_length_per_layer_input", 0, 0);
    c->rms_eps            = arch_float(g, arch, "attention.layer_norm_rms_epsilon", 1e-5f);
    c->rope_freq_base     = arch_float(g, arch, "rope.freq_base", 10000.0f);
    c->rope_freq_base_swa = arch_float(g, arch, "rope.freq_base_swa", c->rope_freq_base);
    c->logit_softcap      = arch_float(g, arch, "final_logit_softcapping", 0.0f);
    c->head_dim_full = arch_int(g, arch, "attention.key_length", 0, 0);
    c->head_dim_swa  = arch_int(g, arch, "attention.key_length_swa", 0, c->head_dim_full);
    int shared = arch_int(g, arch, "attention.shared_kv_layers", 0, 0);
    c->n_kv_start = shared > 0 ? c->n_layer - shared : c->n_layer;
    const struct gguf_meta *vocab = gguf_find_meta(g, "tokenizer.ggml.tokens");
    if (vocab && vocab->type == GGUF_TYPE_ARRAY) c->n_vocab = (int)vocab->value.arr.n;
    if (c->n_layer <= 0 || c->n_layer > 4096) {
        fprintf(stderr, "config: %s.block_count = %d is not a usable layer count\n", arch, c->n_layer);
        return -1;
    }
    return 0;
}

static const struct gguf_tensor *layer_tensor(const struct gguf_context *g, int L, const char *leaf) {
    char name[96];
    snprintf(name, sizeof name, "blk.%d.%s", L, leaf);
    return gguf_find_tensor(g, name);
}

int model_init(struct model *m, const struct gguf_context *g) {
    memset(m, 0, sizeof *m);
    if (config_load(&m->cfg, g) != 0) return -1;
    m->ctx = g;
    const struct config *c = &m->cfg;
    size_t nl = (size_t)c->n_layer;
    m->is_local  = calloc(nl, sizeof(int));
    m->ffn_len   = calloc(nl, sizeof(int));
    m->head_dim  = calloc(nl, sizeof(int));
    m->n_head_kv = calloc(nl, sizeof(int));
    m->last_hidden = calloc((size_t)(c->n_embd > 0 ? c->n_embd : 1), sizeof(float));
    if (!m->is_local || !m->ffn_len || !m->head_dim || !m->n_head_kv || !m->last_hidden) return -1;

    const struct gguf_meta *pat = arch_meta(g, c->arch, "attention.sliding_window_pattern");
    int have_pat = pat && pat->type == GGUF_TYPE_ARRAY && pat->value.arr.type == GGUF_TYPE_BOOL;
    for (int L = 0; L < c->n_layer; L++) {
        m->ffn_len[L] = arch_int(g, c->arch, "feed_forward_length", L, c->n_ff);
        if (is_i32_array(arch_meta(g, c->arch, "feed_forward_length")) &&
            (uint64_t)L >= arch_meta(g, c->arch, "feed_forward_length")->value.arr.n)
            m->ffn_len[L] = c->n_ff;
        if (have_pat && (uint64_t)L < pat->value.arr.n)
            m->is_local[L] = ((const int8_t *)pat->value.arr.data)[L] != 0;
    }
    for (int L = 0; L < c->n_layer; L++) {
        const struct gguf_tensor *q = layer_tensor(g, L, "attn_q.weight");
        const struct gguf_tensor *k = layer_tensor(g, L, "attn_k.weight");
        if (!q || c->n_head <= 0 || (!k && L < c->n_kv_start)) {
            fprintf(stderr, "model: layer %d has no attn_q/attn_k projection\n", L);
            return -1;
        }
        m->head_dim[L] = (int)(q->dims[1] / (uint64_t)c->n_head);
        if (k) m->n_head_kv[L] = (int)(k->dims[1] / (uint64_t)m->head_dim[L]);
        else   m->n_head_kv[L] = m->n_head_kv[c->n_kv_start - (m->is_local[L] ? 2 : 1)];
    }
    return 0;
}

void model_free(struct model *m) {
    if (!m) return;
    free(m->is_local); free(m->ffn_len); free(m->head_dim); free(m->n_head_kv); free(m->last_hidden);
    m->is_local = m->ffn_len = m->head_dim = m->n_head_kv = NULL;
    m->last_hidden = NULL;
}

/* ---- draft head ---------------------------------------------------------------------- */

static const float *f32_data(const struct gguf_tensor *t) { return t ? (const float *)t->data : NULL; }

static const struct gguf_tensor *first_of(const struct gguf_context *g, const char *leaf) {
    static const char *const prefixes[] = { "next_token.", "nextn.", "mtp." };
    char name[96];
    for (size_t i = 0; i < sizeof prefixes / sizeof *prefixes; i++) {
        snprintf(name, sizeof name, "%s%s", prefixes[i], leaf);
        const struct gguf_tensor *t = gguf_find_tensor(g, name);
        if (t) return t;
    }
    return NULL;
}

void mtp_free(struct mtp *t) {
    if (!t) return;
    mtp_free_device(t);
    free_gguf(t->ctx);
    free(t->l);
    free(t);
}

struct mtp *mtp_open(const char *path, const struct model *m) {
    struct gguf_context *g = load_gguf(path);
    if (!g) return NULL;
    const char *arch = gguf_get_str(g, "general.architecture", "");
    if (strcmp(arch, "gemma4-assistant") && strcmp(arch, "gemma4_assistant")) {
        fprintf(stderr, "mtp: %s has architecture '%s', expected gemma4-assistant\n", path, arch);
        free_gguf(g);
        return NULL;
    }
    struct mtp *t = calloc(1, sizeof *t);
    if (!t) { free_gguf(g); return NULL; }
    t->ctx = g;
    t->n_layer = arch_int(g, arch, "block_count", 0, 0);
    t->n_inner = arch_int(g, arch, "embedding_length", 0, 0);
    t->n_bb    = arch_int(g, arch, "embedding_length_out", 0, 0);
    if (!t->n_bb) t->n_bb = arch_int(g, arch, "n_embd_backbone", 0, 0);
    t->n_head  = arch_int(g, arch, "attention.head_count", 0, 0);
    t->n_ff    = arch_int(g, arch, "feed_forward_length", 0, 0);
    t->eps       = arch_float(g, arch, "attention.layer_norm_rms_epsilon", 1e-6f);
    t->base_full = arch_float(g, arch, "rope.freq_base", 1e6f);
    t->base_swa  = arch_float(g, arch, "rope.freq_base_swa", 1e4f);
    t->softcap   = arch_float(g, arch, "final_logit_softcapping", 0.0f);
    t->pre  = first_of(g, "pre_projection.weight");
    t->post = first_of(g, "post_projection.weight");
    t->head = gguf_find_tensor(g, "token_embd.weight");
    t->out_norm = f32_data(gguf_find_tensor(g, "output_norm.weight"));
    if (t->n_layer <= 0 || t->n_inner <= 0 || t->n_head <= 0 || !t->pre || !t->post || !t->head ||
        !t->out_norm || t->n_bb != m->cfg.n_embd || (int)t->pre->dims[0] != 2 * t->n_bb) {
        fprintf(stderr, "mtp: %s does not fit this target (backbone %d, target n_embd %d)\n",
                path, t->n_bb, m->cfg.n_embd);
        mtp_free(t);
        return NULL;
    }
    t->n_vocab = (int)t->head->dims[1];
    const int src_global = m->cfg.n_kv_start - 1, src_local = m->cfg.n_kv_start - 2;
    t->l = calloc((size_t)t->n_layer, sizeof *t->l);
    if (!t->l || src_local < 0) { mtp_free(t); return NULL; }
    for (int L = 0; L < t->n_layer; L++) {
        struct mtp_layer *b = &t->l[L];
        b->attn_norm = f32_data(layer_tensor(g, L, "attn_norm.weight"));
        b->q_norm    = f32_data(layer_tensor(g, L, "attn_q_norm.weight"));
        b->post_attn = f32_data(layer_tensor(g, L, "post_attention_norm.weight"));
        b->ffn_norm  = f32_data(layer_tensor(g, L, "ffn_norm.weight"));
        b->post_ffw  = f32_data(layer_tensor(g, L, "post_ffw_norm.weight"));
        b->out_scale = f32_data(layer_tensor(g, L, "layer_output_scale.weight"));
        b->q    = layer_tensor(g, L, "attn_q.weight");
        b->o    = layer_tensor(g, L, "attn_output.weight");
        b->gate = layer_tensor(g, L, "ffn_gate.weight");
        b->up   = layer_tensor(g, L, "ffn_up.weight");
        b->down = layer_tensor(g, L, "ffn_down.weight");
        if (!b->attn_norm || !b->q_norm || !b->post_attn || !b->ffn_norm || !b->post_ffw ||
            !b->q || !b->o || !b->gate || !b->up || !b->down) {
            fprintf(stderr, "mtp: block %d is missing tensors\n", L);
            mtp_free(t);
            return NULL;
        }
        b->hd = (int)b->q->dims[1] / t->n_head;
        b->local = b->hd == m->head_dim[src_local];
        b->src = b->local ? src_local : src_global;
        if (b->hd != m->head_dim[b->src]) {
            fprintf(stderr, "mtp: block %d head size %d matches no target KV layer\n", L, b->hd);
            mtp_free(t);
            return NULL;
        }
    }
    return t;
}

int mtp_draft(struct mtp *t, const struct model *m, const struct kvcache *kv, int token, int pos) {
    if (model_kv_host) return -1;          /* no host draft in this library: device only */
    return mtp_draft_device(t, m, kv, token, pos);
}
int mtp_draft_chain(struct mtp *t, const struct model *m, const struct kvcache *kv, int token, int pos) {
    if (model_kv_host) return -1;
    return mtp_draft_chain_device(t, m, kv, token, pos);
}
