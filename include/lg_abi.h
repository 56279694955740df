/* lg_abi.h -- data layouts shared between the host C and the sm_100a backend.
 *
 * Every struct here is layout-compatible, field for field, with the struct of
 * the same name that the little-gemma host code passes across its backend
 * seam, so that objects built by either host (this repository's or the
 * reference's) can be handed to the backend unchanged:
 *
 *   gguf_header / gguf_meta / gguf_tensor / gguf_context   include/gguf.h:34-95
 *   config / model / kvcache                               include/model.h:10-77
 *   mtp_layer / mtp                                        src/mtp-internal.h:11-31
 *
 * Only layout is mirrored; the routines that fill these structs are written
 * independently (csrc/host).
 */
#ifndef LG_ABI_H
#define LG_ABI_H

#include <stdint.h>
#include <stddef.h>
#include <stdbool.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- GGUF container ------------------------------------------------------ */

enum gguf_type {
    GGUF_TYPE_UINT8 = 0, GGUF_TYPE_INT8 = 1, GGUF_TYPE_UINT16 = 2, GGUF_TYPE_INT16 = 3,
    GGUF_TYPE_UINT32 = 4, GGUF_TYPE_INT32 = 5, GGUF_TYPE_FLOAT32 = 6, GGUF_TYPE_BOOL = 7,
    GGUF_TYPE_STRING = 8, GGUF_TYPE_ARRAY = 9, GGUF_TYPE_UINT64 = 10, GGUF_TYPE_INT64 = 11,
    GGUF_TYPE_FLOAT64 = 12, GGUF_TYPE_COUNT
};

/* ggml tensor element types that can appear in gguf_tensor.type */
enum ggml_type {
    GGML_TYPE_F32 = 0, GGML_TYPE_F16 = 1, GGML_TYPE_Q4_0 = 2, GGML_TYPE_Q8_0 = 8,
    GGML_TYPE_Q2_K = 10, GGML_TYPE_Q3_K = 11, GGML_TYPE_Q4_K = 12, GGML_TYPE_Q5_K = 13,
    GGML_TYPE_Q6_K = 14, GGML_TYPE_BF16 = 30
};

struct gguf_header {
    uint32_t magic, version;
    uint64_t num_tensors, num_meta;
};

struct gguf_meta {
    char    *key;
    uint32_t type;                     /* enum gguf_type: selects the live member */
    union {
        uint8_t u8; int8_t i8; uint16_t u16; int16_t i16;
        uint32_t u32; int32_t i32; uint64_t u64; int64_t i64;
        float f32; double f64; bool bool_;
        char *str;
        struct { uint32_t type; uint64_t n; void *data; } arr;   /* data: n scalars, or char*[n] */
    } value;
};

struct gguf_tensor {
    char    *name;
    uint32_t n_dims;
    uint64_t dims[4];                  /* dims[0] = contraction length, dims[1] = rows */
    uint32_t type;                     /* enum ggml_type */
    uint64_t offset;                   /* from the start of the data section */
    void    *data;
};

struct gguf_context {
    struct gguf_header  header;
    struct gguf_meta   *meta;
    struct gguf_tensor *tensors;
    size_t  alignment, data_offset;
    void   *data;
    size_t  data_size;
    void   *map_base;
    size_t  map_len;
    int     map_fd;
};

/* ---- model --------------------------------------------------------------- */

struct config {
    char  arch[32];
    int   n_layer, n_embd, n_head, n_head_kv;
    int   head_dim_swa, head_dim_full;
    int   n_ff, n_vocab, n_ctx, sliding_window;
    int   n_embd_per_layer;            /* width of one per-layer-embedding (PLE) slice */
    int   n_kv_start;                  /* layers [0, n_kv_start) own K/V; later ones borrow */
    float rms_eps, rope_freq_base, rope_freq_base_swa, logit_softcap;
};

struct model {
    struct config              cfg;
    const struct gguf_context *ctx;    /* borrowed */
    int   *is_local, *ffn_len, *head_dim, *n_head_kv;   /* one entry per layer */
    float *last_hidden;                /* n_embd floats; host backends fill it */
};

struct kvcache {
    int    n_layer, max_seq;
    int   *kv_dim, *seq, *f16;         /* per layer; seq = ring rows, 0 when borrowing */
    void **k, **v;                     /* per layer; DEVICE pointers for this backend */
    void **px_k, **px_v;               /* saved system-prefix rows, or NULL */
};

/* ---- draft head ---------------------------------------------------------- */

struct mtp_layer {
    const float *attn_norm, *q_norm, *post_attn, *ffn_norm, *post_ffw;
    const float *out_scale;
    const struct gguf_tensor *q, *o, *gate, *up, *down;
    int hd, local, src;                /* src = target layer whose K/V this block reads */
};

struct mtp {
    struct gguf_context *ctx;
    int   n_layer, n_inner, n_bb, n_vocab, n_head, n_ff;
    float eps, base_full, base_swa, softcap;
    const struct gguf_tensor *pre, *post, *head;
    const float *out_norm;
    struct mtp_layer *l;
    float *cat, *x, *h, *q, *xb, *o, *g1, *g2, *att, *logits;   /* host-draft scratch (unused here) */
    int    att_cap;
    void  *cuda;                       /* backend slot: NULL = not built, (void*)-1 = disabled */
};

#ifdef __cplusplus
}
#endif
#endif /* LG_ABI_H */
