/* lg_host.h -- the host-side C API the sm_100a backend is written against.
 *
 * Function names, argument meaning and error behaviour are those of the little-gemma host
 * code (include/gguf.h:97-136, include/quant.h:26-51, include/model.h:31-49,139-192), so the
 * backend object links unchanged against either that host code or the independent
 * implementation in this directory (lg_gguf.c, lg_quant.c, lg_setup.c).
 */
#ifndef LG_HOST_H
#define LG_HOST_H

#include "lg_abi.h"

#ifndef LG_MTP_N
#define LG_MTP_N 4        /* verify width: chosen token + 3 drafts; must equal the caller's */
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* container */
struct gguf_context *load_gguf(const char *path);          /* NULL on any error */
void        free_gguf(struct gguf_context *ctx);
void        gguf_data_dontneed(const struct gguf_context *ctx, const void *p, size_t bytes);
const struct gguf_meta   *gguf_find_meta(const struct gguf_context *ctx, const char *key);
const struct gguf_tensor *gguf_find_tensor(const struct gguf_context *ctx, const char *name);
uint32_t    gguf_get_u32(const struct gguf_context *ctx, const char *key, uint32_t fallback);
int32_t     gguf_get_i32(const struct gguf_context *ctx, const char *key, int32_t fallback);
float       gguf_get_f32(const struct gguf_context *ctx, const char *key, float fallback);
const char *gguf_get_str(const struct gguf_context *ctx, const char *key, const char *fallback);

/* block formats */
int    ggml_blck_size(uint32_t type);                      /* 0 = unsupported */
size_t ggml_type_size(uint32_t type);
size_t ggml_nbytes(uint32_t type, int64_t n_elements);
bool   dequantize_into(uint32_t type, const void *src, float *out, int64_t n);
float *dequantize_row(const struct gguf_tensor *t, int64_t row, int64_t row_len);  /* caller frees */

/* model set-up */
int  config_load(struct config *c, const struct gguf_context *ctx);   /* 0 / -1 */
int  model_init(struct model *m, const struct gguf_context *ctx);     /* 0 / -1 */
void model_free(struct model *m);

/* draft head: open/validate on the host, forward on the device */
struct mtp *mtp_open(const char *path, const struct model *m);        /* NULL = unusable head */
void        mtp_free(struct mtp *t);
int mtp_draft(struct mtp *t, const struct model *m, const struct kvcache *kv, int token, int pos);
int mtp_draft_chain(struct mtp *t, const struct model *m, const struct kvcache *kv, int token, int pos);

/* supplied by the CLI in the reference (src/run.c:83); NULL = greedy */
extern int (*model_pick)(const float *logits, int n);

#ifdef __cplusplus
}
#endif
#endif
