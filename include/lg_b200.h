/* lg_b200.h -- C ABI of liblg_b200.so, the sm_100a backend of the little-gemma speculative-decode
 * step.  Plain C types only.  Struct layouts are in lg_abi.h.
 *
 * Part 1 is the backend seam of the reference: the very symbols its host C (run.c, mtp.c)
 * resolves at link time against model-cuda-i8.cu; each declaration cites the reference
 * interface it replaces.  Part 2 adds entry points the reference does not have.
 */
#ifndef LG_B200_H
#define LG_B200_H

#include "lg_abi.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ===== Part 1: the reference's backend seam ============================================== */

/* 0: cache rows live on the device, so the host draft in mtp.c must call the *_device hooks.
 * Replaces: include/model.h:190 (set in src/cuda/model-cuda.cuh). */
extern const int model_kv_host;

/* Allocate the f16 K/V cache on the device: global layers max_seq rows, sliding-window layers
 * a ring of window + spare rows, row(p) = p % seq; borrowing layers get NULL.  0 / -1.
 * Replaces: include/model.h:79 (src/cuda/model-cuda.cuh:999-1051). */
int  kvcache_init(struct kvcache *kv, const struct model *m, int max_seq);
/* Replaces: include/model.h:80 (src/cuda/model-cuda.cuh:1052-1060). */
void kvcache_free(struct kvcache *kv);
/* Save / restore the first min(n, seq) rows of every owning layer (system-prefix reuse).
 * Replaces: include/model.h:91-92 (src/cuda/model-cuda.cuh:1065-1088). */
void kvcache_save_prefix(struct kvcache *kv, int n);
void kvcache_restore_prefix(struct kvcache *kv, int n);

/* One token at position pos; writes n_vocab soft-capped logits to the caller's host buffer
 * (logits == NULL: cache writes only).  Replaces: include/model.h:98 (model-cuda.cuh:1318-1354). */
void model_forward(struct model *m, struct kvcache *kv, int token, int pos, float *logits);
/* Same forward, returns the greedy next token (argmax on the device, lowest index on ties);
 * with model_pick set, calls it on the logits row instead.
 * Replaces: include/model.h:103 (model-cuda.cuh:1356-1367). */
int  model_forward_next(struct model *m, struct kvcache *kv, int token, int pos);
/* Fill the cache for tokens[0..n) at pos0.., no head.
 * Replaces: include/model.h:123 (src/cuda/prefill-kernel.cuh:631-675). */
void model_prefill(struct model *m, struct kvcache *kv, const int *tokens, int n, int pos0);
/* Media-row prefill forms: rows = f32 embedding rows [.][n_embd] that enter in place of token
 * embeddings as they are (the per-layer table row of token 0 goes with them); _mixed: ids[i] >= 0
 * is a token id, ids[i] < 0 names row -ids[i]-1.  Replaces: include/model.h:133,143
 * (src/cuda/prefill-kernel.cuh:678-810; arithmetic: src/cpu/model-cpu.c:459-465,489-497). */
void model_prefill_embd(struct model *m, struct kvcache *kv, const float *rows, int n, int pos0);
void model_prefill_mixed(struct model *m, struct kvcache *kv, const float *rows, const int *ids, int n, int pos0);
/* No-op here (buffers are sized at load).  Replaces: include/model.h:149. */
void model_prefill_reserve(void);

/* Verify LG_MTP_N tokens (toks[0] chosen, toks[1..] drafts) at pos.. in ONE weight pass:
 * out[j] = greedy successor of toks[j]; returns adv = 1 + the run of out[j-1] == toks[j];
 * leaves the draft head's h_prev at row adv-1.  LG_MTP_N is compile time and must equal the
 * caller's.  Replaces: include/model.h:186 (src/cuda/mtp-kernel.cuh:82-120). */
int  model_forward_spec(struct model *m, struct kvcache *kv, const int *toks, int pos, int *out);

/* Draft the successor of `token` (the token chosen for `pos`) with the head resident on the
 * device; -1 = drafting unavailable.  Replaces: src/mtp-internal.h:33-34 (mtp-kernel.cuh:329-370). */
int  mtp_draft_device(struct mtp *t, const struct model *m, const struct kvcache *kv, int token, int pos);
/* Chained draft on the head's own hidden through the post-projection; -1 = no chaining.
 * Replaces: src/mtp-internal.h:35-36 (mtp-kernel.cuh:378-402). */
int  mtp_draft_chain_device(struct mtp *t, const struct model *m, const struct kvcache *kv, int token, int pos);
/* Replaces: src/mtp-internal.h:37 (mtp-kernel.cuh:404-421). */
void mtp_free_device(struct mtp *t);

/* ===== Part 2: additions ================================================================= */

/* model_forward_spec with a run-time width n in [1, 8] (n = 1 is plain decode). */
int  lg_forward_spec_n(struct model *m, struct kvcache *kv, int n, const int *toks, int pos, int *out);

/* Device-resident rounds: [drafts -> verify of width n -> greedy accept -> advance] repeated
 * n_rounds times with NO host synchronisation in between.  mode 0: no drafts (n must be 1),
 * 1: drafts from head t, 2: drafts from the table given to lg_set_replay (head t, if given,
 * still runs and is overridden).  begin sets the chosen token / position / emitted count,
 * enqueue only launches, collect synchronises once and returns the emitted tokens [from..)
 * and stats = {pos, n_emitted, n_draft, n_accept}. */
int  lg_set_replay(struct model *m, const int *replay, int n);
int  lg_rounds_begin(struct model *m, int first_token, int pos, int n_emitted);
int  lg_rounds_enqueue(struct model *m, struct kvcache *kv, struct mtp *t, int n, int mode, int n_rounds);
int  lg_rounds_collect(struct model *m, int *tokens, int from, int cap, int *stats);

/* One host wait per round behind the blocking calls.  mtp_draft_device runs the whole round on the stream (every draft,
 * the verify of the tokens they turned out to be, the acceptance) and waits once for its record; mtp_draft_chain_device
 * and model_forward_spec / lg_forward_spec_n answer from that record when they are asked about exactly those tokens, and
 * fall back to running synchronously otherwise (the results are the same either way).  The round is run at the width set
 * here (default LG_MTP_N).  LG_LAZY_ROUND=0 in the environment keeps every call synchronous. */
void lg_set_round_width(int n);
/* With a replay table set (lg_set_replay), that whole-round path overrides the head's drafts as the device-resident rounds
 * do: the draft offered for position p is replay[p + offset].  enable = 0 turns the override off. */
void lg_set_replay_origin(struct model *m, int offset, int enable);
long long lg_host_syncs(struct model *m);            /* blocking device-to-host waits made by the blocking calls so far */
/* Variable draft length: a draft whose best logit leads the runner-up by less than `margin` calls off the round's remaining
 * drafts (forwards skipped on the device, slots padded with the previous token as for a head that cannot chain).  0 = off.
 * The idea is the reference's own open lever (docs/upstream-llama-study.md:306-311); the output never changes. */
void lg_set_draft_margin(struct model *m, float margin);
long long lg_drafts_skipped(struct model *m);        /* drafts called off, as of the latest lg_rounds_collect */

/* Introspection for tests and the benchmark. */
long long lg_weight_bytes(struct model *m);          /* file bytes of all matrices uploaded so far */
long long lg_round_launches(struct model *m);        /* kernels in one captured round */
int   lg_last_hidden(struct model *m, float *out);   /* h_prev (n_embd floats) */
int   lg_kv_row(struct model *m, struct kvcache *kv, int layer, int pos, float *k, float *v);
void *lg_stream(struct model *m);                    /* the cudaStream_t all work is issued on */
/* Enqueue only selected kernel classes of one verify step of width n (for timing kernels in
 * isolation); classes is a mask (1 qkv, 2 o, 4 gate/up, 8 down, 16 head, 32 per-layer-embedding
 * matmuls, 64 norms, 128 q/k/v post-processing, 256 attention, 512 the rest; <= 0 = all weight
 * matmuls); returns the number of launches.  A forward must have run before. */
int   lg_bench_matmul_pass(struct model *m, int n, int classes);
/* Enqueue the kernels of one wide prompt block of n <= 256 tokens restricted to kernel classes
 * (<= 0: the four layer matmuls); returns the number of launches or -1.  Timing utility. */
int   lg_bench_prefill_pass(struct model *m, int n, int classes);
/* Long-context attention: caches of at least min_seq rows run full-attention layers through the
 * span kernel (G tiles of 64 keys per CTA, online softmax); force_g > 0 fixes G (tests), 0 derives it
 * from the cache length.  Default: min_seq 4096 (LG_ATTN_DEEP_MIN), G derived.  Set before the
 * session's first forward. */
void  lg_set_attn_deep(int min_seq, int force_g);
void  lg_engine_release(void);                       /* free all device state of the loaded model */
/* Test entry: one CTA waits on a barrier nothing completes, gives up after `polls` polls (1 .. 2^20) and raises the status
 * bit a production kernel's bounded wait would raise; returns the status word read back (1 = the wait ran out, as it must)
 * and clears it.  The device context stays usable: no trap, no fault, no endless loop. */
int   lg_debug_bounded_wait(struct model *m, int polls);
/* Profiling builds only (-DLG_STAMPS): phase time stamps of the latest launches / clear them; -1 in the product build. */
int   lg_debug_stamps(long long *out);
int   lg_debug_clear_stamps(void);

/* Kernel-level entry points (host buffers in, host buffers out) used by the parity tests.
 * Each returns 0 or a negative error. */
/* Decode n_rows rows of k elements of a ggml type (0 f32, 1 f16, 30 bf16, 2 q4_0, 8 q8_0, 11 q3_K, 12 q4_K, 13 q5_K,
 * 14 q6_K) on the device; replaces dequantize_row / dequantize_into (src/quant.c:287-343) bit for bit. */
int  lg_dequant_host(int type, const void *blocks, int n_rows, int k, float *out);
/* y[tok][row] = W x[tok] for tok < M <= 8 through the tile-major repack, the 16-bit activation
 * panel and the tensor-core kernel; W is m rows of file-format blocks (q4_0, q4_K, q8_0, q6_K, q5_K, q3_K). */
int  lg_gemv_host(int type, const void *blocks, int m, int k, const float *x, int M, int kslices, float *y);
/* The decode step's "matmul + residual update + next norm" chain on caller data: o = W act (complete rows with the partial
 * sums of the norms, k slices reduced inside a thread-block cluster where the plan has them), then
 * xres = (xres + rmsnorm(o) add_w) * out_scale and y = rmsnorm(xres) norm_w (norm_w NULL: y = xres) by the residual kernel.
 * The reference does this with separate norm kernels (src/cuda/model-cuda.cuh:119-190).  Returns 1 (cluster reduce used),
 * 0 (whole k range in one CTA), -2 (matrix shape cannot leave complete rows), -1 (bad arguments). */
int  lg_matmul_resid_host(int type, const void *blocks, int m, int k, const float *act, int M, float *xres,
                          const float *add_w, float out_scale, const float *norm_w, float eps, float *y);
/* The wide (prompt) matmul: out[tok][row] = W x[tok] for tok < n <= 256 at once, x rounded to f16,
 * weights expanded q4 -> f16 inside the kernel, tcgen05.mma with f32 accumulation.  With blocks_up
 * != NULL the two matrices are a gate/up pair and out[tok][row] = gelu_tanh(gate.x) * (up.x)
 * rounded to f16 (the fused epilogue the prompt pass uses).  Replaces the reference's wide-batch
 * matmul_q_n / matmul_q4k_mma_kernel (src/cuda/model-cuda-i8.cu:1060-1227). */
int  lg_prefill_matmul_host(int type, const void *blocks, const void *blocks_up, int m, int k, const float *x, int n,
                            float *out);
/* Split-KV flash-decode of M query rows over an f16 cache given as f32 host arrays
 * (rounded to f16 on upload): q [M][H][hd], k/v [seq][Hkv*hd], positions pos..pos+M-1. */
int  lg_flash_decode_host(const float *q, const float *k, const float *v, int M, int H, int Hkv, int hd,
                          int seq, int window, int pos, float *out);
/* The same attention through the kernel the decode step prefers when a KV head's key tiles fit one thread-block
 * cluster (at most 16 tiles of 128 keys): one CTA per tile, partials merged through distributed shared memory
 * instead of global scratch.  -3: the case does not fit a cluster. */
int  lg_flash_decode_cluster_host(const float *q, const float *k, const float *v, int M, int H, int Hkv, int hd,
                                  int seq, int window, int pos, float *out);

/* Split-KV flash-decode for callers that cannot allocate device memory (a captured stream, a
 * serving loop whose memory was fixed at start-up, a process whose allocator owns the device).
 * Same kernel as lg_flash_decode_host, but every pointer is a DEVICE pointer supplied by the
 * caller (q [M][H][hd] f32; k, v [seq][Hkv*hd] f16; out [M][H][hd] f32) and the kernel's scratch
 * lives in a 4 MiB array built into the library, which every GPU that loads the library holds
 * until exit.  No cudaMalloc / cudaFree / allocating call is made.  It has no counterpart in the
 * reference.  The first call on a device looks up the array's device address; make that call
 * before any stream capture.  All calls share the array: two calls that overlap on the GPU
 * (different streams, no ordering) race.  Work is enqueued on `stream` (a cudaStream_t, or NULL)
 * and not waited for.  Alignment: k and v must be 16-byte aligned (their rows are fetched with 16-byte
 * copies), q and out 4-byte aligned; a pointer into the middle of an element is turned away with -1, as
 * are out-of-range arguments.  Returns 0, or a negative code with a message on stderr; -4 means
 * key tiles x M x H x (hd + 2) x 4 bytes exceed the array (e.g. M=4, H=16, hd=256: up to 63 tiles
 * of 128 keys, about 8,000 cached positions). */
int  lg_flash_decode_noalloc(const float *d_q, const void *d_k_f16, const void *d_v_f16, int M, int H, int Hkv, int hd,
                             int seq, int window, int pos, float *d_out, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* LG_B200_H */
