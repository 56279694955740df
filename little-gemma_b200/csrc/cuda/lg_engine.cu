// lg_engine.cu -- the sm_100a backend behind the little-gemma model API.
//
// Exports the backend symbol set the host C links against (kvcache_*, model_forward*,
// model_prefill*, model_forward_spec, mtp_*_device, model_kv_host; see include/lg_b200.h for
// the reference line each one replaces) plus the device-resident round API and a few
// kernel-level entry points used by the parity tests.
//
// One engine per process (the reference keeps its device state in file-scope statics too):
// weights are uploaded and repacked on first use, every forward is a CUDA graph of fused
// kernels whose parameters never change -- position and token ids live in device memory.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cmath>
#include <vector>
#include <map>
#include <string>
#include "lg_kernels.cuh"
#include "lg_prefill.cuh"
#include "lg_attn_deep.cuh"
#include "lg_attn_cluster.cuh"
#include "lg_host.h"
#include "lg_b200.h"

#define LG_CHECK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { \
    fprintf(stderr, "lg_b200: CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); exit(1); } } while (0)

extern "C" const int model_kv_host = 0;      // cache rows live on the device: mtp.c must call the device hooks
extern "C" int lg_set_replay(struct model *m, const int *replay, int n);

namespace {

constexpr int RING_SPARE = 1024;             // ring rows beyond the window (covers the widest block written before its queries run)

constexpr int LOG_CAP = 1 << 20;

struct WMat {
    uint4 *wq = nullptr; uint2 *ws = nullptr; uint2 *wd = nullptr; uint4 *wm = nullptr;      // tiles, scales (see lg_kernels.cuh)
    int fmt = 0, m = 0, k = 0, nkp = 0, n_row_tiles = 0, ldo = 0;
    size_t file_bytes = 0;
};

struct Panel { LgPanel p{}; };

struct LayerW {
    WMat qkv, o, gateup, down, inp_gate, proj;
    // q / k / v tensors of different formats cannot share one stacked matrix: they are kept apart, each multiplied on its
    // own into its rows of the projection buffer (qkv then only carries the row stride)
    std::vector<WMat> qkv_parts; std::vector<int> qkv_row0;
    float *attn_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr, *post_attn = nullptr, *ffn_norm = nullptr,
          *post_ffw = nullptr, *post_norm = nullptr;
    float out_scale = 1.0f;
    int has_v = 1, owns_kv = 1, src = 0, local = 0, hd = 0, nkv = 0, nff = 0;
};

struct DraftBlockW {
    WMat q, o, gateup, down;
    float *attn_norm, *q_norm, *post_attn, *ffn_norm, *post_ffw;
    float out_scale; int hd, local, src;
};
struct DraftW {
    WMat pre, post, head;
    float *out_norm = nullptr;
    std::vector<DraftBlockW> blk;
    int ni = 0, nb = 0, nff = 0, n_head = 0, n_vocab = 0, has_post = 0;
    float eps = 0, base_full = 0, base_swa = 0, softcap = 0;
    // activations (one token)
    float *cat = nullptr, *x = nullptr, *hbuf = nullptr, *qbuf = nullptr, *qrot = nullptr, *obuf = nullptr, *gu = nullptr, *part = nullptr;
    float *amax_val = nullptr; int *amax_idx = nullptr, *best = nullptr;
    float *amax_val2 = nullptr, *margin = nullptr;      // runner-up logits per CTA; best - second best of the latest draft
    float2 *part_ml = nullptr;
    LgPanel p_cat{}, p_ni{}, p_attn{}, p_ff{};
    float2 *rope_local = nullptr, *rope_global = nullptr; int hd_local = 0, hd_global = 0;
    int n_slots_local = 0, n_slots_global = 0;
    std::map<std::string, cudaGraphExec_t> graphs;
};

// Buffers of the wide prompt pass (blocks of up to LG_PF_MAXN tokens), allocated at its first use.
struct PrefillBuf {
    bool ready = false;
    __half *a_ne = nullptr, *a_attn = nullptr, *a_ff = nullptr;     // f16 matmul inputs [LG_PF_MAXN][k]
    float *x = nullptr, *qkv = nullptr, *o = nullptr;               // residual rows, projection rows, o/down rows
    int *toks = nullptr, *pos = nullptr;                            // token ids; pos[g] = position of the g-th group of 8
    float2 *rope_local = nullptr, *rope_global = nullptr;
    __half *q_hi = nullptr, *q_lo = nullptr;                        // normed + rotated queries [LG_PF_MAXN][H][hd], f16 hi + lo
    float *tokrow = nullptr, *pproj = nullptr, *ipl = nullptr, *pg = nullptr;   // per-layer-embedding rows [LG_PF_MAXN][ple * n_layer], gate rows
    __half *a_ple = nullptr;
    float *rows = nullptr; int *ridx = nullptr;                     // media rows of the block and, per token, its row or -1
    int ld_attn = 0, ld_ff = 0;
};

struct Engine {
    const struct model *m = nullptr;
    const struct gguf_context *ctx = nullptr;
    cudaStream_t stream = nullptr;
    int sm_count = 148;
    // weights
    std::vector<LayerW> L;
    WMat head, pmp;                           // token_embd (tied head), per_layer_model_proj
    uint8_t *ple_table = nullptr; int ple_table_type = 0;   // per_layer_token_embd, file layout
    float *out_norm = nullptr, *ple_proj_norm = nullptr, *rope_div = nullptr;
    float2 *rope_local = nullptr, *rope_global = nullptr; int hd_local = 0, hd_global = 0;
    int has_ple = 0;
    size_t weight_bytes = 0;
    // activations
    float *x = nullptr, *qkv = nullptr, *qrot = nullptr, *oout = nullptr, *gu = nullptr, *dout = nullptr, *hidden = nullptr,
          *h_prev = nullptr, *part = nullptr, *tokrow = nullptr, *pproj = nullptr, *ipl = nullptr, *pg = nullptr, *logits = nullptr;
    float *amax_val = nullptr; int *amax_idx = nullptr;
    float2 *part_ml = nullptr;
    LgPanel p_ne{}, p_attn{}, p_ff{}, p_ple{};
    int max_ks = 4, head_ctas = 0;
    int part_slots = 0;
    // session
    LgRoundState *st = nullptr;               // device
    LgRoundState *st_host = nullptr;          // pinned mirror for uploads / downloads
    int *log = nullptr, *replay = nullptr, *d_n_replay = nullptr; int n_replay = 0, replay_cap = 0;   // replay table (capacity grows; its length lives on the device)
    int *err = nullptr, *tickets = nullptr;
    std::map<std::string, cudaGraphExec_t> graphs;
    const struct kvcache *kv_bound = nullptr;
    DraftW *draft = nullptr; const struct mtp *draft_owner = nullptr;
    float *pick_rows = nullptr;               // host logits rows for model_pick
    long long launches = 0;                   // kernels enqueued by the most recent graph build
    int pdl = 1;                              // programmatic dependent launch (LG_PDL=0 turns it off)
    long long round_launches = 0;
    PrefillBuf pf;
    float4 *sums = nullptr;                   // SUMS epilogue: per work item and token the partial sums the next kernel builds the norms from
    int pos_hi = 0;                           // host-side upper bound of the device position (device-resident rounds)
    // One host synchronisation per round behind the blocking calls: mtp_draft_device runs the WHOLE round and keeps its
    // outcome here; the chained-draft and verify calls that follow are answered from it when they ask what was computed.
    struct { bool valid = false; int n = 0, pos = 0, adv = 0, toks[LG_MAXM] = {0}, out[LG_MAXM] = {0}; bool chained = false; } lazy;
    int replay_off = 0; bool lazy_replay = false;   // replay table index of a draft = its position + replay_off (lg_set_replay_origin)
    long long host_syncs = 0;                 // blocking device-to-host waits made by the reference-shaped calls
    float *d_margin_thr = nullptr;            // confidence margin below which a draft calls off the drafts after it (0: never)
    cudaEvent_t mid_event = nullptr;          // LG_MTP_PROFILE: recorded between the layers and the head of a forward
    int mm_launches = 0;                      // kernels in the captured matmul-only pass             // kernels in one captured round (lg_rounds_enqueue)
};

Engine *g_eng = nullptr;

// Kernel launch on the engine's stream, marked for programmatic dependent launch so the kernel may
// start while its predecessor drains (every forward kernel begins with pdl_wait()).
template <typename... KArgs, typename... Args>
void launch_k(Engine *e, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = e->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = e->pdl ? 1 : 0;
    LG_CHECK(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
    e->launches++;
}
// The same with the CTAs of one blockIdx.x forming a thread-block cluster (1, grid.y, 1).
template <typename... KArgs, typename... Args>
void launch_k_cluster_y(Engine *e, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = e->stream;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 1; at[0].val.clusterDim.y = grid.y; at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = e->pdl ? 2 : 1;
    LG_CHECK(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
    e->launches++;
}


// Zero-filled device allocation.  The fill runs on the legacy stream, which does not order against the
// engine's non-blocking stream, so wait for it before anyone can use the buffer.
template <typename T> T *dalloc(size_t n) {
    T *p = nullptr;
    LG_CHECK(cudaMalloc(&p, n * sizeof(T) > 0 ? n * sizeof(T) : 16));
    LG_CHECK(cudaMemset(p, 0, n * sizeof(T)));
    LG_CHECK(cudaDeviceSynchronize());
    return p;
}

LgPanel panel_alloc(int k) {
    LgPanel P;
    P.nsb = k / 32;
    P.q = dalloc<int8_t>((size_t)2 * P.nsb * 256);
    P.s = dalloc<float2>((size_t)2 * P.nsb * 4);
    return P;
}
void panel_free(LgPanel &P) { cudaFree(P.q); cudaFree(P.s); P.q = nullptr; P.s = nullptr; }

// Host -> device copy that is complete on return.  A pageable-source cudaMemcpy may return while
// its last DMA is still in flight on the legacy stream, which the engine's non-blocking stream does
// not order against, so wait for the device.
void h2d_sync(void *dst, const void *src, size_t bytes) {
    LG_CHECK(cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice));
    LG_CHECK(cudaDeviceSynchronize());
}

float *upload_f32(const float *src, size_t n) {
    float *d = dalloc<float>(n);
    h2d_sync(d, src, n * 4);
    return d;
}

const struct gguf_tensor *find_t(const struct gguf_context *g, int L, const char *leaf) {
    char name[96];
    if (L >= 0) snprintf(name, sizeof name, "blk.%d.%s", L, leaf); else snprintf(name, sizeof name, "%s", leaf);
    return gguf_find_tensor(g, name);
}
float *upload_norm(const struct gguf_context *g, int L, const char *leaf) {
    const struct gguf_tensor *t = find_t(g, L, leaf);
    if (!t) return nullptr;
    if (t->type != GGML_TYPE_F32) { fprintf(stderr, "lg_b200: %s must be f32\n", t->name); exit(1); }
    return upload_f32((const float *)t->data, (size_t)t->dims[0]);
}

// Upload file-format tensors and repack them into one tile-major matrix: stacked row-wise, or
// (interleave) two equally shaped tensors woven 8 rows at a time -- gate rows then the matching
// up rows in every 16-row tile.
// While a draft head is being uploaded a tensor this backend cannot run must not end the process: the contract of the
// reference is "drafting off, decoding goes on" (src/cuda/mtp-kernel.cuh:263-267,331-337).  With g_soft_build set,
// build_wmat reports the problem, raises g_soft_failed and returns an empty matrix instead of exiting.
bool g_soft_build = false, g_soft_failed = false;
#define LG_BUILD_FAIL(...) do { fprintf(stderr, __VA_ARGS__); if (g_soft_build) { g_soft_failed = true; return WMat(); } exit(1); } while (0)

WMat build_wmat(Engine *e, std::vector<const struct gguf_tensor *> parts, bool interleave = false) {
    WMat W;
    if (g_soft_build && g_soft_failed) return W;
    for (auto t : parts) if (!t) LG_BUILD_FAIL("lg_b200: a weight tensor is missing from the file\n");
    const struct gguf_tensor *t0 = parts[0];
    // q4_0 / q4_K keep their 4 bits; q8_0, q6_K, q5_K, q3_K become i8 tiles.  Dense f32 / f16 / bf16 matrices are
    // accepted for a DRAFT HEAD only (g_soft_build): there they are re-encoded as q8_0 blocks on the host -- a draft never
    // changes the output, only how often it is accepted -- while a dense matrix in the target model is refused, because a
    // lossy re-encoding there would move the logits.
    uint32_t type = t0->type;
    const bool dense = type == GGML_TYPE_F32 || type == GGML_TYPE_F16 || type == GGML_TYPE_BF16;
    if (dense && !g_soft_build)
        LG_BUILD_FAIL("lg_b200: weight %s is a dense %s matrix; this backend multiplies block-quantised matrices only\n", t0->name,
                      type == GGML_TYPE_F32 ? "f32" : type == GGML_TYPE_F16 ? "f16" : "bf16");
    if (!dense && type != GGML_TYPE_Q4_0 && type != GGML_TYPE_Q4_K && !lg_fmt_is_i8((int)type))
        LG_BUILD_FAIL("lg_b200: weight %s has ggml type %u, which this backend has no kernel for\n", t0->name, type);
    if (dense) type = GGML_TYPE_Q8_0;
    W.fmt = type == GGML_TYPE_Q4_0 ? LG_FMT_Q4_0 : type == GGML_TYPE_Q4_K ? LG_FMT_Q4_K : type == GGML_TYPE_Q5_K ? LG_FMT_I8M : LG_FMT_I8;
    W.k = (int)t0->dims[0];
    if (W.k % 64) LG_BUILD_FAIL("lg_b200: %s: contraction length %d is not a multiple of 64\n", t0->name, W.k);
    if (ggml_blck_size(type) == 256 && W.k % 256) LG_BUILD_FAIL("lg_b200: %s: contraction length %d is not a multiple of 256\n", t0->name, W.k);
    for (auto t : parts) {
        if (t->type != t0->type || (int)t->dims[0] != W.k) LG_BUILD_FAIL("lg_b200: cannot stack %s onto %s\n", t->name, t0->name);
        if (t != parts.back() && t->dims[1] % 16) LG_BUILD_FAIL("lg_b200: %s: %d rows is not a multiple of 16\n", t->name, (int)t->dims[1]);
        W.m += (int)t->dims[1];
    }
    if (interleave && (parts.size() != 2 || parts[0]->dims[1] != parts[1]->dims[1] || parts[0]->dims[1] % 32))
        LG_BUILD_FAIL("lg_b200: %s / gate-up pair cannot be interleaved\n", t0->name);
    W.nkp = W.k / 64;
    W.n_row_tiles = ((W.m + 15) / 16 + 3) / 4 * 4;          // padded with zero tiles: the kernels fetch groups of up to 4
    W.ldo = W.n_row_tiles * 16;
    const size_t tiles = (size_t)W.n_row_tiles * W.nkp;
    const size_t tq = lg_tile_bytes(W.fmt) / 16;             // uint4 per tile
    W.wq = dalloc<uint4>(tiles * tq);
    W.ws = dalloc<uint2>(tiles * 8);
    if (W.fmt != LG_FMT_Q4_0) W.wd = dalloc<uint2>(tiles * 8);
    if (W.fmt == LG_FMT_I8M) W.wm = dalloc<uint4>(tiles * 8);
    const int nsb = W.k / 32;

    // file bytes of one part on the device (dense parts: re-encoded as q8_0 first)
    auto stage_part = [&](const struct gguf_tensor *t, uint8_t *dst, size_t bytes) {
        if (!dense) { h2d_sync(dst, t->data, bytes); return; }
        const int64_t n = (int64_t)t->dims[1] * W.k;
        std::vector<float> f((size_t)W.k);
        std::vector<uint8_t> enc(bytes);
        const size_t esz = t->type == GGML_TYPE_F32 ? 4 : 2;
        for (int64_t r = 0; r < (int64_t)t->dims[1]; r++) {
            dequantize_into(t->type, (const uint8_t *)t->data + (size_t)r * W.k * esz, f.data(), W.k);
            for (int b = 0; b < W.k / 32; b++) {
                float amax = 0.0f;
                for (int j = 0; j < 32; j++) amax = fmaxf(amax, fabsf(f[(size_t)b * 32 + j]));
                const __half dh = __float2half_rn(amax / 127.0f);
                const float d = __half2float(dh), inv = d > 0.0f ? 1.0f / d : 0.0f;
                uint8_t *o = enc.data() + ((size_t)r * (W.k / 32) + b) * 34;
                memcpy(o, &dh, 2);
                for (int j = 0; j < 32; j++) {
                    int q = (int)lrintf(f[(size_t)b * 32 + j] * inv);
                    o[2 + j] = (uint8_t)(int8_t)(q < -127 ? -127 : q > 127 ? 127 : q);
                }
            }
        }
        (void)n;
        h2d_sync(dst, enc.data(), bytes);
    };
    auto repack = [&](const uint8_t *a, const uint8_t *b, size_t toff, int rows, int rts) {
        if (W.fmt >= LG_FMT_I8) {
            const size_t threads = (size_t)rts * W.nkp * 64;
            lg_repack_i8<<<(unsigned)((threads + 255) / 256), 256, 0, e->stream>>>(a, b, (int)type, W.wq + toff * tq, W.ws + toff * 8, W.wd + toff * 8,
                                                                                  W.wm ? W.wm + toff * 8 : nullptr, rows, nsb, rts);
        } else {
            const size_t threads = (size_t)rts * W.nkp * 32;
            const unsigned blocks = (unsigned)((threads + 255) / 256);
            if (W.fmt == LG_FMT_Q4_0) lg_repack_q4_0<<<blocks, 256, 0, e->stream>>>(a, b, W.wq + toff * 32, W.ws + toff * 8, rows, nsb, rts);
            else lg_repack_q4_K<<<blocks, 256, 0, e->stream>>>(a, b, W.wq + toff * 32, W.ws + toff * 8, W.wd + toff * 8, rows, nsb, rts);
        }
        LG_CHECK(cudaGetLastError());
        LG_CHECK(cudaStreamSynchronize(e->stream));
    };
    if (interleave) {
        const int rows = (int)parts[0]->dims[1];
        const size_t bytes = ggml_nbytes(type, (int64_t)rows * W.k);
        uint8_t *stage = nullptr;
        LG_CHECK(cudaMalloc(&stage, 2 * bytes));
        stage_part(parts[0], stage, bytes);
        stage_part(parts[1], stage + bytes, bytes);
        repack(stage, stage + bytes, 0, rows, W.n_row_tiles);
        cudaFree(stage);
        W.file_bytes = 2 * bytes;
        e->weight_bytes += W.file_bytes;
        return W;
    }
    int row_off = 0;
    for (auto t : parts) {
        const int rows = (int)t->dims[1];
        const size_t bytes = ggml_nbytes(type, (int64_t)rows * W.k);
        uint8_t *stage = nullptr;
        LG_CHECK(cudaMalloc(&stage, bytes));
        stage_part(t, stage, bytes);
        repack(stage, nullptr, (size_t)(row_off / 16) * W.nkp, rows, (rows + 15) / 16);
        cudaFree(stage);
        row_off += rows;
        W.file_bytes += bytes;
    }
    e->weight_bytes += W.file_bytes;
    return W;
}
void free_wmat(WMat &W) { cudaFree(W.wq); cudaFree(W.ws); cudaFree(W.wd); cudaFree(W.wm); W = WMat(); }

// ------------------------------------------------------------------------------------------
// launch helpers
// ------------------------------------------------------------------------------------------
int env_int(const char *name, int fb) { const char *v = getenv(name); return v && v[0] ? atoi(v) : fb; }

struct GemvPlan { int r, ks, gx, ns, cl; size_t smem; };
// dynamic shared memory of the small-M matmul: panel slice | ring | warp partials | item sums | peers' sums (cluster) | mbarriers
size_t gemv_smem_bytes(int np, int nkp_slice, int r, int fmt, int ns, int cl_ks) {
    const int stage = fmt == LG_FMT_Q4_0 ? gemv_stage_bytes<LG_FMT_Q4_0>() : fmt == LG_FMT_Q4_K ? gemv_stage_bytes<LG_FMT_Q4_K>()
                    : fmt == LG_FMT_I8 ? gemv_stage_bytes<LG_FMT_I8>() : gemv_stage_bytes<LG_FMT_I8M>();
    return (size_t)np * nkp_slice * 2 * (256 + 32) + 128 + (size_t)ns * stage + (size_t)(LG_GEMV_CW + 1) * r * np * 64 * 4
         + (cl_ks > 1 ? (size_t)(cl_ks - 1) * r * np * 64 * 4 : 0) + (2 * LG_GEMV_STAGES_MAX + 2) * 8 + 16;
}
// most dynamic shared memory a CTA may take while two CTAs still share an SM (228 KB per SM, 1 KB reserved per CTA), less
// the kernel's few static bytes
constexpr size_t GEMV_SMEM_2CTA = (233472 - 2 * 1024) / 2 - 256;
// One more ring stage where two CTAs per SM still fit: a short kernel (an item or two per CTA) then has its whole share of
// the weights in flight before the activations arrive instead of refilling a stage behind a full memory latency.
void gemv_pick_stages(GemvPlan &p, int np, int nkp_slice, int fmt) {
    static const int max_ns = env_int("LG_GEMV_STAGES", LG_GEMV_STAGES_MAX);
    const int cl_ks = p.cl ? p.ks : 0;
    p.ns = LG_GEMV_STAGES;
    p.smem = gemv_smem_bytes(np, nkp_slice, p.r, fmt, p.ns, cl_ks);
    if (max_ns >= 4 && p.smem <= GEMV_SMEM_2CTA) {
        const size_t s4 = gemv_smem_bytes(np, nkp_slice, p.r, fmt, 4, cl_ks);
        if (s4 <= GEMV_SMEM_2CTA) { p.ns = 4; p.smem = s4; }
    }
}
constexpr size_t GEMV_SMEM_MAX = 200 * 1024, ATTN_SMEM_MAX = 220 * 1024;
constexpr int MAX_KV_HEADS = 64;

template <int R, int NP, int FMT, int EPI> void gemv_attr() {
    LG_CHECK(cudaFuncSetAttribute(lg_gemv_kernel<R, NP, FMT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMV_SMEM_MAX));
}
template <int R, int FMT> void gemv_attr_rf() {
    gemv_attr<R, 1, FMT, LG_EPI_STORE>(); gemv_attr<R, 2, FMT, LG_EPI_STORE>();
}
template <int FMT> void gemv_attr_f() {
    gemv_attr_rf<1, FMT>(); gemv_attr_rf<2, FMT>(); gemv_attr_rf<4, FMT>();
    gemv_attr<4, 1, FMT, LG_EPI_HEAD>(); gemv_attr<4, 2, FMT, LG_EPI_HEAD>();
    gemv_attr<4, 1, FMT, LG_EPI_GEGLU>(); gemv_attr<4, 2, FMT, LG_EPI_GEGLU>();
    gemv_attr<1, 1, FMT, LG_EPI_SUMS>(); gemv_attr<1, 2, FMT, LG_EPI_SUMS>();
    gemv_attr<2, 1, FMT, LG_EPI_SUMS>(); gemv_attr<2, 2, FMT, LG_EPI_SUMS>();
    gemv_attr<4, 1, FMT, LG_EPI_SUMS>(); gemv_attr<4, 2, FMT, LG_EPI_SUMS>();
    gemv_attr<2, 1, FMT, LG_EPI_GATE>(); gemv_attr<2, 2, FMT, LG_EPI_GATE>();
}
// Opt every kernel into large dynamic shared memory once, outside any stream capture.
template <int NT, int FMT, int EPI> void pf_attr() {
    LG_CHECK(cudaFuncSetAttribute(lg_pf_gemm_kernel<NT, FMT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pf_smem_bytes<NT, FMT>()));
}
template <int NT> void pf_attr_n() {
    pf_attr<NT, LG_FMT_Q4_0, LG_PF_STORE>(); pf_attr<NT, LG_FMT_Q4_0, LG_PF_GEGLU>();
    pf_attr<NT, LG_FMT_Q4_K, LG_PF_STORE>(); pf_attr<NT, LG_FMT_Q4_K, LG_PF_GEGLU>();
}
// cudaFuncSetAttribute applies to the current device only, so the opt-in is tracked per device.
template <int HD> void attn_cluster_attr() {
    LG_CHECK(cudaFuncSetAttribute(lg_attn_cluster_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ATTN_SMEM_MAX));
    LG_CHECK(cudaFuncSetAttribute(lg_attn_cluster_kernel<HD>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
}
void set_kernel_attributes() {
    static bool done[64] = {false};
    int dev = 0;
    LG_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) { fprintf(stderr, "lg_b200: device ordinal %d out of range\n", dev); exit(1); }
    if (done[dev]) return;
    done[dev] = true;
    gemv_attr_f<LG_FMT_Q4_0>(); gemv_attr_f<LG_FMT_Q4_K>(); gemv_attr_f<LG_FMT_I8>(); gemv_attr_f<LG_FMT_I8M>();
    LG_CHECK(cudaFuncSetAttribute(lg_attn_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ATTN_SMEM_MAX));
    LG_CHECK(cudaFuncSetAttribute(lg_attn_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ATTN_SMEM_MAX));
    LG_CHECK(cudaFuncSetAttribute(lg_attn_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ATTN_SMEM_MAX));
    LG_CHECK(cudaFuncSetAttribute(lg_attn_kernel<512>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ATTN_SMEM_MAX));
    attn_cluster_attr<64>(); attn_cluster_attr<128>(); attn_cluster_attr<256>(); attn_cluster_attr<512>();
    pf_attr_n<64>(); pf_attr_n<128>(); pf_attr_n<256>();
    LG_CHECK(cudaFuncSetAttribute(lg_attn_deep_kernel<128, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ATTN_SMEM_MAX));
    LG_CHECK(cudaFuncSetAttribute(lg_attn_deep_kernel<128, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ATTN_SMEM_MAX));
    LG_CHECK(cudaFuncSetAttribute(lg_attn_deep_kernel<256, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ATTN_SMEM_MAX));
    LG_CHECK(cudaFuncSetAttribute(lg_attn_deep_kernel<256, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ATTN_SMEM_MAX));
    LG_CHECK(cudaFuncSetAttribute(lg_pf_attn_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pf_attn_smem<64>()));
    LG_CHECK(cudaFuncSetAttribute(lg_pf_attn_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pf_attn_smem<128>()));
    LG_CHECK(cudaFuncSetAttribute(lg_pf_attn_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pf_attn_smem<256>()));
}


// Decomposition of one matmul into CTA work items: R row tiles x one of ks column slices, walked
// by a persistent grid of about two CTAs per SM.  Few slices (each slice's partial costs an extra
// pass in the consumer), and as many row tiles per item as still leave enough items to balance.
GemvPlan plan_gemv(const Engine *e, const WMat &W, int np_actual, int want_ks, bool head, bool geglu = false, bool complete = false) {
    GemvPlan p;
    p.cl = 0;
    // The decomposition (row tiles per item, k slices) fixes the order in which a row's products are added, so it must not
    // depend on the block width: it is planned for two activation panels (5..8 rows) always; only the shared memory and the
    // ring depth at the end follow the panels this launch really has.
    const int np = 2;
    static const int cta_mult = env_int("LG_GEMV_CTAS_PER_SM", 2);
    const int ctas = e->sm_count * cta_mult;
    static const int force_r = env_int("LG_GEMV_R", 0), force_ks = env_int("LG_GEMV_KS", 0);
    p.r = 0; p.ks = want_ks;
    int ks_lo = want_ks > 0 ? want_ks : 1, ks_hi = want_ks > 0 ? want_ks : e->max_ks;
    // First choice: a single wave -- as many items as fit the resident CTAs at once (one item per CTA, no second
    // item's fill/drain behind the first), fewer k slices and fatter items on ties.
    int best = 0;
    for (int ks = ks_lo; ks <= ks_hi; ks *= 2) {
        if (W.nkp / ks > 80 && ks < ks_hi) continue;                      // keep a slice's panel below ~45 KB
        if (ks > W.nkp) break;
        for (int r = 4; r >= 1; r >>= 1) {
            int items = ((W.n_row_tiles + r - 1) / r) * ks;
            if (items <= ctas && items > best) { best = items; p.r = r; p.ks = ks; }
        }
    }
    if (best * 2 < ctas) p.r = 0;                                         // too few items for one wave: several waves instead
    for (int ks = ks_lo; ks <= ks_hi && !p.r; ks *= 2) {
        if (W.nkp / ks > 80 && ks < ks_hi) continue;
        if (ks > W.nkp) break;
        for (int r = 4; r >= 1; r >>= 1)
            if (((W.n_row_tiles + r - 1) / r) * ks >= 3 * ctas / 2 || (ks == ks_hi && r == 1)) { p.r = r; p.ks = ks; break; }
    }
    if (!p.r) { p.r = 1; p.ks = ks_lo; }
    if (head || geglu) { p.r = 4; p.ks = 1; }
    if (force_r && !head && !geglu) p.r = force_r;
    if (force_ks && want_ks <= 0 && !head && !geglu) p.ks = force_ks;
    if (p.ks > e->max_ks) p.ks = e->max_ks;
    if (p.ks > W.nkp) p.ks = W.nkp;
    for (;;) {
        int nkp_s = (W.nkp + p.ks - 1) / p.ks + 1;
        gemv_pick_stages(p, np, nkp_s, W.fmt);
        if (p.smem <= GEMV_SMEM_MAX || p.ks >= e->max_ks || p.ks * 2 > W.nkp || head || geglu) break;
        p.ks *= 2;                                   // the slice's panel does not fit: cut k finer
    }
    // items beyond one wave: spread them evenly -- every CTA walks the same number of items (or one fewer), so no CTA
    // is still on its second item while the others have left
    int groups = (W.n_row_tiles + p.r - 1) / p.r;
    int cap = head ? ctas : ctas / p.ks;
    if (cap < 1) cap = 1;
    const int waves = (groups + cap - 1) / cap;
    p.gx = (groups + waves - 1) / waves;
    if (p.gx < 1) p.gx = 1;
    // The caller wants complete rows in one CTA (an epilogue that needs them): the k slices of a row group become one
    // thread-block cluster that adds its partial sums in rank 0 -- possible with one item per CTA and a portable cluster size.
    static const int cl_on = env_int("LG_GEMV_CLUSTER", 1);
    if (complete && cl_on && p.ks > 1 && p.ks <= LG_GEMV_CL_MAX && waves == 1) p.cl = 1;
    gemv_pick_stages(p, np_actual, (W.nkp + p.ks - 1) / p.ks + 1, W.fmt);
    if (p.cl && (gemv_smem_bytes(2, (W.nkp + p.ks - 1) / p.ks + 1, p.r, W.fmt, LG_GEMV_STAGES, p.ks) > GEMV_SMEM_MAX)) {
        p.cl = 0;
        gemv_pick_stages(p, np_actual, (W.nkp + p.ks - 1) / p.ks + 1, W.fmt);
    }

    return p;
}

template <int R, int NP, int FMT, int EPI>
void launch_gemv_t(Engine *e, const LgGemvArgs &a, const GemvPlan &p) {
    if (p.smem > GEMV_SMEM_MAX) { fprintf(stderr, "lg_b200: matmul slice needs %zu bytes of shared memory\n", p.smem); exit(1); }
    dim3 grid(p.gx, p.ks);
    if (p.cl) launch_k_cluster_y(e, (lg_gemv_kernel<R, NP, FMT, EPI>), dim3(grid), dim3(LG_GEMV_THREADS), p.smem, a);
    else launch_k(e, (lg_gemv_kernel<R, NP, FMT, EPI>), dim3(grid), dim3(LG_GEMV_THREADS), p.smem, a);
}
// dispatch on the weight format (a template parameter of the kernel)
template <int R, int NP, int EPI>
void launch_gemv_f(Engine *e, const LgGemvArgs &a, const GemvPlan &p, int fmt) {
    switch (fmt) {
    case LG_FMT_Q4_0: launch_gemv_t<R, NP, LG_FMT_Q4_0, EPI>(e, a, p); break;
    case LG_FMT_Q4_K: launch_gemv_t<R, NP, LG_FMT_Q4_K, EPI>(e, a, p); break;
    case LG_FMT_I8:   launch_gemv_t<R, NP, LG_FMT_I8, EPI>(e, a, p); break;
    default:          launch_gemv_t<R, NP, LG_FMT_I8M, EPI>(e, a, p); break;
    }
}

struct GemvExtra {
    float softcap = 0.0f; float *logits = nullptr; float *amax_val = nullptr; int *amax_idx = nullptr;
    const LgPanel *outp = nullptr;            // GeGLU epilogue target
    int *ks_out = nullptr, *gx_out = nullptr;
    int ldo = 0;                              // row stride of the output when it is not the matrix's own padded row count
    const int *skip = nullptr;                // the launch does nothing when this device word is non-zero
    float *amax_val2 = nullptr;               // head epilogue: runner-up logits
    // SUMS epilogue
    const float *xres = nullptr; int ldx = 0, n_cols = 0; const float *add_w = nullptr; float4 *sums = nullptr;
    int *groups_out = nullptr;                // items of the launch (= entries of sums written)
    const float *mul = nullptr; int ld_mul = 0;   // GATE epilogue: the per-token vector the activation is multiplied by
};

// Whether a matmul can run with the SUMS epilogue: complete rows in one CTA (no k slices, or k slices reduced inside a
// cluster) and few enough items for the consumer's one-round read of the partial sums.  Decided from the matrix alone,
// never from the block's width.
bool sums_ok(const Engine *e, const WMat &W) {
    static const int on = env_int("LG_SUMS", 1);
    if (!on) return false;
    GemvPlan p = plan_gemv(e, W, 2, 0, false, false, true);
    const int groups = (W.n_row_tiles + p.r - 1) / p.r;
    return (p.ks == 1 || p.cl) && groups <= LG_SUMS_ITEMS;
}

// out[ks][tok][ldo] partial sums (EPI_STORE, optional tail), the GeGLU epilogue, or the head epilogue.
void launch_gemv(Engine *e, const WMat &W, const LgPanel &X, int M, float *out, int epi, int force_ks,
                 const GemvExtra &x = GemvExtra()) {
    int np = M > 4 ? 2 : 1;
    const bool sums = epi == LG_EPI_SUMS;
    GemvPlan p = plan_gemv(e, W, np, (epi == LG_EPI_STORE || sums) ? force_ks : 1, epi == LG_EPI_HEAD, epi == LG_EPI_GEGLU, sums);
    if (sums && p.ks > 1 && !p.cl) { fprintf(stderr, "lg_b200: the SUMS epilogue needs complete rows (see sums_ok)\n"); exit(1); }
    if (epi == LG_EPI_GATE) {                    // one panel group (32 rows) per item, the whole k range in one CTA
        p.r = 2; p.ks = 1; p.cl = 0; p.gx = std::max(1, std::min(W.n_row_tiles / 2, e->sm_count * 2));
        gemv_pick_stages(p, np, W.nkp + 1, W.fmt);
    }
    LgGemvArgs a{};
    a.wq = W.wq; a.ws = W.ws; a.wd = W.wd; a.wm = W.wm; a.x = X; a.nkp = W.nkp; a.n_row_tiles = W.n_row_tiles; a.kslices = p.ks;
    a.out = out; a.ldo = x.ldo ? x.ldo : W.ldo; a.M = M; a.softcap = x.softcap; a.logits = x.logits; a.n_valid_rows = W.m;
    a.amax_val = x.amax_val; a.amax_idx = x.amax_idx; a.amax_val2 = x.amax_val2; a.skip = x.skip; a.err = e->err;
    if (x.outp) a.outp = *x.outp;
    a.cl_ks = p.cl;
    a.xres = x.xres; a.ldx = x.ldx; a.n_cols = x.n_cols; a.add_w = x.add_w; a.sums = x.sums; a.mul = x.mul; a.ld_mul = x.ld_mul;
    a.tag = (int)e->launches; a.ns = p.ns;
    if (X.nsb * 32 != W.k) { fprintf(stderr, "lg_b200: panel width %d does not match matrix k %d\n", X.nsb * 32, W.k); exit(1); }
    if (x.ks_out) *x.ks_out = p.cl ? 1 : p.ks;
    if (x.gx_out) *x.gx_out = p.gx;
    if (x.groups_out) *x.groups_out = (W.n_row_tiles + p.r - 1) / p.r;
    if (sums) {
        if (np == 1) {
            if (p.r == 4) launch_gemv_f<4, 1, LG_EPI_SUMS>(e, a, p, W.fmt); else if (p.r == 2) launch_gemv_f<2, 1, LG_EPI_SUMS>(e, a, p, W.fmt); else launch_gemv_f<1, 1, LG_EPI_SUMS>(e, a, p, W.fmt);
        } else {
            if (p.r == 4) launch_gemv_f<4, 2, LG_EPI_SUMS>(e, a, p, W.fmt); else if (p.r == 2) launch_gemv_f<2, 2, LG_EPI_SUMS>(e, a, p, W.fmt); else launch_gemv_f<1, 2, LG_EPI_SUMS>(e, a, p, W.fmt);
        }
        return;
    }
    if (epi == LG_EPI_GATE) {
        // 32 rows per item, complete rows: the whole k range in one CTA, or k slices reduced inside a cluster
        if (W.n_row_tiles % 2) { fprintf(stderr, "lg_b200: the gate matmul needs a multiple of 32 outputs\n"); exit(1); }
        if (np == 1) launch_gemv_f<2, 1, LG_EPI_GATE>(e, a, p, W.fmt); else launch_gemv_f<2, 2, LG_EPI_GATE>(e, a, p, W.fmt);
        return;
    }
    if (epi == LG_EPI_GEGLU) {
        if (W.n_row_tiles % 4) { fprintf(stderr, "lg_b200: GeGLU matmul needs a multiple of 32 outputs\n"); exit(1); }
        if (np == 1) launch_gemv_f<4, 1, LG_EPI_GEGLU>(e, a, p, W.fmt); else launch_gemv_f<4, 2, LG_EPI_GEGLU>(e, a, p, W.fmt);
        return;
    }
    if (epi == LG_EPI_HEAD) {
        if (np == 1) launch_gemv_f<4, 1, LG_EPI_HEAD>(e, a, p, W.fmt); else launch_gemv_f<4, 2, LG_EPI_HEAD>(e, a, p, W.fmt);
        return;
    }
    if (np == 1) {
        if (p.r == 4) launch_gemv_f<4, 1, LG_EPI_STORE>(e, a, p, W.fmt); else if (p.r == 2) launch_gemv_f<2, 1, LG_EPI_STORE>(e, a, p, W.fmt); else launch_gemv_f<1, 1, LG_EPI_STORE>(e, a, p, W.fmt);
    } else {
        if (p.r == 4) launch_gemv_f<4, 2, LG_EPI_STORE>(e, a, p, W.fmt); else if (p.r == 2) launch_gemv_f<2, 2, LG_EPI_STORE>(e, a, p, W.fmt); else launch_gemv_f<1, 2, LG_EPI_STORE>(e, a, p, W.fmt);
    }
}

void launch_norm(Engine *e, int M, float *x, int ldx, int n, float eps,
                 const float *add_src, int n_parts, size_t part_stride, int ld_add, const float *add_w, float out_scale,
                 const float *norm_w, const LgPanel *panel, float *y, int ldy, const int *skip = nullptr) {
    LgNormArgs a{};
    a.skip = skip;
    a.x = x; a.ldx = ldx; a.add_src = add_src; a.n_parts = n_parts; a.part_stride = part_stride; a.ld_add = ld_add;
    a.add_w = add_w; a.out_scale = out_scale; a.norm_w = norm_w;
    if (panel) { a.panel = *panel; a.want_panel = 1; }
    a.y = y; a.ldy = ldy; a.n = n; a.eps = eps;
    a.tag = (int)e->launches;
    static const int use_cluster = env_int("LG_NORM_CLUSTER", 1);
    if (use_cluster && n >= 32 * LG_NORM_CL) {
        // one cluster of LG_NORM_CL CTAs per token row
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(M * LG_NORM_CL); cfg.blockDim = dim3(LG_NORM_CL_THREADS);
        int gpc = ((n >> 5) + LG_NORM_CL - 1) / LG_NORM_CL;
        cfg.dynamicSmemBytes = (size_t)3 * gpc * 32 * sizeof(float); cfg.stream = e->stream;
        cudaLaunchAttribute at[2];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = LG_NORM_CL; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at; cfg.numAttrs = e->pdl ? 2 : 1;
        LG_CHECK(cudaLaunchKernelEx(&cfg, lg_norm_cluster_kernel, a));
        e->launches++;
        return;
    }
    int threads = n >= 2048 ? 1024 : (n >= 512 ? 512 : 256);
    launch_k(e, lg_norm_kernel, dim3(M), dim3(threads), (size_t)(2 * n + 32) * 4, a);
}

// x = (x + rmsnorm(o) add_w) * out_scale and the next panel / f32 row, from the SUMS epilogue's partial sums.
void launch_elt(Engine *e, int M, float *x, int ldx, int n, float eps, const float *o, int ldo, int n_sums,
                const float *add_w, float out_scale, const float *norm_w, const LgPanel *panel, float *y, int ldy, const int *skip = nullptr) {
    LgEltArgs a{};
    a.x = x; a.ldx = ldx; a.o = o; a.ldo = ldo; a.sums = e->sums; a.n_sums = n_sums;
    a.add_w = add_w; a.norm_w = norm_w; a.out_scale = out_scale; a.eps = eps; a.n = n;
    if (panel) { a.panel = *panel; a.want_panel = 1; }
    a.y = y; a.ldy = ldy; a.skip = skip; a.tag = (int)e->launches;
    launch_k(e, lg_elt_kernel, dim3((n / 32 + LG_ELT_WARPS - 1) / LG_ELT_WARPS, M), dim3(LG_ELT_WARPS * 32), 0, a);
}

// A projection followed by the residual update and the next norm: x = (x + rmsnorm(W in) add_w) out_scale, then the panel /
// f32 row of rmsnorm(x) norm_w.  Where the matrix can leave complete rows (decided from the matrix alone), the matmul's
// sums epilogue + one elementwise kernel; otherwise k-slice partials + the norm kernel.
void launch_matmul_resid(Engine *e, const WMat &W, const LgPanel &in, int M, float *out, float *x, int n, float eps,
                         const float *add_w, float out_scale, const float *norm_w, const LgPanel *panel, float *y, const int *skip = nullptr) {
    if (sums_ok(e, W)) {
        int groups = 0;
        GemvExtra xs; xs.xres = x; xs.ldx = n; xs.n_cols = n; xs.add_w = add_w; xs.sums = e->sums; xs.groups_out = &groups; xs.skip = skip;
        launch_gemv(e, W, in, M, out, LG_EPI_SUMS, 0, xs);
        launch_elt(e, M, x, n, n, eps, out, W.ldo, groups, add_w, out_scale, norm_w, panel, y, n, skip);
    } else {
        int ks = 1;
        GemvExtra xs; xs.ks_out = &ks; xs.skip = skip;
        launch_gemv(e, W, in, M, out, LG_EPI_STORE, 0, xs);
        launch_norm(e, M, x, n, n, eps, out, ks, (size_t)LG_MAXM * W.ldo, W.ldo, add_w, out_scale, norm_w, panel, y, n, skip);
    }
}

size_t attn_smem(int nq, int hd) {
    size_t nq16 = (size_t)((nq + 15) & ~15), ldh = hd + 8, S = lg_attn_tile(hd);
    return 2 * nq16 * ldh * 2 + 2 * S * ldh * 2 + nq16 * S * 4 + 2 * nq16 * (S + 8) * 2 + nq16 * 8 + 64;
}

// ---- the wide (prompt) matmul -----------------------------------------------------------------
// Tiled-copy descriptor of an f16 activation block [rows][k] (row-major), box = 64 columns x nt rows,
// 128-byte swizzle: the layout tcgen05.mma reads as a K-major operand.
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
CUtensorMap act_tensor_map(const __half *ptr, int k, int rows, int nt) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        LG_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr));
        if (!p || qr != cudaDriverEntryPointSuccess) { fprintf(stderr, "lg_b200: the driver has no cuTensorMapEncodeTiled\n"); exit(1); }
        fn = (EncodeTiledFn)p;
    }
    CUtensorMap map;
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    cuuint32_t box[2] = {(cuuint32_t)LG_PF_BK, (cuuint32_t)nt};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { fprintf(stderr, "lg_b200: cuTensorMapEncodeTiled failed (%d) for k=%d rows=%d\n", (int)r, k, rows); exit(1); }
    return map;
}

CUtensorMap kv_tensor_map(const __half *ptr, int kv_dim, int seq, int S) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        LG_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr));
        if (!p || qr != cudaDriverEntryPointSuccess) { fprintf(stderr, "lg_b200: the driver has no cuTensorMapEncodeTiled\n"); exit(1); }
        fn = (EncodeTiledFn)p;
    }
    CUtensorMap map;
    cuuint64_t dims[2] = {(cuuint64_t)kv_dim, (cuuint64_t)seq};
    cuuint64_t strides[1] = {(cuuint64_t)kv_dim * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)S};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { fprintf(stderr, "lg_b200: cuTensorMapEncodeTiled failed (%d) for a cache of %d rows x %d\n", (int)r, seq, kv_dim); exit(1); }
    return map;
}

template <int NT, int FMT> void launch_pf_nt(Engine *e, const CUtensorMap &tm, const LgPfGemmArgs &a, int epi, dim3 grid) {
    const size_t sm = pf_smem_bytes<NT, FMT>();
    if (epi == LG_PF_GEGLU) launch_k(e, (lg_pf_gemm_kernel<NT, FMT, LG_PF_GEGLU>), grid, dim3(LG_PF_THREADS), sm, tm, a);
    else launch_k(e, (lg_pf_gemm_kernel<NT, FMT, LG_PF_STORE>), grid, dim3(LG_PF_THREADS), sm, tm, a);
}

// out[tok][ldo] (f32) = W x X^T for n_tok <= 256 tokens; X is f16 [x_rows >= token tile][W.k], 16-byte aligned.
// epi == LG_PF_GEGLU: W holds interleaved gate/up rows and act[tok][ld_act] (f16) receives gelu(gate)*up.
// k slices of the wide matmul for a matrix with few rows (each slice writes its own plane of `out`)
int pf_kslices(const Engine *e, const WMat &W, int max_ks) {
    const int ctas = (W.n_row_tiles + 7) / 8;
    int ks = 1;
    while (ks < max_ks && ctas * ks * 2 <= e->sm_count && W.nkp / (ks * 2) >= 8) ks *= 2;
    return ks;
}

void launch_pf_gemm(Engine *e, const WMat &W, const __half *X, int x_rows, int n_tok, float *out, __half *act, int ld_act, int epi,
                    int ks = 1) {
    if (n_tok < 1 || n_tok > LG_PF_MAXN) { fprintf(stderr, "lg_b200: wide matmul takes 1..%d tokens\n", LG_PF_MAXN); exit(1); }
    const int nt = n_tok > 128 ? 256 : n_tok > 64 ? 128 : 64;
    if (x_rows < nt) { fprintf(stderr, "lg_b200: activation block of %d rows is smaller than the token tile %d\n", x_rows, nt); exit(1); }
    CUtensorMap tm = act_tensor_map(X, W.k, x_rows, nt);
    LgPfGemmArgs a{};
    a.wq = W.wq; a.ws = W.ws; a.wd = W.wd; a.nkp = W.nkp; a.n_row_tiles = W.n_row_tiles; a.n_tok = n_tok;
    a.out = out; a.ldo = W.ldo; a.n_rows = W.ldo; a.act = act; a.ld_act = ld_act; a.err = e->err;
    a.part_stride = (size_t)LG_PF_MAXN * W.ldo;
    dim3 grid((W.n_row_tiles + 7) / 8, 1, epi == LG_PF_GEGLU ? 1 : ks);
    const bool k4 = W.fmt == LG_FMT_Q4_K;
    switch (nt) {
    case 64:  if (k4) launch_pf_nt<64, LG_FMT_Q4_K>(e, tm, a, epi, grid); else launch_pf_nt<64, LG_FMT_Q4_0>(e, tm, a, epi, grid); break;
    case 128: if (k4) launch_pf_nt<128, LG_FMT_Q4_K>(e, tm, a, epi, grid); else launch_pf_nt<128, LG_FMT_Q4_0>(e, tm, a, epi, grid); break;
    default:  if (k4) launch_pf_nt<256, LG_FMT_Q4_K>(e, tm, a, epi, grid); else launch_pf_nt<256, LG_FMT_Q4_0>(e, tm, a, epi, grid); break;
    }
}

void launch_attn(Engine *e, LgAttnArgs a, int n_tiles_max) {
    int nq = (a.H / a.Hkv) * a.M;
    size_t sm = attn_smem(nq, a.hd);
    if (sm > ATTN_SMEM_MAX) { fprintf(stderr, "lg_b200: attention tile needs %zu bytes of shared memory\n", sm); exit(1); }
    if (a.Hkv > MAX_KV_HEADS) { fprintf(stderr, "lg_b200: more than %d KV heads\n", MAX_KV_HEADS); exit(1); }
    if ((size_t)nq * n_tiles_max * 8 > 2 * (size_t)lg_attn_tile(a.hd) * (a.hd + 8) * 2) {
        fprintf(stderr, "lg_b200: %d key tiles x %d queries exceed the merge buffer of the attention kernel\n", n_tiles_max, nq); exit(1);
    }
    a.tickets = e->tickets; a.tag = (int)e->launches;
    dim3 grid(a.Hkv, n_tiles_max), block(LG_ATTN_THREADS);
    switch (a.hd) {
    case 64:  launch_k(e, lg_attn_kernel<64>, grid, block, sm, a); break;
    case 128: launch_k(e, lg_attn_kernel<128>, grid, block, sm, a); break;
    case 256: launch_k(e, lg_attn_kernel<256>, grid, block, sm, a); break;
    case 512: launch_k(e, lg_attn_kernel<512>, grid, block, sm, a); break;
    default: fprintf(stderr, "lg_b200: head size %d unsupported (64, 128, 256, 512)\n", a.hd); exit(1);
    }
}

// Long-context sessions: full-attention layers walk spans of G tiles of 64 keys per CTA (lg_attn_deep_kernel).
// G is a property of the cache length alone, so every query position sees the same decomposition in plain and
// in speculative decoding.  0 = the one-tile-per-CTA kernel.
int g_deep_min = -1, g_deep_force = 0;
int deep_span_tiles(const Engine *e, int max_seq, int n_kv_heads, int hd, int nq) {
    if (g_deep_min < 0) { g_deep_min = env_int("LG_ATTN_DEEP_MIN", 4096); g_deep_force = env_int("LG_ATTN_DEEP_G", 0); }
    static const int on = env_int("LG_ATTN_DEEP", 1);
    if (!on || max_seq < g_deep_min || (hd != 128 && hd != 256) || ((nq + 15) & ~15) > 32) return 0;
    if (g_deep_force > 0) return g_deep_force;
    const int tiles = (max_seq + LG_DEEP_S - 1) / LG_DEEP_S;
    const int want = std::max(1, 2 * e->sm_count / std::max(1, n_kv_heads));     // spans per KV head that fill the GPU once
    int G = (tiles + want - 1) / want;
    return G < 2 ? 0 : std::min(G, 64);
}

void launch_attn_deep(Engine *e, LgAttnArgs a, int max_seq, int G) {
    const int nq = (a.H / a.Hkv) * a.M, nmt = ((nq + 15) & ~15) / 16;
    const size_t sm = attn_deep_smem(nq, a.hd);
    const int n_spans = ((max_seq + LG_DEEP_S - 1) / LG_DEEP_S + G - 1) / G + 1;
    if (n_spans > a.n_slots || (size_t)nq * n_spans * 8 > 2 * (size_t)LG_DEEP_S * (a.hd + 8) * 2 || sm > ATTN_SMEM_MAX || a.Hkv > MAX_KV_HEADS) {
        fprintf(stderr, "lg_b200: %d key spans x %d queries do not fit the span attention kernel\n", n_spans, nq); exit(1);
    }
    a.tickets = e->tickets; a.G = G; a.tag = (int)e->launches;
    dim3 grid(a.Hkv, n_spans), block(LG_ATTN_THREADS);
    if (a.hd == 256) { if (nmt <= 1) launch_k(e, lg_attn_deep_kernel<256, 1>, grid, block, sm, a); else launch_k(e, lg_attn_deep_kernel<256, 2>, grid, block, sm, a); }
    else             { if (nmt <= 1) launch_k(e, lg_attn_deep_kernel<128, 1>, grid, block, sm, a); else launch_k(e, lg_attn_deep_kernel<128, 2>, grid, block, sm, a); }
}

int tiles_for(int window, int max_seq, int M, int hd);

const void *attn_cluster_fn(int hd) {
    switch (hd) {
    case 64: return (const void *)lg_attn_cluster_kernel<64>;
    case 128: return (const void *)lg_attn_cluster_kernel<128>;
    case 256: return (const void *)lg_attn_cluster_kernel<256>;
    case 512: return (const void *)lg_attn_cluster_kernel<512>;
    default: return nullptr;
    }
}

void attn_cluster_config(cudaLaunchConfig_t &cfg, cudaLaunchAttribute *at, int Hkv, int C, size_t smem, cudaStream_t stream, bool pdl) {
    cfg = {};
    cfg.gridDim = dim3(Hkv, C); cfg.blockDim = dim3(LG_ATTN_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 1; at[0].val.clusterDim.y = C; at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = pdl ? 2 : 1;
}

// Tiled-copy descriptor of one layer's K (or V) cache [seq rows][kv_dim] f16: boxes of 64 columns x S rows, 128-byte swizzle.
CUtensorMap kv_tensor_map(const __half *ptr, int kv_dim, int seq, int S);

// Cluster size for the attention of a layer: the CTAs of one KV head form one cluster and merge through distributed
// shared memory (lg_attn_cluster_kernel).  A sliding-window layer gets one CTA per key tile a block can touch; a
// full-attention layer (first tile always 0) may give a CTA up to 4 tiles.  The choice is a property of the layer and
// the cache (never of the block width), so plain and speculative steps of a session run the same kernel.
// 0 = no cluster (too many tiles, a ring whose length is not a whole number of tiles, or the device cannot hold such
// clusters): the ticket kernel.
int attn_cluster_size(const Engine *e, int window, int max_seq, int seq, int hd, int H, int Hkv) {
    static const int on = env_int("LG_ATTN_CLUSTER", 1);
    if (!on || Hkv < 1 || Hkv > MAX_KV_HEADS) return 0;
    const int S = lg_attn_tile(hd);
    if (seq < max_seq && seq % S) return 0;                    // a tile must not straddle the ring's wrap
    const bool from_zero = window <= 0 || window + LG_MAXM >= max_seq;      // every block's first tile is tile 0
    const int tiles = tiles_for(window, max_seq, LG_MAXM, hd);
    if (tiles > (from_zero ? 4 * LG_ATTN_CL_MAX : LG_ATTN_CL_MAX)) return 0;
    const int nq_max = (H / Hkv) * LG_MAXM;
    const size_t sm = attn_cluster_smem(nq_max, hd);
    const void *fn = attn_cluster_fn(hd);
    if (!fn || sm > ATTN_SMEM_MAX || ((nq_max + 15) & ~15) > 32) return 0;
    if ((size_t)((nq_max + 15) & ~15) * hd * 4 > (size_t)S * hd * 2) return 0;          // accumulators reuse the K tile
    // What matters is that the clusters of ALL KV heads are resident at once (a cluster that has to wait for another one
    // to finish doubles the kernel's latency).  Ask the device how many clusters of each size it can hold.
    static std::map<long long, int> cache;        // (hd, tiles, from_zero, Hkv, smem) -> chosen size
    const long long key = ((long long)hd << 48) | ((long long)tiles << 40) | ((long long)from_zero << 39) | ((long long)Hkv << 32) | (long long)sm;
    auto it = cache.find(key);
    if (it == cache.end()) {
        static const int verbose = env_int("LG_VERBOSE", 0), force = env_int("LG_ATTN_CLUSTER_SIZE", 0);
        int fit[LG_ATTN_CL_MAX + 1] = {0};
        for (int C = 1; C <= LG_ATTN_CL_MAX; C++) {
            cudaLaunchConfig_t cfg; cudaLaunchAttribute at[2];
            attn_cluster_config(cfg, at, Hkv, C, sm, e->stream, false);
            int n = 0;
            cudaError_t rc = cudaOccupancyMaxActiveClusters(&n, fn, &cfg);
            if (rc != cudaSuccess) { cudaGetLastError(); n = 0; }
            fit[C] = n;
        }
        int best_c = 0;
        if (!from_zero) {
            // one tile per CTA: the smallest size >= tiles that holds every head at once, else the one that holds most
            int best_n = 0;
            for (int C = tiles; C <= LG_ATTN_CL_MAX; C++) {
                const int useful = fit[C] < Hkv ? fit[C] : Hkv;
                if (useful > best_n) { best_n = useful; best_c = C; }
            }
        } else {
            // tiles are dealt round-robin: the largest size (fewest tiles per CTA) that still holds every head at once
            for (int C = std::min(tiles, LG_ATTN_CL_MAX); C >= 1; C--)
                if (fit[C] >= Hkv && (tiles + C - 1) / C <= 4) { best_c = C; break; }
        }
        if (force && force <= LG_ATTN_CL_MAX && fit[force] > 0 && (from_zero || force >= tiles)) best_c = force;
        if (verbose) {
            fprintf(stderr, "lg_b200: attention clusters (head size %d, %zu bytes of shared memory, %d KV heads, %d tiles%s): fit per size",
                    hd, sm, Hkv, tiles, from_zero ? " from tile 0" : "");
            for (int C = 1; C <= LG_ATTN_CL_MAX; C++) fprintf(stderr, " %d:%d", C, fit[C]);
            fprintf(stderr, " -> %d\n", best_c);
        }
        it = cache.emplace(key, best_c).first;
    }
    return it->second;
}

void launch_attn_cluster(Engine *e, LgAttnArgs a, int C) {
    const int nq = (a.H / a.Hkv) * a.M;
    a.tag = (int)e->launches;
    const int S = lg_attn_tile(a.hd);
    const CUtensorMap tmk = kv_tensor_map(a.kc, a.kv_dim, a.seq, S), tmv = kv_tensor_map(a.vc, a.kv_dim, a.seq, S);
    cudaLaunchConfig_t cfg; cudaLaunchAttribute at[2];
    attn_cluster_config(cfg, at, a.Hkv, C, attn_cluster_smem(nq, a.hd), e->stream, e->pdl != 0);
    switch (a.hd) {
    case 64:  LG_CHECK(cudaLaunchKernelEx(&cfg, lg_attn_cluster_kernel<64>, tmk, tmv, a)); break;
    case 128: LG_CHECK(cudaLaunchKernelEx(&cfg, lg_attn_cluster_kernel<128>, tmk, tmv, a)); break;
    case 256: LG_CHECK(cudaLaunchKernelEx(&cfg, lg_attn_cluster_kernel<256>, tmk, tmv, a)); break;
    default:  LG_CHECK(cudaLaunchKernelEx(&cfg, lg_attn_cluster_kernel<512>, tmk, tmv, a)); break;
    }
    e->launches++;
}

int tiles_for(int window, int max_seq, int M, int hd) {
    const int S = lg_attn_tile(hd);
    if (window > 0 && window + M < max_seq) return (window + M + S - 1) / S + 1;
    return (max_seq + S - 1) / S + 1;
}

// ------------------------------------------------------------------------------------------
// engine construction
// ------------------------------------------------------------------------------------------
void engine_free(Engine *e);

Engine *engine_for(const struct model *m) {
    if (g_eng && g_eng->m == m && g_eng->ctx == m->ctx) return g_eng;
    if (g_eng) { engine_free(g_eng); g_eng = nullptr; }
    set_kernel_attributes();
    Engine *e = new Engine();
    e->m = m; e->ctx = m->ctx;
    const struct config *c = &m->cfg;
    const struct gguf_context *g = m->ctx;
    int dev = 0;
    LG_CHECK(cudaGetDevice(&dev));
    LG_CHECK(cudaDeviceGetAttribute(&e->sm_count, cudaDevAttrMultiProcessorCount, dev));
    LG_CHECK(cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking));
    e->head_ctas = e->sm_count * 2;
    e->pdl = env_int("LG_PDL", 1);
    e->err = dalloc<int>(1);
    e->tickets = dalloc<int>(MAX_KV_HEADS);
    e->sums = dalloc<float4>((size_t)LG_SUMS_ITEMS * LG_MAXM);
    e->d_margin_thr = dalloc<float>(1);
    { float thr = (float)atof(getenv("LG_DRAFT_MARGIN") ? getenv("LG_DRAFT_MARGIN") : "0"); if (thr != 0.0f) h2d_sync(e->d_margin_thr, &thr, 4); }

    const int ne = c->n_embd, H = c->n_head, ple = c->n_embd_per_layer;
    const struct gguf_tensor *emb = find_t(g, -1, "token_embd.weight");
    if (!emb) { fprintf(stderr, "lg_b200: token_embd.weight is missing\n"); exit(1); }
    e->head = build_wmat(e, {emb});
    e->out_norm = upload_norm(g, -1, "output_norm.weight");
    e->rope_div = upload_norm(g, -1, "rope_freqs.weight");
    const struct gguf_tensor *pte = ple > 0 ? find_t(g, -1, "per_layer_token_embd.weight") : nullptr;
    e->has_ple = pte != nullptr;
    if (e->has_ple) {
        size_t bytes = ggml_nbytes(pte->type, (int64_t)pte->dims[0] * pte->dims[1]);
        if (!bytes) { fprintf(stderr, "lg_b200: per_layer_token_embd has unsupported type %u\n", pte->type); exit(1); }
        LG_CHECK(cudaMalloc(&e->ple_table, bytes));
        h2d_sync(e->ple_table, pte->data, bytes);
        e->ple_table_type = (int)pte->type;
        e->pmp = build_wmat(e, {find_t(g, -1, "per_layer_model_proj.weight")});
        if (e->pmp.ldo != ple * c->n_layer) { fprintf(stderr, "lg_b200: per-layer width %d x %d layers is not a multiple of 64\n", ple, c->n_layer); exit(1); }
        e->ple_proj_norm = upload_norm(g, -1, "per_layer_proj_norm.weight");
    }
    int max_qkv = 0, max_q = 0, max_ff = 0, max_hd = 0;
    e->L.resize(c->n_layer);
    for (int l = 0; l < c->n_layer; l++) {
        LayerW &w = e->L[l];
        w.hd = m->head_dim[l]; w.nkv = m->n_head_kv[l]; w.local = m->is_local[l]; w.nff = m->ffn_len[l];
        w.owns_kv = l < c->n_kv_start;
        w.src = w.owns_kv ? l : c->n_kv_start - (w.local ? 2 : 1);
        std::vector<const struct gguf_tensor *> parts{find_t(g, l, "attn_q.weight")};
        if (w.owns_kv) {
            parts.push_back(find_t(g, l, "attn_k.weight"));
            const struct gguf_tensor *v = find_t(g, l, "attn_v.weight");
            w.has_v = v != nullptr;
            if (v) parts.push_back(v);
        }
        bool one_type = true;
        for (auto t : parts) one_type = one_type && t && parts[0] && t->type == parts[0]->type;
        if (one_type) {
            w.qkv = build_wmat(e, parts);
        } else {
            int row0 = 0;
            for (auto t : parts) {
                w.qkv_parts.push_back(build_wmat(e, {t}));
                w.qkv_row0.push_back(row0);
                row0 += t ? (int)t->dims[1] : 0;
            }
            w.qkv.ldo = (row0 + 63) / 64 * 64 + 64;          // room for the last part's zero padding rows
        }
        w.o = build_wmat(e, {find_t(g, l, "attn_output.weight")});
        w.gateup = build_wmat(e, {find_t(g, l, "ffn_gate.weight"), find_t(g, l, "ffn_up.weight")}, true);
        w.down = build_wmat(e, {find_t(g, l, "ffn_down.weight")});
        if (e->has_ple) {
            w.inp_gate = build_wmat(e, {find_t(g, l, "inp_gate.weight")});
            w.proj = build_wmat(e, {find_t(g, l, "proj.weight")});
            w.post_norm = upload_norm(g, l, "post_norm.weight");
        }
        w.attn_norm = upload_norm(g, l, "attn_norm.weight");
        w.q_norm = upload_norm(g, l, "attn_q_norm.weight");
        w.k_norm = upload_norm(g, l, "attn_k_norm.weight");
        w.post_attn = upload_norm(g, l, "post_attention_norm.weight");
        w.ffn_norm = upload_norm(g, l, "ffn_norm.weight");
        w.post_ffw = upload_norm(g, l, "post_ffw_norm.weight");
        const struct gguf_tensor *os = find_t(g, l, "layer_output_scale.weight");
        w.out_scale = os ? ((const float *)os->data)[0] : 1.0f;
        if (w.qkv.ldo > max_qkv) max_qkv = w.qkv.ldo;
        if (H * w.hd > max_q) max_q = H * w.hd;
        if (w.gateup.ldo > max_ff) max_ff = w.gateup.ldo;
        if (w.hd > max_hd) max_hd = w.hd;
        if (w.local) { if (e->hd_local && e->hd_local != w.hd) { fprintf(stderr, "lg_b200: sliding-window layers disagree on the head size\n"); exit(1); } e->hd_local = w.hd; }
        else         { if (e->hd_global && e->hd_global != w.hd) { fprintf(stderr, "lg_b200: global layers disagree on the head size\n"); exit(1); } e->hd_global = w.hd; }
    }
    const int M8 = LG_MAXM;
    e->x = dalloc<float>((size_t)M8 * ne);
    e->qkv = dalloc<float>((size_t)M8 * max_qkv);
    e->qrot = dalloc<float>((size_t)M8 * max_q);
    e->oout = dalloc<float>((size_t)e->max_ks * M8 * (ne + 64));
    e->gu = dalloc<float>((size_t)M8 * max_ff);
    e->dout = dalloc<float>((size_t)e->max_ks * M8 * (ne + 64));
    e->hidden = dalloc<float>((size_t)M8 * ne);
    e->h_prev = dalloc<float>(ne);
    if (!e->hd_local) e->hd_local = e->hd_global;
    if (!e->hd_global) e->hd_global = e->hd_local;
    e->rope_local = dalloc<float2>((size_t)M8 * e->hd_local / 2);
    e->rope_global = dalloc<float2>((size_t)M8 * e->hd_global / 2);
    e->p_ne = panel_alloc(ne);
    e->p_attn = panel_alloc(max_q);
    e->p_ff = panel_alloc(c->n_ff);
    if (e->has_ple) {
        size_t total = (size_t)ple * c->n_layer;
        e->tokrow = dalloc<float>(M8 * total);
        e->pproj = dalloc<float>((size_t)M8 * e->pmp.ldo);
        e->ipl = dalloc<float>(M8 * total);
        e->pg = dalloc<float>((size_t)M8 * (ple + 64));
        e->p_ple = panel_alloc(ple);
    }
    e->amax_val = dalloc<float>((size_t)e->head_ctas * LG_MAXM);
    e->amax_idx = dalloc<int>((size_t)e->head_ctas * LG_MAXM);
    e->st = dalloc<LgRoundState>(1);
    LG_CHECK(cudaMallocHost(&e->st_host, sizeof(LgRoundState)));
    memset(e->st_host, 0, sizeof(LgRoundState));
    e->log = dalloc<int>(LOG_CAP);
    g_eng = e;
    return e;
}

void free_graphs(std::map<std::string, cudaGraphExec_t> &gs) {
    for (auto &kv : gs) cudaGraphExecDestroy(kv.second);
    gs.clear();
}

void draft_free(DraftW *d) {
    if (!d) return;
    free_graphs(d->graphs);
    free_wmat(d->pre); free_wmat(d->post); free_wmat(d->head);
    for (auto &b : d->blk) {
        free_wmat(b.q); free_wmat(b.o); free_wmat(b.gateup); free_wmat(b.down);
        cudaFree(b.attn_norm); cudaFree(b.q_norm); cudaFree(b.post_attn); cudaFree(b.ffn_norm); cudaFree(b.post_ffw);
    }
    cudaFree(d->out_norm); cudaFree(d->cat); cudaFree(d->x); cudaFree(d->hbuf); cudaFree(d->qbuf); cudaFree(d->qrot);
    cudaFree(d->rope_local); cudaFree(d->rope_global); cudaFree(d->part_ml);
    cudaFree(d->obuf); cudaFree(d->gu); cudaFree(d->part); cudaFree(d->amax_val); cudaFree(d->amax_idx); cudaFree(d->best); cudaFree(d->amax_val2); cudaFree(d->margin);
    panel_free(d->p_cat); panel_free(d->p_ni); panel_free(d->p_attn); panel_free(d->p_ff);
    delete d;
}

void engine_free(Engine *e) {
    if (!e) return;
    cudaStreamSynchronize(e->stream);
    free_graphs(e->graphs);
    draft_free(e->draft);
    for (auto &w : e->L) {
        free_wmat(w.qkv); free_wmat(w.o); free_wmat(w.gateup); free_wmat(w.down); free_wmat(w.inp_gate); free_wmat(w.proj);
        for (auto &pw : w.qkv_parts) free_wmat(pw);
        cudaFree(w.attn_norm); cudaFree(w.q_norm); cudaFree(w.k_norm); cudaFree(w.post_attn); cudaFree(w.ffn_norm);
        cudaFree(w.post_ffw); cudaFree(w.post_norm);
    }
    free_wmat(e->head); free_wmat(e->pmp);
    cudaFree(e->rope_local); cudaFree(e->rope_global); cudaFree(e->part_ml);
    cudaFree(e->ple_table); cudaFree(e->out_norm); cudaFree(e->ple_proj_norm); cudaFree(e->rope_div);
    cudaFree(e->x); cudaFree(e->qkv); cudaFree(e->qrot); cudaFree(e->oout); cudaFree(e->gu); cudaFree(e->dout);
    cudaFree(e->hidden); cudaFree(e->h_prev); cudaFree(e->part); cudaFree(e->tokrow); cudaFree(e->pproj); cudaFree(e->ipl);
    cudaFree(e->pg); cudaFree(e->logits); cudaFree(e->amax_val); cudaFree(e->amax_idx);
    panel_free(e->p_ne); panel_free(e->p_attn); panel_free(e->p_ff); panel_free(e->p_ple);
    cudaFree(e->st); cudaFreeHost(e->st_host); cudaFree(e->log); cudaFree(e->replay); cudaFree(e->d_n_replay); cudaFree(e->err); cudaFree(e->tickets); cudaFree(e->d_margin_thr);
    free(e->pick_rows);
    cudaStreamDestroy(e->stream);
    delete e;
}

// Scratch for the flash-decode partials depends on the cache geometry; (re)bind when the cache changes.
void bind_kv(Engine *e, const struct kvcache *kv) {
    if (e->kv_bound == kv && e->part) return;
    LG_CHECK(cudaStreamSynchronize(e->stream));
    free_graphs(e->graphs);
    if (e->draft) free_graphs(e->draft->graphs);
    const struct config *c = &e->m->cfg;
    int slots = 0, maxhd = 0;
    for (int l = 0; l < c->n_layer; l++) {
        int s = tiles_for(e->L[l].local ? c->sliding_window : 0, kv->max_seq, LG_MAXM, e->L[l].hd);
        if (s > slots) slots = s;
        if (e->L[l].hd > maxhd) maxhd = e->L[l].hd;
    }
    cudaFree(e->part);
    e->part_slots = slots;
    e->part = dalloc<float>((size_t)slots * LG_MAXM * c->n_head * maxhd);
    cudaFree(e->part_ml);
    e->part_ml = dalloc<float2>((size_t)slots * LG_MAXM * c->n_head);
    e->kv_bound = kv;
}

// ------------------------------------------------------------------------------------------
// the forward of M token rows (enqueue only; captured into graphs by the callers)
// ------------------------------------------------------------------------------------------
enum { F_HEAD = 1, F_LOGITS = 2, F_ACCEPT = 4, F_ADVANCE = 8, F_NOEMBED = 16 };   // NOEMBED: x rows are already in place

// `only` selects kernel classes (the benchmark times them in isolation); the default runs everything.
// C_FUSED: a class-restricted pass keeps the epilogue variants of the full step (the o / down / PLE projections that leave
// complete rows and the partial sums of the norms that follow them) instead of the plain ones.
enum { C_QKV = 1, C_O = 2, C_GATEUP = 4, C_DOWN = 8, C_HEAD = 16, C_PLE = 32, C_NORM = 64, C_ATTN = 256, C_MISC = 512,
       C_ALL = 1023, C_FUSED = 1024 };

void enqueue_forward(Engine *e, const struct kvcache *kv, int M, int flags, int only = C_ALL | C_FUSED) {
    const struct model *m = e->m;
    const struct config *c = &m->cfg;
    const int ne = c->n_embd, H = c->n_head, ple = c->n_embd_per_layer, nl = c->n_layer;
    const int *d_toks = e->st->toks, *d_pos = &e->st->pos;

    if ((only & C_MISC) && !(flags & F_NOEMBED))
        launch_k(e, lg_embed_rows, dim3(M), dim3(1024), 0, e->head.wq, e->head.ws, e->head.wd, e->head.wm, e->head.fmt, e->head.nkp, e->head.m, d_toks,
                 sqrtf((float)ne), e->x, ne);
    const int total = ple * nl;
    if (e->has_ple) {
        if (only & C_MISC) launch_k(e, lg_dequant_rows, dim3(M), dim3(256), 0, e->ple_table, e->ple_table_type, total, d_toks, c->n_vocab, 0, sqrtf((float)ple), e->tokrow, total);
        if (only & C_MISC) launch_k(e, lg_quant_rows, dim3((ne / 32 + 7) / 8, M), dim3(256), 0, e->x, ne, ne, e->p_ne);
        if (only & C_PLE) launch_gemv(e, e->pmp, e->p_ne, M, e->pproj, LG_EPI_STORE, 1);
        if (only & C_MISC) launch_k(e, lg_ple_build_kernel, dim3(nl, M), dim3(ple), 0, e->pproj, e->tokrow, e->ple_proj_norm, e->ipl, ple, e->pmp.ldo,
                                                       1.0f / sqrtf((float)ne), c->rms_eps);
    }
    // rotation tables of this block's positions, one per layer kind
    if (only & (C_ATTN | C_MISC)) {
        launch_k(e, lg_rope_tables_kernel, dim3(1, 2), dim3(256), 0, d_pos, M, e->hd_local, c->rope_freq_base_swa, (const float *)nullptr, e->rope_local,
                 e->hd_global, c->rope_freq_base, (const float *)e->rope_div, e->rope_global);
    }
    if (only & C_NORM) launch_norm(e, M, e->x, ne, ne, c->rms_eps, nullptr, 0, 0, 0, nullptr, 1.0f, e->L[0].attn_norm, &e->p_ne, nullptr, 0);

    for (int l = 0; l < nl; l++) {
        LayerW &w = e->L[l];
        const int hd = w.hd, src = w.src;
        if ((only & C_QKV) && w.qkv_parts.empty()) launch_gemv(e, w.qkv, e->p_ne, M, e->qkv, LG_EPI_STORE, 1);
        if ((only & C_QKV) && !w.qkv_parts.empty())
            for (size_t i = 0; i < w.qkv_parts.size(); i++) {     // in row order: a part's zero padding rows are overwritten by the next part
                GemvExtra xp; xp.ldo = w.qkv.ldo;
                launch_gemv(e, w.qkv_parts[i], e->p_ne, M, e->qkv + w.qkv_row0[i], LG_EPI_STORE, 1, xp);
            }
        LgAttnArgs aa{};
        aa.qkv = e->qkv; aa.ld = w.qkv.ldo; aa.q_ready = 0; aa.has_v = w.has_v; aa.owns_kv = w.owns_kv;
        aa.q_norm = w.q_norm; aa.k_norm = w.k_norm; aa.eps = c->rms_eps;
        aa.rope = w.local ? e->rope_local : e->rope_global;
        aa.kc = (__half *)kv->k[src]; aa.vc = (__half *)kv->v[src]; aa.seq = kv->seq[src]; aa.kv_dim = kv->kv_dim[src];
        aa.H = H; aa.Hkv = w.nkv; aa.hd = hd; aa.M = M;
        aa.window = w.local ? c->sliding_window : 0; aa.qpos_off = 0; aa.win_shrink = 0; aa.pos = d_pos;
        aa.n_slots = e->part_slots; aa.part = e->part; aa.part_ml = e->part_ml; aa.out_f32 = nullptr; aa.err = e->err;
        LgPanel pa = e->p_attn; pa.nsb = H * hd / 32;
        aa.out = pa;
        static const int early_kv = env_int("LG_ATTN_EARLY_KV", 1);
        aa.early_kv = early_kv && w.owns_kv;     // the target's position and this layer's older rows come from earlier graph launches
        static const int deep_local = env_int("LG_ATTN_DEEP_LOCAL", 0);
        const int deepG = (w.local && !deep_local) ? 0 : deep_span_tiles(e, kv->max_seq, w.nkv, hd, (H / w.nkv) * LG_MAXM);
        if (only & C_ATTN) {
            const int cl = deepG ? 0 : attn_cluster_size(e, aa.window, kv->max_seq, aa.seq, hd, H, w.nkv);
            if (deepG) launch_attn_deep(e, aa, kv->max_seq, deepG);
            else if (cl) launch_attn_cluster(e, aa, cl);
            else launch_attn(e, aa, tiles_for(aa.window, kv->max_seq, M, hd));
        }

        // o-projection, then x += norm(o)*w_post_attn and the ffn_norm panel.  Where the matmul can leave complete rows
        // and their partial sums (decided from the matrix, never from the block's width: a verify row must run the very
        // kernels -- and so carry the very bits -- of the plain decode step at its position), one elementwise kernel
        // follows it; otherwise the norm kernel adds the k-slice partials and reduces the row itself.
        const bool fused_pass = (only & C_ALL) == C_ALL || (only & C_FUSED);
        // a matmul followed by the residual update (and the next norm): out -> x, panel, y
        auto matmul_resid = [&](const WMat &W, const LgPanel &in, float *out, int cls, const float *add_w, float out_scale,
                                const float *norm_w, const LgPanel *panel, float *y) {
            if (fused_pass && sums_ok(e, W)) {
                int groups = 0;
                GemvExtra xs; xs.xres = e->x; xs.ldx = ne; xs.n_cols = ne; xs.add_w = add_w; xs.sums = e->sums; xs.groups_out = &groups;
                if (only & cls) launch_gemv(e, W, in, M, out, LG_EPI_SUMS, 0, xs);
                else { GemvPlan p = plan_gemv(e, W, M > 4 ? 2 : 1, 0, false, false, true); groups = (W.n_row_tiles + p.r - 1) / p.r; }
                if (only & C_NORM) launch_elt(e, M, e->x, ne, ne, c->rms_eps, out, W.ldo, groups, add_w, out_scale, norm_w, panel, y, ne);
            } else {
                int ks = 1;
                GemvExtra xs; xs.ks_out = &ks;
                if (only & cls) launch_gemv(e, W, in, M, out, LG_EPI_STORE, 0, xs); else ks = plan_gemv(e, W, M > 4 ? 2 : 1, 0, false).ks;
                if (only & C_NORM) launch_norm(e, M, e->x, ne, ne, c->rms_eps, out, ks, (size_t)LG_MAXM * W.ldo, W.ldo, add_w, out_scale, norm_w, panel, y, ne);
            }
        };
        matmul_resid(w.o, pa, e->oout, C_O, w.post_attn, 1.0f, w.ffn_norm, &e->p_ne, nullptr);
        // gate/up with the GeGLU epilogue writing the down-projection's panel
        LgPanel pf = e->p_ff; pf.nsb = w.nff / 32;
        GemvExtra xg; xg.outp = &pf;
        if (only & C_GATEUP) launch_gemv(e, w.gateup, e->p_ne, M, nullptr, LG_EPI_GEGLU, 1, xg);

        const bool last = l == nl - 1;
        const float *next_w = last ? ((flags & F_HEAD) ? e->out_norm : nullptr) : e->L[l + 1].attn_norm;
        float *y = (last && (flags & F_HEAD)) ? e->hidden : nullptr;
        const LgPanel *next_p = next_w ? &e->p_ne : nullptr;
        if (e->has_ple) {
            // down, then x += norm(down)*w_post_ffw and the panel of x itself for the PLE gate
            matmul_resid(w.down, pf, e->dout, C_DOWN, w.post_ffw, 1.0f, nullptr, &e->p_ne, nullptr);
            // the PLE gate: gelu(inp_gate x) * (this layer's per-layer input) straight into the projection's panel
            static const int gate_epi = env_int("LG_GATE_EPILOGUE", 1);
            if (gate_epi && fused_pass && w.inp_gate.n_row_tiles % 2 == 0 && w.inp_gate.nkp <= 160) {
                GemvExtra xq; xq.outp = &e->p_ple; xq.mul = e->ipl + (size_t)l * ple; xq.ld_mul = total;
                if (only & C_PLE) launch_gemv(e, w.inp_gate, e->p_ne, M, nullptr, LG_EPI_GATE, 1, xq);
            } else {
                if (only & C_PLE) launch_gemv(e, w.inp_gate, e->p_ne, M, e->pg, LG_EPI_STORE, 1);
                if (only & C_MISC) launch_k(e, lg_geglu_kernel, dim3((ple / 32 + 7) / 8, M), dim3(256), 0, e->pg, e->ipl + (size_t)l * ple, w.inp_gate.ldo, total, ple, e->p_ple);
            }
            matmul_resid(w.proj, e->p_ple, e->oout, C_PLE, w.post_norm, w.out_scale, next_w, next_p, y);
        } else {
            matmul_resid(w.down, pf, e->dout, C_DOWN, w.post_ffw, w.out_scale, next_w, next_p, y);
        }
    }
    if (e->mid_event) LG_CHECK(cudaEventRecord(e->mid_event, e->stream));
    if (flags & F_HEAD) {
        float *lg = nullptr;
        if (flags & F_LOGITS) {
            if (!e->logits) e->logits = dalloc<float>((size_t)LG_MAXM * e->head.ldo);
            lg = e->logits;
        }
        int gx = 0;
        GemvExtra xh; xh.softcap = c->logit_softcap; xh.logits = lg; xh.amax_val = e->amax_val; xh.amax_idx = e->amax_idx; xh.gx_out = &gx;
        if (only & C_HEAD) launch_gemv(e, e->head, e->p_ne, M, nullptr, LG_EPI_HEAD, 1, xh); else gx = 1;
        if (only & C_MISC) launch_k(e, lg_argmax_final, dim3(M), dim3(256), 0, (const float *)e->amax_val, (const int *)e->amax_idx, gx, e->st->out, (const float *)nullptr, (float *)nullptr);
        if (flags & F_ACCEPT) {
            if (only & C_MISC) launch_k(e, lg_accept_kernel, dim3(1), dim3(256), 0, e->st, M, e->hidden, ne, ne, e->h_prev, e->log, LOG_CAP, (flags & F_ADVANCE) ? 1 : 0);
        }
    }
}


// ------------------------------------------------------------------------------------------
// the wide prompt pass: blocks of up to LG_PF_MAXN tokens, matmuls on tcgen05
// ------------------------------------------------------------------------------------------
constexpr int PF_MAX_KS = 4;
void prefill_alloc(Engine *e) {
    PrefillBuf &b = e->pf;
    if (b.ready) return;
    const struct config *c = &e->m->cfg;
    const int ne = c->n_embd, H = c->n_head;
    int max_attn = 0, max_ff = 0, max_qkv = 0, max_o = 0, max_hd = 0;
    for (auto &w : e->L) {
        max_attn = std::max(max_attn, H * w.hd); max_ff = std::max(max_ff, w.nff);
        max_qkv = std::max(max_qkv, w.qkv.ldo); max_o = std::max(max_o, std::max(w.o.ldo, w.down.ldo));
        max_hd = std::max(max_hd, w.hd);
    }
    b.ld_attn = max_attn; b.ld_ff = max_ff;
    b.a_ne = dalloc<__half>((size_t)LG_PF_MAXN * ne);
    b.a_attn = dalloc<__half>((size_t)LG_PF_MAXN * max_attn);
    b.a_ff = dalloc<__half>((size_t)LG_PF_MAXN * max_ff);
    b.x = dalloc<float>((size_t)LG_PF_MAXN * ne);
    b.qkv = dalloc<float>((size_t)PF_MAX_KS * LG_PF_MAXN * max_qkv);
    b.o = dalloc<float>((size_t)PF_MAX_KS * LG_PF_MAXN * max_o);
    b.toks = dalloc<int>(LG_PF_MAXN);
    b.pos = dalloc<int>(LG_PF_MAXN / LG_MAXM);
    b.rope_local = dalloc<float2>((size_t)LG_PF_MAXN * max_hd / 2);
    b.rope_global = dalloc<float2>((size_t)LG_PF_MAXN * max_hd / 2);
    b.q_hi = dalloc<__half>((size_t)LG_PF_MAXN * max_attn);
    b.q_lo = dalloc<__half>((size_t)LG_PF_MAXN * max_attn);
    b.rows = dalloc<float>((size_t)LG_PF_MAXN * ne); b.ridx = dalloc<int>(LG_PF_MAXN);
    if (e->has_ple) {
        const size_t total = e->pmp.ldo;
        b.tokrow = dalloc<float>((size_t)LG_PF_MAXN * total); b.pproj = dalloc<float>((size_t)LG_PF_MAXN * total);
        b.ipl = dalloc<float>((size_t)LG_PF_MAXN * total);
        int max_g = 0;
        for (auto &w : e->L) max_g = std::max(max_g, w.inp_gate.ldo);
        b.pg = dalloc<float>((size_t)LG_PF_MAXN * max_g);
        b.a_ple = dalloc<__half>((size_t)LG_PF_MAXN * c->n_embd_per_layer);
    }
    b.ready = true;
}

// x += norm(add)*add_w (optional), x *= out_scale; yh = norm(x)*norm_w as f16 rows.  One CTA per token.
void launch_norm_pf(Engine *e, int n_tok, float *x, int n, float eps, const float *add, int n_parts, int ld_add, const float *add_w,
                    float out_scale, const float *norm_w, __half *yh, bool row_itself = false) {
    LgNormArgs a{};
    a.x = x; a.ldx = n; a.add_src = add; a.n_parts = n_parts; a.part_stride = (size_t)LG_PF_MAXN * ld_add; a.ld_add = ld_add; a.add_w = add_w; a.out_scale = out_scale;
    a.norm_w = norm_w; a.n = n; a.eps = eps; a.yh = (norm_w || row_itself) ? yh : nullptr; a.ldyh = n;   // row_itself: the f16 row is x, not a norm of it
    int threads = n >= 2048 ? 1024 : (n >= 512 ? 512 : 256);
    launch_k(e, lg_norm_kernel, dim3(n_tok), dim3(threads), (size_t)(2 * n + 32) * 4, a);
}

// One block of n <= LG_PF_MAXN prompt tokens at positions pos0.. (ids in pf.toks, group positions in pf.pos):
// fills the KV rows of every layer.  The layer matmuls see all n tokens at once; attention walks the block in
// groups of LG_MAXM query rows with the decode step's kernel, so a group's keys include the rows of the groups
// before it.  Models with per-layer embeddings take the narrow path instead.
void enqueue_prefill_block(Engine *e, const struct kvcache *kv, int n, int only = C_ALL, bool media = false) {
    const struct config *c = &e->m->cfg;
    const int ne = c->n_embd, H = c->n_head, nl = c->n_layer;
    PrefillBuf &b = e->pf;
    if (only & C_MISC) {
        launch_k(e, lg_embed_rows, dim3(n), dim3(256), 0, e->head.wq, e->head.ws, e->head.wd, e->head.wm, e->head.fmt, e->head.nkp, e->head.m,
                 (const int *)b.toks, sqrtf((float)ne), b.x, ne);
        if (media) launch_k(e, lg_inject_rows, dim3(n), dim3(256), 0, b.x, ne, (const float *)b.rows, (const int *)b.ridx, ne);
        launch_k(e, lg_rope_table_kernel, dim3((n + 7) / 8), dim3(256), 0, (const int *)b.pos, n, e->hd_local, c->rope_freq_base_swa, (const float *)nullptr, b.rope_local);
        launch_k(e, lg_rope_table_kernel, dim3((n + 7) / 8), dim3(256), 0, (const int *)b.pos, n, e->hd_global, c->rope_freq_base, (const float *)e->rope_div, b.rope_global);
    }
    const int ple = c->n_embd_per_layer, total = ple * nl;
    if (e->has_ple) {
        // per-layer inputs of the block: table rows, projection of the embedding rows, their combination
        if (only & C_MISC) {
            launch_k(e, lg_dequant_rows, dim3(n), dim3(256), 0, e->ple_table, e->ple_table_type, total, (const int *)b.toks, c->n_vocab, 0,
                     sqrtf((float)ple), b.tokrow, total);
            launch_k(e, lg_f32_to_f16_rows, dim3((ne + 255) / 256, n), dim3(256), 0, (const float *)b.x, ne, b.a_ne, ne, ne);
        }
        if (only & C_PLE) launch_pf_gemm(e, e->pmp, b.a_ne, LG_PF_MAXN, n, b.pproj, nullptr, 0, LG_PF_STORE);
        if (only & C_MISC) launch_k(e, lg_ple_build_kernel, dim3(nl, n), dim3(ple), 0, b.pproj, b.tokrow, e->ple_proj_norm, b.ipl, ple, e->pmp.ldo,
                                    1.0f / sqrtf((float)ne), c->rms_eps);
    }
    if (only & C_NORM) launch_norm_pf(e, n, b.x, ne, c->rms_eps, nullptr, 0, 0, nullptr, 1.0f, e->L[0].attn_norm, b.a_ne);
    for (int l = 0; l < nl; l++) {
        LayerW &w = e->L[l];
        const int hd = w.hd, src = w.src;
        const int gqa = H / w.nkv;
        static const int block_attn = env_int("LG_PREFILL_BLOCK_ATTN", 1);
        const bool whole = block_attn && (hd == 64 || hd == 128 || hd == 256) && LG_PFA_Q % gqa == 0;
        const int ks_q = whole ? pf_kslices(e, w.qkv, 2) : 1, ks_o = pf_kslices(e, w.o, PF_MAX_KS), ks_d = pf_kslices(e, w.down, PF_MAX_KS);
        if (only & C_QKV) launch_pf_gemm(e, w.qkv, b.a_ne, LG_PF_MAXN, n, b.qkv, nullptr, 0, LG_PF_STORE, ks_q);
        if ((only & C_ATTN) && whole) {
            // the whole block at once: rows to the cache + f16 queries, then the tiled online-softmax kernel
            LgPfPrepArgs pa{};
            pa.qkv = b.qkv; pa.ld = w.qkv.ldo; pa.n_parts = ks_q; pa.part_stride = (size_t)LG_PF_MAXN * w.qkv.ldo; pa.has_v = w.has_v; pa.owns_kv = w.owns_kv; pa.q_norm = w.q_norm; pa.k_norm = w.k_norm;
            pa.eps = c->rms_eps; pa.rope = w.local ? b.rope_local : b.rope_global;
            pa.kc = (__half *)kv->k[src]; pa.vc = (__half *)kv->v[src]; pa.seq = kv->seq[src]; pa.kv_dim = kv->kv_dim[src];
            pa.H = H; pa.Hkv = w.nkv; pa.pos = b.pos; pa.q_hi = b.q_hi; pa.q_lo = b.q_lo;
            LgPfAttnArgs fa{};
            fa.q_hi = b.q_hi; fa.q_lo = b.q_lo; fa.kc = pa.kc; fa.vc = pa.vc; fa.seq = pa.seq; fa.kv_dim = pa.kv_dim;
            fa.H = H; fa.Hkv = w.nkv; fa.n = n; fa.window = w.local ? c->sliding_window : 0; fa.pos = b.pos;
            fa.out = b.a_attn; fa.ld_out = H * hd;
            const int qb = LG_PFA_Q / gqa;
            dim3 grid(w.nkv, (n + qb - 1) / qb);
            dim3 prep_grid(n, (H + (w.owns_kv ? 2 * w.nkv : 0) + 7) / 8);           // one head vector per warp
            switch (hd) {
            case 64:  launch_k(e, lg_pf_qkv_prep_kernel<64>, prep_grid, dim3(256), 0, pa);
                      launch_k(e, lg_pf_attn_kernel<64>, grid, dim3(256), pf_attn_smem<64>(), fa); break;
            case 128: launch_k(e, lg_pf_qkv_prep_kernel<128>, prep_grid, dim3(256), 0, pa);
                      launch_k(e, lg_pf_attn_kernel<128>, grid, dim3(256), pf_attn_smem<128>(), fa); break;
            default:  launch_k(e, lg_pf_qkv_prep_kernel<256>, prep_grid, dim3(256), 0, pa);
                      launch_k(e, lg_pf_attn_kernel<256>, grid, dim3(256), pf_attn_smem<256>(), fa); break;
            }
        } else if (only & C_ATTN)
            for (int g0 = 0; g0 < n; g0 += LG_MAXM) {
                const int M = std::min(LG_MAXM, n - g0);
                LgAttnArgs aa{};
                aa.qkv = b.qkv + (size_t)g0 * w.qkv.ldo; aa.ld = w.qkv.ldo; aa.q_ready = 0; aa.has_v = w.has_v; aa.owns_kv = w.owns_kv;
                aa.q_norm = w.q_norm; aa.k_norm = w.k_norm; aa.eps = c->rms_eps;
                aa.rope = (w.local ? b.rope_local : b.rope_global) + (size_t)g0 * (hd / 2);
                aa.kc = (__half *)kv->k[src]; aa.vc = (__half *)kv->v[src]; aa.seq = kv->seq[src]; aa.kv_dim = kv->kv_dim[src];
                aa.H = H; aa.Hkv = w.nkv; aa.hd = hd; aa.M = M;
                aa.window = w.local ? c->sliding_window : 0; aa.qpos_off = 0; aa.win_shrink = 0; aa.pos = b.pos + g0 / LG_MAXM;
                aa.n_slots = e->part_slots; aa.part = e->part; aa.part_ml = e->part_ml; aa.out_f32 = nullptr;
                aa.out_h = b.a_attn + (size_t)g0 * (H * hd); aa.ld_h = H * hd;
                launch_attn(e, aa, tiles_for(aa.window, kv->max_seq, M, hd));
            }
        if (only & C_O) launch_pf_gemm(e, w.o, b.a_attn, LG_PF_MAXN, n, b.o, nullptr, 0, LG_PF_STORE, ks_o);
        if (only & C_NORM) launch_norm_pf(e, n, b.x, ne, c->rms_eps, b.o, ks_o, w.o.ldo, w.post_attn, 1.0f, w.ffn_norm, b.a_ne);
        if (only & C_GATEUP) launch_pf_gemm(e, w.gateup, b.a_ne, LG_PF_MAXN, n, nullptr, b.a_ff, w.nff, LG_PF_GEGLU);
        if (only & C_DOWN) launch_pf_gemm(e, w.down, b.a_ff, LG_PF_MAXN, n, b.o, nullptr, 0, LG_PF_STORE, ks_d);
        const float *next_w = l == nl - 1 ? nullptr : e->L[l + 1].attn_norm;
        if (e->has_ple) {
            // x += norm(down) * w_post_ffw; gate = inp_gate(x); x = (x + norm(proj(gelu(gate) * per-layer input)) * w_post_norm) * out_scale
            if (only & C_NORM) launch_norm_pf(e, n, b.x, ne, c->rms_eps, b.o, ks_d, w.down.ldo, w.post_ffw, 1.0f, nullptr, b.a_ne, true);
            if (only & C_PLE) launch_pf_gemm(e, w.inp_gate, b.a_ne, LG_PF_MAXN, n, b.pg, nullptr, 0, LG_PF_STORE);
            if (only & C_MISC) launch_k(e, lg_pf_geglu_rows, dim3((ple + 255) / 256, n), dim3(256), 0, (const float *)b.pg, (const float *)(b.ipl + (size_t)l * ple),
                                        w.inp_gate.ldo, e->pmp.ldo, ple, b.a_ple, ple);
            if (only & C_PLE) launch_pf_gemm(e, w.proj, b.a_ple, LG_PF_MAXN, n, b.o, nullptr, 0, LG_PF_STORE);
            if (only & C_NORM) launch_norm_pf(e, n, b.x, ne, c->rms_eps, b.o, 1, w.proj.ldo, w.post_norm, w.out_scale, next_w, b.a_ne);
        } else {
            if (only & C_NORM) launch_norm_pf(e, n, b.x, ne, c->rms_eps, b.o, ks_d, w.down.ldo, w.post_ffw, w.out_scale, next_w, b.a_ne);
        }
    }
}

// Whether the wide pass can take this model (LG_PREFILL_WIDE=0 keeps every prompt on the narrow path).
bool prefill_wide_ok(const Engine *e) {
    static const int on = env_int("LG_PREFILL_WIDE", 1);
    if (!on) return false;
    for (auto &w : e->L) {
        if (w.o.k != e->m->cfg.n_head * w.hd || w.down.k != w.nff || !w.qkv_parts.empty()) return false;
        // the wide matmul expands q4 tiles; layers in another format take the 8-token path
        for (const WMat *W : {&w.qkv, &w.o, &w.gateup, &w.down, &w.inp_gate, &w.proj}) if (W->wq && W->fmt > LG_FMT_Q4_K) return false;
    }
    if (e->has_ple && e->pmp.fmt > LG_FMT_Q4_K) return false;
    if (e->has_ple && (e->m->cfg.n_embd_per_layer % 64 || e->m->cfg.n_embd_per_layer > 1024 || e->pmp.ldo != e->m->cfg.n_embd_per_layer * e->m->cfg.n_layer))
        return false;
    return true;
}

// Run (capturing on first use) the forward graph for (M, flags).
void run_forward(Engine *e, const struct kvcache *kv, int M, int flags) {
    bind_kv(e, kv);
    char key[48];
    snprintf(key, sizeof key, "f%d_%d", M, flags);
    auto it = e->graphs.find(key);
    if (it == e->graphs.end()) {
        e->launches = 0;
        cudaGraph_t graph;
        if ((flags & F_LOGITS) && !e->logits) e->logits = dalloc<float>((size_t)LG_MAXM * e->head.ldo);   // not inside capture
        LG_CHECK(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeRelaxed));
        enqueue_forward(e, kv, M, flags);
        LG_CHECK(cudaStreamEndCapture(e->stream, &graph));
        cudaGraphExec_t exec;
        LG_CHECK(cudaGraphInstantiate(&exec, graph, 0));
        LG_CHECK(cudaGraphDestroy(graph));
        it = e->graphs.emplace(key, exec).first;
    }
    LG_CHECK(cudaGraphLaunch(it->second, e->stream));
}

// LG_MTP_PROFILE (any value, as in the reference: src/cuda/mtp-kernel.cuh:44-61,99-101): the verify forward runs
// un-captured with an event between its two halves, and every 50 calls the mean time of the layers and of the head is
// printed in the reference's words.  The whole-round path behind mtp_draft_device is bypassed (each call synchronous).
void run_forward_profiled(Engine *e, const struct kvcache *kv, int M, int flags) {
    static cudaEvent_t ev[3] = {nullptr, nullptr, nullptr};
    static double tl = 0, th = 0;
    static int calls = 0;
    bind_kv(e, kv);
    if (!ev[0]) for (auto &x : ev) LG_CHECK(cudaEventCreate(&x));
    if ((flags & F_LOGITS) && !e->logits) e->logits = dalloc<float>((size_t)LG_MAXM * e->head.ldo);
    e->mid_event = ev[1];
    LG_CHECK(cudaEventRecord(ev[0], e->stream));
    enqueue_forward(e, kv, M, flags);
    e->mid_event = nullptr;
    LG_CHECK(cudaEventRecord(ev[2], e->stream));
    LG_CHECK(cudaEventSynchronize(ev[2]));
    float a = 0, b = 0;
    LG_CHECK(cudaEventElapsedTime(&a, ev[0], ev[1]));
    LG_CHECK(cudaEventElapsedTime(&b, ev[1], ev[2]));
    tl += a; th += b;
    if (++calls % 50 == 0)
        fprintf(stderr, "verify profile over %d: layers %.3fms ea, head %.3fms ea\n", calls, tl / calls, th / calls);
}

void upload_round(Engine *e, const int *toks, int n, int pos) {
    LgRoundState *h = e->st_host;
    h->pos = pos;
    for (int j = 0; j < n; j++) h->toks[j] = toks[j];
    // pos and toks[] are the first 1 + LG_MAXM ints of the state
    LG_CHECK(cudaMemcpyAsync(e->st, h, sizeof(int) * (1 + n), cudaMemcpyHostToDevice, e->stream));
}

void check_err(Engine *e) {
    int err = 0;
    LG_CHECK(cudaMemcpyAsync(&err, e->err, sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    LG_CHECK(cudaStreamSynchronize(e->stream));
    if (err) { fprintf(stderr, "lg_b200: device status %d (a bounded wait inside a kernel gave up)\n", err); exit(1); }
}

// ------------------------------------------------------------------------------------------
// draft head
// ------------------------------------------------------------------------------------------
void draft_free(DraftW *d);

// Returns nullptr (after a message) when the head cannot run here: a tensor type this backend has no kernel for, or a
// head count the target's KV heads do not divide.  The caller then disables drafting; decoding continues.
DraftW *draft_build(Engine *e, struct mtp *t, const struct kvcache *kv) {
    const struct model *m = e->m;
    DraftW *d = new DraftW();
    struct SoftScope { SoftScope() { g_soft_build = true; g_soft_failed = false; } ~SoftScope() { g_soft_build = false; } } soft_scope;
    d->ni = t->n_inner; d->nb = t->n_bb; d->nff = t->n_ff; d->n_head = t->n_head; d->n_vocab = t->n_vocab;
    d->eps = t->eps; d->base_full = t->base_full; d->base_swa = t->base_swa; d->softcap = t->softcap;
    d->pre = build_wmat(e, {t->pre});
    d->head = build_wmat(e, {t->head});
    d->has_post = t->post && t->post->n_dims == 2 && (int)t->post->dims[0] == t->n_inner && (int)t->post->dims[1] == t->n_bb;
    if (d->has_post) d->post = build_wmat(e, {t->post});
    d->out_norm = upload_f32(t->out_norm, d->ni);
    int qmax = 0, maxhd = 0;
    for (int L = 0; L < t->n_layer; L++) {
        const struct mtp_layer *s = &t->l[L];
        DraftBlockW b{};
        b.q = build_wmat(e, {s->q}); b.o = build_wmat(e, {s->o});
        b.gateup = build_wmat(e, {s->gate, s->up}, true); b.down = build_wmat(e, {s->down});
        b.attn_norm = upload_f32(s->attn_norm, d->ni); b.q_norm = upload_f32(s->q_norm, s->hd);
        b.post_attn = upload_f32(s->post_attn, d->ni); b.ffn_norm = upload_f32(s->ffn_norm, d->ni);
        b.post_ffw = upload_f32(s->post_ffw, d->ni);
        b.out_scale = s->out_scale ? s->out_scale[0] : 1.0f;
        b.hd = s->hd; b.local = s->local; b.src = s->src;
        if (d->n_head * s->hd > qmax) qmax = d->n_head * s->hd;
        if (s->hd > maxhd) maxhd = s->hd;
        if (s->local) d->hd_local = s->hd; else d->hd_global = s->hd;
        d->blk.push_back(b);
        if (d->n_head % m->n_head_kv[s->src]) {
            fprintf(stderr, "lg_b200: the draft head's %d query heads are not a multiple of the target's %d KV heads\n", d->n_head, m->n_head_kv[s->src]);
            g_soft_failed = true;
        }
        if (g_soft_failed) break;
    }
    if (g_soft_failed) {
        fprintf(stderr, "lg_b200: draft head unusable on the device; drafting is off, decoding continues\n");
        draft_free(d);
        return nullptr;
    }
    d->cat = dalloc<float>(2 * d->nb + 64); d->x = dalloc<float>(d->ni + 64); d->hbuf = dalloc<float>(d->ni);     // + 64: matmuls write whole row tiles
    d->qbuf = dalloc<float>((size_t)LG_MAXM * (qmax + 64)); d->qrot = dalloc<float>(qmax);
    d->obuf = dalloc<float>((size_t)e->max_ks * LG_MAXM * (std::max(d->ni, d->nb) + 64));
    d->gu = dalloc<float>(32);
    int slots = tiles_for(0, kv->max_seq, 1, 512);
    d->n_slots_global = slots;
    d->part = dalloc<float>((size_t)slots * d->n_head * maxhd);
    d->part_ml = dalloc<float2>((size_t)slots * d->n_head);
    d->amax_val = dalloc<float>((size_t)e->head_ctas * LG_MAXM); d->amax_idx = dalloc<int>((size_t)e->head_ctas * LG_MAXM);
    d->best = dalloc<int>(LG_MAXM);
    d->amax_val2 = dalloc<float>((size_t)e->head_ctas * LG_MAXM); d->margin = dalloc<float>(LG_MAXM);
    if (!d->hd_local) d->hd_local = d->hd_global;
    if (!d->hd_global) d->hd_global = d->hd_local;
    d->rope_local = dalloc<float2>(d->hd_local / 2);
    d->rope_global = dalloc<float2>(d->hd_global / 2);
    d->p_cat = panel_alloc(2 * d->nb); d->p_ni = panel_alloc(d->ni); d->p_attn = panel_alloc(qmax); d->p_ff = panel_alloc(d->nff);
    return d;
}

// One draft: cat[0:nb] = embed(toks[slot-1]) * sqrt(nb); cat[nb:] = h_prev (first draft) or post(x) (chained);
// the head's forward; argmax -> st->toks[slot].  Position = st->dpos.
void enqueue_draft(Engine *e, DraftW *d, const struct kvcache *kv, int slot, bool chained, int set_pos_j = -1) {
    const struct model *m = e->m;
    const struct config *c = &m->cfg;
    const int ni = d->ni, nb = d->nb;
    // a chained draft does nothing when the round's drafting was called off (the previous draft's confidence margin fell
    // below the threshold): its heavy kernels return at once on this word and lg_draft_pick_kernel pads the slot
    const int *skip = chained ? &e->st->stop : nullptr;
    GemvExtra xs_; xs_.skip = skip;
    if (chained) {
        // h_prev = post(x): x still holds the previous draft's normed hidden, p_ni its panel; the matmul writes its row
        // straight into the second half of the concatenated input
        if (plan_gemv(e, d->post, 1, 1, false).ks == 1) {
            launch_gemv(e, d->post, d->p_ni, 1, d->cat + nb, LG_EPI_STORE, 1, xs_);
        } else {                                             // (a k range too long for one slice: partial planes, then slice 0 .. added by the copy)
            launch_gemv(e, d->post, d->p_ni, 1, d->obuf, LG_EPI_STORE, 1, xs_);
            launch_k(e, lg_copy_f32, dim3((nb + 255) / 256), dim3(256), 0, d->cat + nb, d->obuf, nb);
        }
    }
    // position, embedding + hidden row -> the pre-projection's panel, rotation tables: one launch
    {
        LgDraftBeginArgs b{};
        b.st = e->st; b.slot = slot; b.set_pos_j = set_pos_j;
        b.wq = e->head.wq; b.ws = e->head.ws; b.wd = e->head.wd; b.wm = e->head.wm; b.fmt = e->head.fmt; b.nkp = e->head.nkp; b.n_rows = e->head.m;
        b.scale = sqrtf((float)nb); b.h_src = chained ? nullptr : e->h_prev; b.cat = d->cat; b.nb = nb; b.p_cat = d->p_cat;
        b.hd_a = d->hd_local; b.base_a = d->base_swa; b.tab_a = d->rope_local; b.hd_b = d->hd_global; b.base_b = d->base_full; b.tab_b = d->rope_global;
        const int groups = 2 * nb / 32;
        launch_k(e, lg_draft_begin_kernel, dim3((groups + 7) / 8 + 1), dim3(256), 0, b);
    }
    if (plan_gemv(e, d->pre, 1, 1, false).ks == 1) {
        launch_gemv(e, d->pre, d->p_cat, 1, d->x, LG_EPI_STORE, 1, xs_);      // straight into the head's residual row
    } else {
        launch_gemv(e, d->pre, d->p_cat, 1, d->obuf, LG_EPI_STORE, 1, xs_);
        launch_k(e, lg_copy_f32, dim3((ni + 255) / 256), dim3(256), 0, d->x, d->obuf, ni);
    }
    launch_norm(e, 1, d->x, ni, ni, d->eps, nullptr, 0, 0, 0, nullptr, 1.0f, d->blk[0].attn_norm, &d->p_ni, nullptr, 0, skip);
    for (size_t L = 0; L < d->blk.size(); L++) {
        DraftBlockW &b = d->blk[L];
        const int hd = b.hd, src = b.src, Hkv = m->n_head_kv[src];
        launch_gemv(e, b.q, d->p_ni, 1, d->qbuf, LG_EPI_STORE, 1, xs_);
        LgAttnArgs aa{};
        aa.qkv = d->qbuf; aa.ld = b.q.ldo; aa.q_ready = 0; aa.has_v = 0; aa.owns_kv = 0;
        aa.q_norm = b.q_norm; aa.k_norm = nullptr; aa.eps = d->eps;
        aa.rope = b.local ? d->rope_local : d->rope_global;
        aa.kc = (__half *)kv->k[src]; aa.vc = (__half *)kv->v[src]; aa.seq = kv->seq[src]; aa.kv_dim = kv->kv_dim[src];
        aa.H = d->n_head; aa.Hkv = Hkv; aa.hd = hd; aa.M = 1;
        aa.window = (b.local && c->sliding_window > 0) ? c->sliding_window : 0;
        aa.qpos_off = -1; aa.win_shrink = aa.window > 0 ? 1 : 0; aa.pos = &e->st->dpos;
        aa.n_slots = d->n_slots_global; aa.part = d->part; aa.part_ml = d->part_ml; aa.err = e->err; aa.skip = skip;
        LgPanel pa = d->p_attn; pa.nsb = d->n_head * hd / 32;
        aa.out = pa; aa.out_f32 = nullptr;
        const int cl = attn_cluster_size(e, aa.window, kv->max_seq, aa.seq, hd, d->n_head, Hkv);
        if (cl) launch_attn_cluster(e, aa, cl);
        else launch_attn(e, aa, tiles_for(aa.window, kv->max_seq, 1, hd));
        launch_matmul_resid(e, b.o, pa, 1, d->obuf, d->x, ni, d->eps, b.post_attn, 1.0f, b.ffn_norm, &d->p_ni, nullptr, skip);
        GemvExtra xg; xg.outp = &d->p_ff; xg.skip = skip;
        launch_gemv(e, b.gateup, d->p_ni, 1, nullptr, LG_EPI_GEGLU, 1, xg);
        bool last = L + 1 == d->blk.size();
        launch_matmul_resid(e, b.down, d->p_ff, 1, d->obuf, d->x, ni, d->eps, b.post_ffw, b.out_scale,
                            last ? d->out_norm : d->blk[L + 1].attn_norm, &d->p_ni, last ? d->hbuf : nullptr, skip);
    }
    int gx = 0;
    GemvExtra xh; xh.softcap = d->softcap; xh.amax_val = d->amax_val; xh.amax_idx = d->amax_idx; xh.gx_out = &gx; xh.skip = skip; xh.amax_val2 = d->amax_val2;
    launch_gemv(e, d->head, d->p_ni, 1, nullptr, LG_EPI_HEAD, 1, xh);
    launch_k(e, lg_draft_pick_kernel, dim3(1), dim3(256), 0, (const float *)d->amax_val, (const int *)d->amax_idx, gx, (const float *)d->amax_val2,
             e->st, slot, (const float *)e->d_margin_thr);
}

DraftW *draft_for(Engine *e, struct mtp *t, const struct kvcache *kv) {
    if (t->cuda == (void *)-1) return nullptr;
    if (e->draft && e->draft_owner == t) return e->draft;
    if (e->draft) { draft_free(e->draft); e->draft = nullptr; }
    e->draft = draft_build(e, t, kv);
    if (!e->draft) { t->cuda = (void *)-1; e->draft_owner = nullptr; return nullptr; }     // permanently off for this head
    e->draft_owner = t;
    t->cuda = e->draft;
    return e->draft;
}

void run_draft(Engine *e, DraftW *d, const struct kvcache *kv, int slot, bool chained) {
    bind_kv(e, kv);
    char key[32];
    snprintf(key, sizeof key, "d%d_%d", slot, chained ? 1 : 0);
    auto it = d->graphs.find(key);
    if (it == d->graphs.end()) {
        cudaGraph_t graph;
        LG_CHECK(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeRelaxed));
        enqueue_draft(e, d, kv, slot, chained);
        LG_CHECK(cudaStreamEndCapture(e->stream, &graph));
        cudaGraphExec_t exec;
        LG_CHECK(cudaGraphInstantiate(&exec, graph, 0));
        LG_CHECK(cudaGraphDestroy(graph));
        it = d->graphs.emplace(key, exec).first;
    }
    LG_CHECK(cudaGraphLaunch(it->second, e->stream));
}

// Positions [pos, pos + n) must lie inside the cache: past max_seq the full-attention layers would wrap over their
// oldest rows and a block would touch more key tiles than the attention grid has.  The reference's callers guard this
// themselves (src/run.c:752 falls back to plain decode near the end); a call that got through anyway is refused.
bool pos_in_cache(const struct kvcache *kv, int pos, int n, const char *what) {
    if (pos >= 0 && n >= 0 && (long long)pos + n <= kv->max_seq) return true;
    fprintf(stderr, "lg_b200: %s at positions %d..%d lies outside the cache of %d rows\n", what, pos, pos + n - 1, kv->max_seq);
    return false;
}

int spec_n(struct model *m, struct kvcache *kv, int n, const int *toks, int pos, int *out) {
    Engine *e = engine_for(m);
    if (!pos_in_cache(kv, pos, n, "a forward")) exit(1);
    if (e->lazy.valid) {
        // the round this verify belongs to has already run (mtp_draft_device): if the caller verifies exactly the tokens it
        // was handed, the outcome is on the host already -- no launch, no wait
        bool same = e->lazy.n == n && e->lazy.pos == pos && !model_pick;
        for (int j = 0; same && j < n; j++) same = toks[j] == e->lazy.toks[j];
        e->lazy.valid = false;
        if (same) {
            for (int j = 0; j < n; j++) out[j] = e->lazy.out[j];
            return e->lazy.adv;
        }
        // other tokens than predicted (or a sampling hook): run the verify now; it overwrites the same cache rows
    }
    upload_round(e, toks, n, pos);
    int flags = F_HEAD | F_ACCEPT | (model_pick ? F_LOGITS : 0);
    static const int profile = getenv("LG_MTP_PROFILE") != nullptr;
    if (profile && n > 1) run_forward_profiled(e, kv, n, flags);
    else run_forward(e, kv, n, flags);
    const struct config *c = &m->cfg;
    if (model_pick) {
        if (!e->pick_rows) e->pick_rows = (float *)malloc((size_t)LG_MAXM * c->n_vocab * sizeof(float));
        for (int j = 0; j < n; j++)
            LG_CHECK(cudaMemcpyAsync(e->pick_rows + (size_t)j * c->n_vocab, e->logits + (size_t)j * e->head.ldo,
                                     (size_t)c->n_vocab * 4, cudaMemcpyDeviceToHost, e->stream));
        LG_CHECK(cudaStreamSynchronize(e->stream));
        e->host_syncs++;
        for (int j = 0; j < n; j++) out[j] = model_pick(e->pick_rows + (size_t)j * c->n_vocab, c->n_vocab);
        int adv = 1;
        while (adv < n && out[adv - 1] == toks[adv]) adv++;
        LG_CHECK(cudaMemcpyAsync(e->h_prev, e->hidden + (size_t)(adv - 1) * c->n_embd, (size_t)c->n_embd * 4,
                                 cudaMemcpyDeviceToDevice, e->stream));
        return adv;
    }
    LG_CHECK(cudaMemcpyAsync(e->st_host->out, e->st->out, sizeof(int) * (LG_MAXM + 1), cudaMemcpyDeviceToHost, e->stream));
    LG_CHECK(cudaStreamSynchronize(e->stream));
    e->host_syncs++;
    for (int j = 0; j < n; j++) out[j] = e->st_host->out[j];
    return e->st_host->adv;
}

// One whole round as a graph: drafts of head d (if any) into toks[1..n-1], the replay override, the verify forward of
// width n, greedy acceptance; `advance` also moves the device state on to the next round (device-resident rounds).
cudaGraphExec_t round_graph(Engine *e, const struct kvcache *kv, DraftW *d, int n, bool replay, bool advance) {
    bind_kv(e, kv);
    // a round that replays drafts needs the table's device addresses at capture time: with none set yet, make the empty one
    // (its address stays valid when a table is set later; only growing past its capacity rebuilds the round graphs)
    if (replay && !e->replay) lg_set_replay(const_cast<struct model *>(e->m), nullptr, 0);
    char key[48];
    snprintf(key, sizeof key, "r%d_%d_%d_%d", n, replay ? 1 : 0, d ? 1 : 0, advance ? 1 : 0);
    auto it = e->graphs.find(key);
    if (it == e->graphs.end()) {
        cudaGraph_t graph;
        e->launches = 0;
        LG_CHECK(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeRelaxed));
        if (d) {
            for (int j = 1; j < n; j++) {
                if (j >= 2 && !d->has_post) {           // no chaining: pad like the reference caller does
                    launch_k(e, lg_pad_drafts, dim3(1), dim3(1), 0, e->st, j, n);
                    break;
                }
                enqueue_draft(e, d, kv, j, j >= 2, j - 1);
            }
        }
        if (replay && n > 1) launch_k(e, lg_replay_drafts_kernel, dim3(1), dim3(32), 0, e->st, n, (const int *)e->replay, (const int *)e->d_n_replay);
        enqueue_forward(e, kv, n, F_HEAD | F_ACCEPT | (advance ? F_ADVANCE : 0));
        LG_CHECK(cudaStreamEndCapture(e->stream, &graph));
        cudaGraphExec_t exec;
        LG_CHECK(cudaGraphInstantiate(&exec, graph, 0));
        LG_CHECK(cudaGraphDestroy(graph));
        it = e->graphs.emplace(key, exec).first;
        e->round_launches = e->launches;
    }
    return it->second;
}

int g_round_width = LG_MTP_N;                 // verify width the blocking calls' whole-round path assumes (lg_set_round_width)

}  // namespace

// ==========================================================================================
// exported backend symbols
// ==========================================================================================
extern "C" {

int kvcache_init(struct kvcache *kv, const struct model *m, int max_seq) {
    const struct config *c = &m->cfg;
    kv->n_layer = c->n_layer; kv->max_seq = max_seq; kv->px_k = kv->px_v = nullptr;
    kv->kv_dim = (int *)calloc(c->n_layer, sizeof(int));
    kv->seq = (int *)calloc(c->n_layer, sizeof(int));
    kv->f16 = (int *)calloc(c->n_layer, sizeof(int));
    kv->k = (void **)calloc(c->n_layer, sizeof(void *));
    kv->v = (void **)calloc(c->n_layer, sizeof(void *));
    if (!kv->kv_dim || !kv->seq || !kv->f16 || !kv->k || !kv->v) return -1;
    for (int L = 0; L < c->n_layer; L++) {
        kv->kv_dim[L] = m->n_head_kv[L] * m->head_dim[L];
        if (L >= c->n_kv_start) continue;
        int seq = max_seq;
        // a ring holds the window plus the spare, rounded up to whole key tiles of 128 so that a tile never straddles the wrap
        if (m->is_local[L] && c->sliding_window > 0 && ((c->sliding_window + RING_SPARE + 127) & ~127) < max_seq)
            seq = (c->sliding_window + RING_SPARE + 127) & ~127;
        kv->seq[L] = seq;
        kv->f16[L] = 1;
        size_t bytes = (size_t)seq * kv->kv_dim[L] * 2;
        LG_CHECK(cudaMalloc(&kv->k[L], bytes)); LG_CHECK(cudaMemset(kv->k[L], 0, bytes));
        LG_CHECK(cudaMalloc(&kv->v[L], bytes)); LG_CHECK(cudaMemset(kv->v[L], 0, bytes));
    }
    LG_CHECK(cudaDeviceSynchronize());        // the fills ran on the legacy stream; forwards use their own
    return 0;
}

void kvcache_free(struct kvcache *kv) {
    if (!kv || !kv->k) return;
    if (g_eng && g_eng->kv_bound == kv) {
        cudaStreamSynchronize(g_eng->stream);
        free_graphs(g_eng->graphs);
        if (g_eng->draft) free_graphs(g_eng->draft->graphs);
        g_eng->kv_bound = nullptr;
    }
    for (int L = 0; L < kv->n_layer; L++) { cudaFree(kv->k[L]); cudaFree(kv->v[L]); }
    if (kv->px_k) for (int L = 0; L < kv->n_layer; L++) { cudaFree(kv->px_k[L]); cudaFree(kv->px_v[L]); }
    free(kv->px_k); free(kv->px_v); free(kv->k); free(kv->v); free(kv->kv_dim); free(kv->seq); free(kv->f16);
    kv->k = kv->v = kv->px_k = kv->px_v = nullptr;
    kv->kv_dim = kv->seq = kv->f16 = nullptr;
}

void kvcache_save_prefix(struct kvcache *kv, int n) {
    kv->px_k = (void **)calloc(kv->n_layer, sizeof(void *));
    kv->px_v = (void **)calloc(kv->n_layer, sizeof(void *));
    if (!kv->px_k || !kv->px_v) return;
    if (g_eng) LG_CHECK(cudaStreamSynchronize(g_eng->stream));
    for (int L = 0; L < kv->n_layer; L++) {
        if (!kv->k[L]) continue;
        int rows = n < kv->seq[L] ? n : kv->seq[L];
        size_t bytes = (size_t)rows * kv->kv_dim[L] * 2;
        LG_CHECK(cudaMalloc(&kv->px_k[L], bytes)); LG_CHECK(cudaMalloc(&kv->px_v[L], bytes));
        LG_CHECK(cudaMemcpy(kv->px_k[L], kv->k[L], bytes, cudaMemcpyDeviceToDevice));
        LG_CHECK(cudaMemcpy(kv->px_v[L], kv->v[L], bytes, cudaMemcpyDeviceToDevice));
    }
    LG_CHECK(cudaDeviceSynchronize());
}

void kvcache_restore_prefix(struct kvcache *kv, int n) {
    if (!kv->px_k) return;
    cudaStream_t s = g_eng ? g_eng->stream : 0;
    for (int L = 0; L < kv->n_layer; L++) {
        if (!kv->px_k[L]) continue;
        int rows = n < kv->seq[L] ? n : kv->seq[L];
        size_t bytes = (size_t)rows * kv->kv_dim[L] * 2;
        LG_CHECK(cudaMemcpyAsync(kv->k[L], kv->px_k[L], bytes, cudaMemcpyDeviceToDevice, s));
        LG_CHECK(cudaMemcpyAsync(kv->v[L], kv->px_v[L], bytes, cudaMemcpyDeviceToDevice, s));
    }
}

void model_forward(struct model *m, struct kvcache *kv, int token, int pos, float *logits) {
    Engine *e = engine_for(m);
    e->lazy.valid = false;
    if (!pos_in_cache(kv, pos, 1, "model_forward")) exit(1);
    upload_round(e, &token, 1, pos);
    run_forward(e, kv, 1, logits ? (F_HEAD | F_LOGITS | F_ACCEPT) : 0);
    if (logits) LG_CHECK(cudaMemcpyAsync(logits, e->logits, (size_t)m->cfg.n_vocab * 4, cudaMemcpyDeviceToHost, e->stream));
    if (logits && m->last_hidden)
        LG_CHECK(cudaMemcpyAsync(m->last_hidden, e->hidden, (size_t)m->cfg.n_embd * 4, cudaMemcpyDeviceToHost, e->stream));
    check_err(e);
}

int model_forward_next(struct model *m, struct kvcache *kv, int token, int pos) {
    int out[LG_MAXM];
    spec_n(m, kv, 1, &token, pos, out);
    return out[0];
}

// The prompt pass.  ids[i] >= 0: token id; ids[i] < 0 (only with rows): media position, embedding row -ids[i]-1 of
// `rows` enters as it is and the per-layer table row of token 0 is used (src/cpu/model-cpu.c:459-465,489-497).
static void prefill_impl(struct model *m, struct kvcache *kv, const float *rows, const int *ids, int n, int pos0) {
    Engine *e = engine_for(m);
    const int ne = m->cfg.n_embd;
    if (n <= 0) return;
    e->lazy.valid = false;
    if (!pos_in_cache(kv, pos0, n, "a prompt pass")) exit(1);
    std::vector<int> toks(n), ridx(n, -1);
    bool media = false;
    for (int i = 0; i < n; i++) {
        toks[i] = ids[i] >= 0 ? ids[i] : 0;
        if (ids[i] < 0) { if (!rows) { fprintf(stderr, "lg_b200: a media position without embedding rows\n"); exit(1); } media = true; }
    }
    int i = 0;
    if (prefill_wide_ok(e) && n >= 4 * LG_MAXM) {
        // Blocks of up to LG_PF_MAXN tokens on the wide pass.  A ragged tail of more than one attention group is padded to
        // a whole number of groups by repeating the last token (src/cuda/prefill-kernel.cuh:631-660 pads its tail the same
        // way): the cache rows the pad positions write lie past the prompt, where the next step overwrites them before any
        // query can see them.  Host staging of every block stays alive until the single synchronisation at the end.
        bind_kv(e, kv);
        prefill_alloc(e);
        std::vector<std::vector<int>> gpos_all, toks_all, ridx_all;
        std::vector<std::vector<float>> stage_all;
        while (n - i > LG_MAXM) {                                    // a last group of <= 8 tokens is cheaper on the verify path
            const int real = std::min(LG_PF_MAXN, n - i);
            const int b = (real + LG_MAXM - 1) / LG_MAXM * LG_MAXM;
            if ((long long)pos0 + i + b > kv->max_seq) break;          // pad rows would wrap onto the cache's first rows: narrow path
            gpos_all.emplace_back(LG_PF_MAXN / LG_MAXM);
            for (int g = 0; g < LG_PF_MAXN / LG_MAXM; g++) gpos_all.back()[g] = pos0 + i + g * LG_MAXM;
            toks_all.emplace_back(b);
            ridx_all.emplace_back(b, -1);
            stage_all.emplace_back();
            std::vector<int> &bt = toks_all.back(), &br = ridx_all.back();
            std::vector<float> &stage = stage_all.back();
            bool blk_media = false;
            for (int j = 0; j < b; j++) {
                const int src = i + std::min(j, real - 1);          // pad: the block's last token again
                bt[j] = toks[src];
                if (j < real && ids[src] < 0) {                      // this block's media rows, packed
                    br[j] = (int)(stage.size() / ne);
                    const float *r = rows + (size_t)(-ids[src] - 1) * ne;
                    stage.insert(stage.end(), r, r + ne);
                    blk_media = true;
                }
            }
            if (blk_media) {
                LG_CHECK(cudaMemcpyAsync(e->pf.rows, stage.data(), stage.size() * sizeof(float), cudaMemcpyHostToDevice, e->stream));
                LG_CHECK(cudaMemcpyAsync(e->pf.ridx, br.data(), sizeof(int) * b, cudaMemcpyHostToDevice, e->stream));
            }
            LG_CHECK(cudaMemcpyAsync(e->pf.toks, bt.data(), sizeof(int) * b, cudaMemcpyHostToDevice, e->stream));
            LG_CHECK(cudaMemcpyAsync(e->pf.pos, gpos_all.back().data(), sizeof(int) * (LG_PF_MAXN / LG_MAXM), cudaMemcpyHostToDevice, e->stream));
            enqueue_prefill_block(e, kv, b, C_ALL, blk_media);
            i += real;
        }
        check_err(e);                                               // the one wait: every copy above has read its host buffer by now
    }
    for (; i < n; i += LG_MAXM) {
        int b = n - i < LG_MAXM ? n - i : LG_MAXM;
        upload_round(e, toks.data() + i, b, pos0 + i);
        bool blk_media = false;
        for (int j = 0; j < b; j++) blk_media |= ids[i + j] < 0;
        if (blk_media) {
            // token embeddings first, then the media rows over them; the forward then starts from x as it stands
            launch_k(e, lg_embed_rows, dim3(b), dim3(256), 0, e->head.wq, e->head.ws, e->head.wd, e->head.wm, e->head.fmt, e->head.nkp, e->head.m,
                     (const int *)e->st->toks, sqrtf((float)ne), e->x, ne);
            for (int j = 0; j < b; j++)
                if (ids[i + j] < 0)
                    LG_CHECK(cudaMemcpyAsync(e->x + (size_t)j * ne, rows + (size_t)(-ids[i + j] - 1) * ne, sizeof(float) * ne,
                                             cudaMemcpyHostToDevice, e->stream));
        }
        run_forward(e, kv, b, blk_media ? F_NOEMBED : 0);
        LG_CHECK(cudaStreamSynchronize(e->stream));      // st_host is reused by the next upload
    }
}

void model_prefill(struct model *m, struct kvcache *kv, const int *tokens, int n, int pos0) {
    prefill_impl(m, kv, nullptr, tokens, n, pos0);
}
void model_prefill_embd(struct model *m, struct kvcache *kv, const float *rows, int n, int pos0) {
    std::vector<int> ids(n);
    for (int i = 0; i < n; i++) ids[i] = -(i + 1);
    prefill_impl(m, kv, rows, ids.data(), n, pos0);
}
void model_prefill_mixed(struct model *m, struct kvcache *kv, const float *rows, const int *ids, int n, int pos0) {
    prefill_impl(m, kv, rows, ids, n, pos0);
}
void model_prefill_reserve(void) {}

int model_forward_spec(struct model *m, struct kvcache *kv, const int *toks, int pos, int *out) {
    return spec_n(m, kv, LG_MTP_N, toks, pos, out);
}

int lg_forward_spec_n(struct model *m, struct kvcache *kv, int n, const int *toks, int pos, int *out) {
    if (n < 1 || n > LG_MAXM) return -1;
    if (!pos_in_cache(kv, pos, n, "lg_forward_spec_n")) return -2;
    return spec_n(m, kv, n, toks, pos, out);
}

int mtp_draft_device(struct mtp *t, const struct model *m, const struct kvcache *kv, int token, int pos) {
    Engine *e = engine_for(m);
    DraftW *d = draft_for(e, t, kv);
    if (!d) return -1;
    LgRoundState *h = e->st_host;
    static const int lazy_on = env_int("LG_LAZY_ROUND", 1) && getenv("LG_MTP_PROFILE") == nullptr;
    const int n = g_round_width;
    e->lazy.valid = false;
    if (lazy_on && n >= 2 && n <= LG_MAXM && !model_pick && pos >= 0 && (long long)pos + n <= kv->max_seq) {
        // The reference's caller asks for the drafts one by one and then for the verify, blocking on each answer
        // (src/run.c:54-71).  Here the first call runs the whole round on the stream -- every draft, the verify of the
        // tokens the drafts turned out to be, the acceptance -- and waits ONCE for its record; the calls that follow
        // find their answers in it.
        memset(h, 0, sizeof *h);
        h->pos = pos; h->toks[0] = token; h->n_emitted = pos + e->replay_off;
        LG_CHECK(cudaMemcpyAsync(e->st, h, sizeof *h, cudaMemcpyHostToDevice, e->stream));
        const bool replay = e->lazy_replay && e->replay != nullptr && e->n_replay > 0;
        LG_CHECK(cudaGraphLaunch(round_graph(e, kv, d, n, replay, false), e->stream));
        LG_CHECK(cudaMemcpyAsync(h, e->st, sizeof *h, cudaMemcpyDeviceToHost, e->stream));
        check_err(e);                                    // the one wait of this round
        e->host_syncs++;
        e->lazy.valid = true; e->lazy.n = n; e->lazy.pos = pos; e->lazy.adv = h->adv; e->lazy.chained = d->has_post != 0;
        for (int j = 0; j < n; j++) { e->lazy.toks[j] = h->toks[j]; e->lazy.out[j] = h->out[j]; }
        h->pos = pos;                                    // what the chained-draft call derives its slot from
        return e->lazy.toks[1];
    }
    h->pos = pos; h->toks[0] = token; h->stop = 0;
    LG_CHECK(cudaMemcpyAsync(e->st, h, sizeof(int) * 2, cudaMemcpyHostToDevice, e->stream));
    LG_CHECK(cudaMemcpyAsync(&e->st->dpos, &h->pos, sizeof(int), cudaMemcpyHostToDevice, e->stream));
    LG_CHECK(cudaMemcpyAsync(&e->st->stop, &h->stop, sizeof(int), cudaMemcpyHostToDevice, e->stream));
    run_draft(e, d, kv, 1, false);
    LG_CHECK(cudaMemcpyAsync(&h->toks[1], &e->st->toks[1], sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    LG_CHECK(cudaStreamSynchronize(e->stream));
    e->host_syncs++;
    return h->toks[1];
}

// token sits at pos-1's successor slot: the caller passes (previous draft, its position)
int mtp_draft_chain_device(struct mtp *t, const struct model *m, const struct kvcache *kv, int token, int pos) {
    Engine *e = engine_for(m);
    DraftW *d = (t->cuda && t->cuda != (void *)-1) ? draft_for(e, t, kv) : nullptr;
    if (!d || !d->has_post) return -1;
    LgRoundState *h = e->st_host;
    int slot = pos - h->pos + 1;                         // chained draft j lands in toks[j], drafted at pos + j - 1
    if (slot < 2 || slot >= LG_MAXM) return -1;
    if (e->lazy.valid) {
        // asked to extend exactly the draft the round produced: that draft's successor is known
        if (slot < e->lazy.n && pos == e->lazy.pos + slot - 1 && token == e->lazy.toks[slot - 1]) return e->lazy.toks[slot];
        // anything else leaves the recorded round behind: draft synchronously from the device state as it stands
        e->lazy.valid = false;
        for (int j = 0; j < slot - 1 && j < LG_MAXM; j++) h->toks[j] = e->lazy.toks[j];
        LG_CHECK(cudaMemcpyAsync(&e->st->pos, &h->pos, sizeof(int), cudaMemcpyHostToDevice, e->stream));
    }
    h->toks[slot - 1] = token; h->dpos = pos;
    LG_CHECK(cudaMemcpyAsync(&e->st->toks[slot - 1], &h->toks[slot - 1], sizeof(int), cudaMemcpyHostToDevice, e->stream));
    LG_CHECK(cudaMemcpyAsync(&e->st->dpos, &h->dpos, sizeof(int), cudaMemcpyHostToDevice, e->stream));
    run_draft(e, d, kv, slot, true);
    LG_CHECK(cudaMemcpyAsync(&h->toks[slot], &e->st->toks[slot], sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    LG_CHECK(cudaStreamSynchronize(e->stream));
    e->host_syncs++;
    return h->toks[slot];
}

void mtp_free_device(struct mtp *t) {
    if (!t || !t->cuda || t->cuda == (void *)-1) return;
    if (g_eng && g_eng->draft == t->cuda) { draft_free(g_eng->draft); g_eng->draft = nullptr; g_eng->draft_owner = nullptr; }
    t->cuda = nullptr;
}

// ---- extensions beyond the reference seam ---------------------------------------------------

void lg_engine_release(void) { if (g_eng) { engine_free(g_eng); g_eng = nullptr; } }

long long lg_weight_bytes(struct model *m) { return (long long)engine_for(m)->weight_bytes; }

int lg_last_hidden(struct model *m, float *out) {
    Engine *e = engine_for(m);
    LG_CHECK(cudaMemcpyAsync(out, e->h_prev, (size_t)m->cfg.n_embd * 4, cudaMemcpyDeviceToHost, e->stream));
    LG_CHECK(cudaStreamSynchronize(e->stream));
    return 0;
}

int lg_kv_row(struct model *m, struct kvcache *kv, int layer, int pos, float *k, float *v) {
    Engine *e = engine_for(m);
    if (layer < 0 || layer >= kv->n_layer || !kv->k[layer]) return 0;
    int d = kv->kv_dim[layer];
    std::vector<__half> hk(d), hv(d);
    LG_CHECK(cudaStreamSynchronize(e->stream));
    size_t off = (size_t)(pos % kv->seq[layer]) * d;
    LG_CHECK(cudaMemcpy(hk.data(), (__half *)kv->k[layer] + off, d * 2, cudaMemcpyDeviceToHost));
    LG_CHECK(cudaMemcpy(hv.data(), (__half *)kv->v[layer] + off, d * 2, cudaMemcpyDeviceToHost));
    for (int i = 0; i < d; i++) { k[i] = __half2float(hk[i]); v[i] = __half2float(hv[i]); }
    return d;
}

// Device-resident rounds: no host synchronisation between rounds.  Starting from chosen token
// `first` at position `pos`, run `n_rounds` rounds of [drafts -> verify of width n -> accept]
// back to back on the stream.  Drafts come from the head `t` (mode 1), from the replay table set
// with lg_set_replay (mode 2: the head still runs when `t` is given, its tokens are overridden),
// and n == 1 is plain greedy decode.  Emitted tokens accumulate in a device log; the call
// returns after ONE synchronisation at the end.  Returns the number of tokens emitted.
int lg_set_replay(struct model *m, const int *replay, int n) {
    Engine *e = engine_for(m);
    LG_CHECK(cudaStreamSynchronize(e->stream));
    e->lazy.valid = false;
    if (n < 0) n = 0;
    if (!e->d_n_replay) e->d_n_replay = dalloc<int>(1);
    if (n > e->replay_cap || !e->replay) {
        // the table moves: graphs that hold its address are rebuilt on their next use
        for (auto it = e->graphs.begin(); it != e->graphs.end();)
            if (it->first[0] == 'r') { cudaGraphExecDestroy(it->second); it = e->graphs.erase(it); } else ++it;
        cudaFree(e->replay);
        e->replay_cap = n > 2 * e->replay_cap ? n : 2 * e->replay_cap;
        if (e->replay_cap < 1024) e->replay_cap = 1024;
        e->replay = dalloc<int>(e->replay_cap);
    }
    if (n > 0) h2d_sync(e->replay, replay, (size_t)n * 4);
    h2d_sync(e->d_n_replay, &n, 4);
    e->n_replay = n;
    if (n == 0) e->lazy_replay = false;
    return 0;
}

// Verify width the blocking calls assume when mtp_draft_device runs a whole round ahead (default: LG_MTP_N, the width
// model_forward_spec is compiled for); callers of lg_forward_spec_n with another width set it here.
void lg_set_round_width(int n) { g_round_width = n; }
// With a replay table set, the whole-round path behind the blocking calls overrides the head's drafts too: the draft
// for position p is replay[p + offset].  enable = 0 turns the override off again.
void lg_set_replay_origin(struct model *m, int offset, int enable) {
    Engine *e = engine_for(m);
    e->replay_off = offset; e->lazy_replay = enable != 0; e->lazy.valid = false;
}
// Confidence early-exit of the draft head: a draft whose best logit leads the runner-up by less than `margin` calls off the
// drafts after it in that round (their forwards are skipped, their slots repeat the previous token and the verify rejects
// them).  0 = never (default; LG_DRAFT_MARGIN sets it at load).  Drafts never change the output, only the cost of a round.
void lg_set_draft_margin(struct model *m, float margin) {
    Engine *e = engine_for(m);
    LG_CHECK(cudaStreamSynchronize(e->stream));
    h2d_sync(e->d_margin_thr, &margin, 4);
    e->lazy.valid = false;
}
long long lg_drafts_skipped(struct model *m) { return (long long)engine_for(m)->st_host->n_skipped; }   // as of the latest lg_rounds_collect
// Blocking device-to-host waits the reference-shaped calls have made so far (the benchmark reports waits per round).
long long lg_host_syncs(struct model *m) { return engine_for(m)->host_syncs; }

int lg_rounds_begin(struct model *m, int first, int pos, int n_emitted) {
    Engine *e = engine_for(m);
    LgRoundState *h = e->st_host;
    e->lazy.valid = false;
    memset(h, 0, sizeof *h);
    h->pos = pos; h->toks[0] = first; h->n_emitted = n_emitted;
    LG_CHECK(cudaMemcpyAsync(e->st, h, sizeof *h, cudaMemcpyHostToDevice, e->stream));
    LG_CHECK(cudaStreamSynchronize(e->stream));
    e->pos_hi = pos;
    return 0;
}

int lg_rounds_enqueue(struct model *m, struct kvcache *kv, struct mtp *t, int n, int mode, int n_rounds) {
    Engine *e = engine_for(m);
    if (n < 1 || n > LG_MAXM) return -1;
    DraftW *d = (t && n > 1) ? draft_for(e, t, kv) : nullptr;
    if (mode == 1 && n > 1 && !d) return -1;
    // The position advances on the device; the host only knows an upper bound (every round accepts everything).  Rounds
    // that could step outside the cache are refused before anything is enqueued; lg_rounds_collect tightens the bound.
    if (n_rounds < 0 || (long long)e->pos_hi + (long long)n_rounds * n > kv->max_seq) {
        fprintf(stderr, "lg_b200: %d rounds of width %d from position <= %d could leave the cache of %d rows\n", n_rounds, n, e->pos_hi, kv->max_seq);
        return -2;
    }
    e->pos_hi += n_rounds * n;
    cudaGraphExec_t g = round_graph(e, kv, d, n, mode == 2, true);
    for (int r = 0; r < n_rounds; r++) LG_CHECK(cudaGraphLaunch(g, e->stream));
    return 0;
}

// Wait for the enqueued rounds; copies the state and up to `cap` log entries starting at `from`.
int lg_rounds_collect(struct model *m, int *tokens, int from, int cap, int *stats /* pos, n_emitted, n_draft, n_accept */) {
    Engine *e = engine_for(m);
    LG_CHECK(cudaMemcpyAsync(e->st_host, e->st, sizeof(LgRoundState), cudaMemcpyDeviceToHost, e->stream));
    check_err(e);
    LgRoundState *h = e->st_host;
    e->pos_hi = h->pos;
    int n = h->n_emitted - from;
    if (n > cap) n = cap;
    if (n > 0 && tokens) LG_CHECK(cudaMemcpy(tokens, e->log + from, (size_t)n * 4, cudaMemcpyDeviceToHost));
    if (stats) { stats[0] = h->pos; stats[1] = h->n_emitted; stats[2] = h->n_draft; stats[3] = h->n_accept; }
    return n > 0 ? n : 0;
}

// Enqueue, on the engine's stream, only the selected kernel classes of one verify step of width n
// (default: every weight matmul -- qkv / o / gate+up / down / PLE pair per layer and the output head):
// lets a caller time the streaming kernel alone, on cold weights, with events around the call.
// Needs a forward to have run first (the cache must be bound).
int lg_bench_matmul_pass(struct model *m, int n, int classes) {
    Engine *e = engine_for(m);
    if (n < 1 || n > LG_MAXM || !e->kv_bound) return -1;
    char key[32];
    if (classes <= 0) classes = C_QKV | C_O | C_GATEUP | C_DOWN | C_HEAD | C_PLE | C_FUSED;
    snprintf(key, sizeof key, "mm%d_%d", n, classes);
    auto it = e->graphs.find(key);
    if (it == e->graphs.end()) {
        cudaGraph_t graph;
        long long before = e->launches;
        LG_CHECK(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeRelaxed));
        enqueue_forward(e, e->kv_bound, n, F_HEAD | F_ACCEPT, classes);
        LG_CHECK(cudaStreamEndCapture(e->stream, &graph));
        e->mm_launches = (int)(e->launches - before);
        cudaGraphExec_t exec;
        LG_CHECK(cudaGraphInstantiate(&exec, graph, 0));
        LG_CHECK(cudaGraphDestroy(graph));
        it = e->graphs.emplace(key, exec).first;
    }
    LG_CHECK(cudaGraphLaunch(it->second, e->stream));
    return e->mm_launches;
}

// Enqueue (no synchronisation) the kernels of one wide prompt block of n tokens, restricted to `classes`
// (<= 0: the four layer matmuls).  Timing utility: whatever ids / activations the block buffers hold are used,
// and with the attention class the KV rows at the buffered positions are overwritten.
int lg_bench_prefill_pass(struct model *m, int n, int classes) {
    Engine *e = engine_for(m);
    if (n < 1 || n > LG_PF_MAXN || !e->kv_bound || !prefill_wide_ok(e)) return -1;
    prefill_alloc(e);
    if (classes <= 0) classes = C_QKV | C_O | C_GATEUP | C_DOWN;
    long long before = e->launches;
    enqueue_prefill_block(e, e->kv_bound, n, classes);
    return (int)(e->launches - before);
}

// Session-wide choice of the span attention kernel: caches of at least min_seq rows use it on full-attention
// layers; force_g > 0 fixes the tiles per span (tests), 0 derives it from the cache length.  Takes effect for
// forwards captured afterwards (a new cache re-captures).
void lg_set_attn_deep(int min_seq, int force_g) { g_deep_min = min_seq; g_deep_force = force_g; }

// Profiling builds (-DLG_STAMPS): copy the phase time stamps of the most recent launches to the host;
// out is [96 launches][320 CTAs][12 slots] of nanosecond timer values (0 = not written; the last slot of CTA 0 = kernel kind).  -1 in the product build.
int lg_debug_stamps(long long *out) {
#ifdef LG_STAMPS
    LG_CHECK(cudaDeviceSynchronize());
    LG_CHECK(cudaMemcpyFromSymbol(out, lg_stamps, sizeof(long long) * LG_STAMP_LAUNCHES * LG_STAMP_CTAS * LG_STAMP_SLOTS));
    return 0;
#else
    (void)out; return -1;
#endif
}
int lg_debug_clear_stamps(void) {
#ifdef LG_STAMPS
    void *p = nullptr;
    LG_CHECK(cudaGetSymbolAddress(&p, lg_stamps));
    LG_CHECK(cudaMemset(p, 0, sizeof(long long) * LG_STAMP_LAUNCHES * LG_STAMP_CTAS * LG_STAMP_SLOTS));
    LG_CHECK(cudaDeviceSynchronize());
    return 0;
#else
    return -1;
#endif
}

// Test entry for the bounded waits: one CTA waits on an mbarrier that nothing will ever complete, with a limit of
// `polls` polls, gives up, raises the status bit a real kernel would raise, and returns.  The call hands back the status
// word it read (LG_ERR_MBAR_TIMEOUT = 1 expected) and clears it, so the engine stays usable.
int lg_debug_bounded_wait(struct model *m, int polls) {
    Engine *e = engine_for(m);
    if (polls < 1 || polls > (1 << 20)) return -1;
    lg_wait_probe_kernel<<<1, 32, 0, e->stream>>>(e->err, polls);
    int err = 0;
    LG_CHECK(cudaMemcpyAsync(&err, e->err, sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    LG_CHECK(cudaMemsetAsync(e->err, 0, sizeof(int), e->stream));
    LG_CHECK(cudaStreamSynchronize(e->stream));
    return err;
}

void *lg_stream(struct model *m) { return (void *)engine_for(m)->stream; }
long long lg_round_launches(struct model *m) { return engine_for(m)->round_launches; }

}  // extern "C"
#include "lg_capi.cuh"

// ==========================================================================================
// Flash-decode for callers that must not allocate
// ==========================================================================================
// Some hosts of this library run where device allocation is off the table: inside a stream
// capture, inside a latency-critical serving loop whose memory was carved up at start-up, or
// under an allocator that owns the whole device and forbids cudaMalloc behind its back.  For
// them the split-KV attention kernel is also reachable through an entry point whose scratch
// (per-tile partial accumulators, per-tile (max, sum), the per-head tickets and the position
// word) lives in a fixed array inside the library image instead of in memory it would have to
// allocate.  Every GPU that loads the library holds this array until the process exits.
#define LG_NOALLOC_SCRATCH_BYTES (4u << 20)
static __device__ __align__(256) unsigned char lg_noalloc_scratch[LG_NOALLOC_SCRATCH_BYTES];

namespace {
// device address of the array, looked up once per device (the symbol name itself is only a
// host-side handle; a kernel must be given the address cudaGetSymbolAddress returns)
unsigned char *g_noalloc_ptr[64];

__global__ void lg_noalloc_set_pos(int *p, int v) { *p = v; }
}  // namespace

extern "C" int lg_flash_decode_noalloc(const float *d_q, const void *d_k_f16, const void *d_v_f16, int M, int H, int Hkv,
                                       int hd, int seq, int window, int pos, float *d_out, void *stream) {
    if (M < 1 || M > LG_MAXM || (hd != 64 && hd != 128 && hd != 256 && hd != 512) || Hkv < 1 || H % Hkv || Hkv > MAX_KV_HEADS ||
        seq < 1 || pos < 0 || !d_q || !d_k_f16 || !d_v_f16 || !d_out) {
        fprintf(stderr, "lg_flash_decode_noalloc: bad arguments\n");
        return -1;
    }
    // K and V rows are fetched with 16-byte asynchronous copies and q / out with 4-byte accesses: a pointer into the
    // middle of a tensor (an odd element offset) would fault on the device, so it is turned away here
    if ((((uintptr_t)d_k_f16 | (uintptr_t)d_v_f16) & 15) || (((uintptr_t)d_q | (uintptr_t)d_out) & 3)) {
        fprintf(stderr, "lg_flash_decode_noalloc: k and v must be 16-byte aligned, q and out 4-byte aligned\n");
        return -1;
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -2;
    if (!g_noalloc_ptr[dev]) {
        // first call on this device: resolve the array's device address (do this before any capture)
        void *p = nullptr;
        cudaError_t rc = cudaGetSymbolAddress(&p, lg_noalloc_scratch);
        if (rc != cudaSuccess || !p) {
            fprintf(stderr, "lg_flash_decode_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(rc));
            return -3;
        }
        set_kernel_attributes();
        g_noalloc_ptr[dev] = (unsigned char *)p;
    }
    const int max_seq = pos + M > seq ? pos + M : seq;
    const int slots = tiles_for(window, max_seq, M, hd);
    const int nq = (H / Hkv) * M;
    // layout inside the array: [tickets 256 B][pos 256 B][(max,sum) pairs][accumulators]
    const size_t ml_bytes = ((size_t)slots * M * H * sizeof(float2) + 255) & ~(size_t)255;
    const size_t acc_bytes = (size_t)slots * M * H * hd * sizeof(float);
    const size_t need = 512 + ml_bytes + acc_bytes;
    const size_t sm = attn_smem(nq, hd);
    if (need > LG_NOALLOC_SCRATCH_BYTES || sm > ATTN_SMEM_MAX ||
        (size_t)nq * slots * 8 > 2 * (size_t)lg_attn_tile(hd) * (hd + 8) * 2) {
        fprintf(stderr, "lg_flash_decode_noalloc: %d key tiles x %d rows x %d heads x %d dims need %zu bytes of scratch; "
                        "the built-in array holds %u\n", slots, M, H, hd, need, LG_NOALLOC_SCRATCH_BYTES);
        return -4;
    }
    unsigned char *base = g_noalloc_ptr[dev];
    cudaStream_t st = (cudaStream_t)stream;
    // the array keeps whatever the previous call left: tickets must start at zero
    if (cudaMemsetAsync(base, 0, 256, st) != cudaSuccess) return -5;
    lg_noalloc_set_pos<<<1, 1, 0, st>>>((int *)(base + 256), pos);
    LgAttnArgs a{};
    a.qkv = d_q; a.ld = 0; a.q_ready = 1; a.has_v = 1; a.owns_kv = 0; a.eps = 0.0f; a.rope = nullptr;
    a.kc = (__half *)d_k_f16; a.vc = (__half *)d_v_f16; a.seq = seq; a.kv_dim = Hkv * hd;
    a.H = H; a.Hkv = Hkv; a.hd = hd; a.M = M; a.n_slots = slots; a.window = window; a.qpos_off = 0; a.win_shrink = 0;
    a.pos = (const int *)(base + 256);
    a.tickets = (int *)base;
    a.part_ml = (float2 *)(base + 512);
    a.part = (float *)(base + 512 + ml_bytes);
    a.out.q = nullptr; a.out_f32 = d_out;
    dim3 grid(Hkv, slots), block(LG_ATTN_THREADS);
    switch (hd) {
    case 64:  lg_attn_kernel<64><<<grid, block, sm, st>>>(a); break;
    case 128: lg_attn_kernel<128><<<grid, block, sm, st>>>(a); break;
    case 256: lg_attn_kernel<256><<<grid, block, sm, st>>>(a); break;
    default:  lg_attn_kernel<512><<<grid, block, sm, st>>>(a); break;
    }
    cudaError_t rc = cudaGetLastError();
    if (rc != cudaSuccess) { fprintf(stderr, "lg_flash_decode_noalloc: launch failed: %s\n", cudaGetErrorString(rc)); return -6; }
    return 0;
}
