// lg_capi.cuh -- kernel-level entry points: host buffers in, host buffers out.  They run the
// SAME kernels the engine launches (repack, panel quantisation, tensor-core matmul, split-KV
// flash-decode) on caller-supplied data so each can be checked in isolation.
// Included at the end of lg_engine.cu (one translation unit).

namespace {
Engine *scratch_engine() {
    static Engine *e = nullptr;
    if (!e) {
        set_kernel_attributes();
        e = new Engine();
        int dev = 0;
        LG_CHECK(cudaGetDevice(&dev));
        LG_CHECK(cudaDeviceGetAttribute(&e->sm_count, cudaDevAttrMultiProcessorCount, dev));
        LG_CHECK(cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking));
        e->head_ctas = e->sm_count * 2;
        e->pdl = env_int("LG_PDL", 1);
        e->err = dalloc<int>(1);
        e->tickets = dalloc<int>(MAX_KV_HEADS);
    }
    return e;
}
}  // namespace

extern "C" int lg_dequant_host(int type, const void *blocks, int n_rows, int k, float *out) {
    Engine *e = scratch_engine();
    size_t bytes = ggml_nbytes((uint32_t)type, (int64_t)n_rows * k);
    if (!bytes) return -1;
    uint8_t *d_src = nullptr; float *d_out = nullptr;
    LG_CHECK(cudaMalloc(&d_src, bytes));
    LG_CHECK(cudaMalloc(&d_out, (size_t)n_rows * k * 4));
    LG_CHECK(cudaMemcpyAsync(d_src, blocks, bytes, cudaMemcpyHostToDevice, e->stream));
    launch_k(e, lg_dequant_rows, dim3(n_rows), dim3(256), 0, d_src, type, k, nullptr, n_rows, 0, 1.0f, d_out, k);
    LG_CHECK(cudaGetLastError());
    LG_CHECK(cudaMemcpyAsync(out, d_out, (size_t)n_rows * k * 4, cudaMemcpyDeviceToHost, e->stream));
    LG_CHECK(cudaStreamSynchronize(e->stream));
    cudaFree(d_src); cudaFree(d_out);
    return 0;
}

extern "C" int lg_gemv_host(int type, const void *blocks, int m, int k, const float *x, int M, int kslices, float *y) {
    if (M < 1 || M > LG_MAXM || k % 64 || (type != GGML_TYPE_Q4_0 && type != GGML_TYPE_Q4_K && !lg_fmt_is_i8(type))) return -1;
    if (ggml_blck_size((uint32_t)type) == 256 && k % 256) return -1;
    Engine *e = scratch_engine();
    struct gguf_tensor t;
    memset(&t, 0, sizeof t);
    char name[] = "lg_gemv_host";
    t.name = name; t.n_dims = 2; t.dims[0] = k; t.dims[1] = m; t.dims[2] = t.dims[3] = 1; t.type = type; t.data = (void *)blocks;
    WMat W = build_wmat(e, {&t});
    LgPanel P = panel_alloc(k);
    float *d_x = dalloc<float>((size_t)M * k);
    float *d_out = dalloc<float>((size_t)e->max_ks * LG_MAXM * W.ldo);
    LG_CHECK(cudaMemcpyAsync(d_x, x, (size_t)M * k * 4, cudaMemcpyHostToDevice, e->stream));
    launch_k(e, lg_quant_rows, dim3((k / 32 + 7) / 8, M), dim3(256), 0, d_x, k, k, P);
    LG_CHECK(cudaGetLastError());
    int ks = 1;
    GemvExtra gx; gx.ks_out = &ks;
    launch_gemv(e, W, P, M, d_out, LG_EPI_STORE, kslices, gx);
    std::vector<float> h((size_t)ks * LG_MAXM * W.ldo);
    LG_CHECK(cudaMemcpyAsync(h.data(), d_out, h.size() * 4, cudaMemcpyDeviceToHost, e->stream));
    check_err(e);
    for (int tok = 0; tok < M; tok++)
        for (int r = 0; r < m; r++) {
            float s = 0.0f;
            for (int p = 0; p < ks; p++) s += h[((size_t)p * LG_MAXM + tok) * W.ldo + r];
            y[(size_t)tok * m + r] = s;
        }
    free_wmat(W); panel_free(P); cudaFree(d_x); cudaFree(d_out);
    return 0;
}

// The matmul with complete rows + norm sums followed by the residual kernel, as the decode step chains them:
//   o = W act;  xres' = (xres + rmsnorm(o) add_w) * out_scale;  y = rmsnorm(xres') norm_w   (norm_w may be NULL: y = xres')
// act [M][k], xres [M][m] (updated in place), y [M][m].  Returns 1 when the k slices were reduced inside a cluster, 0 when one
// CTA held the whole k range, -2 when this matrix cannot leave complete rows (the engine then uses the norm kernel), -1 on bad arguments.
extern "C" int lg_matmul_resid_host(int type, const void *blocks, int m, int k, const float *act, int M, float *xres,
                                    const float *add_w, float out_scale, const float *norm_w, float eps, float *y) {
    if (M < 1 || M > LG_MAXM || k % 64 || m % 32 || (type != GGML_TYPE_Q4_0 && type != GGML_TYPE_Q4_K && !lg_fmt_is_i8(type))) return -1;
    if (ggml_blck_size((uint32_t)type) == 256 && k % 256) return -1;
    Engine *e = scratch_engine();
    if (!e->sums) e->sums = dalloc<float4>((size_t)LG_SUMS_ITEMS * LG_MAXM);
    struct gguf_tensor t;
    memset(&t, 0, sizeof t);
    char name[] = "lg_matmul_resid_host";
    t.name = name; t.n_dims = 2; t.dims[0] = k; t.dims[1] = m; t.dims[2] = t.dims[3] = 1; t.type = type; t.data = (void *)blocks;
    WMat W = build_wmat(e, {&t});
    if (!sums_ok(e, W)) { free_wmat(W); return -2; }
    LgPanel P = panel_alloc(k), Py = panel_alloc(m);
    float *d_act = dalloc<float>((size_t)M * k), *d_x = dalloc<float>((size_t)M * m), *d_y = dalloc<float>((size_t)M * m);
    float *d_out = dalloc<float>((size_t)LG_MAXM * W.ldo), *d_aw = dalloc<float>(m), *d_nw = norm_w ? dalloc<float>(m) : nullptr;
    LG_CHECK(cudaMemcpyAsync(d_act, act, (size_t)M * k * 4, cudaMemcpyHostToDevice, e->stream));
    LG_CHECK(cudaMemcpyAsync(d_x, xres, (size_t)M * m * 4, cudaMemcpyHostToDevice, e->stream));
    LG_CHECK(cudaMemcpyAsync(d_aw, add_w, (size_t)m * 4, cudaMemcpyHostToDevice, e->stream));
    if (norm_w) LG_CHECK(cudaMemcpyAsync(d_nw, norm_w, (size_t)m * 4, cudaMemcpyHostToDevice, e->stream));
    launch_k(e, lg_quant_rows, dim3((k / 32 + 7) / 8, M), dim3(256), 0, d_act, k, k, P);
    int groups = 0;
    GemvExtra xs; xs.xres = d_x; xs.ldx = m; xs.n_cols = m; xs.add_w = d_aw; xs.sums = e->sums; xs.groups_out = &groups;
    const GemvPlan pl = plan_gemv(e, W, M > 4 ? 2 : 1, 0, false, false, true);
    launch_gemv(e, W, P, M, d_out, LG_EPI_SUMS, 0, xs);
    launch_elt(e, M, d_x, m, m, eps, d_out, W.ldo, groups, d_aw, out_scale, d_nw, &Py, d_y, m);
    LG_CHECK(cudaGetLastError());
    LG_CHECK(cudaMemcpyAsync(xres, d_x, (size_t)M * m * 4, cudaMemcpyDeviceToHost, e->stream));
    LG_CHECK(cudaMemcpyAsync(y, d_y, (size_t)M * m * 4, cudaMemcpyDeviceToHost, e->stream));
    check_err(e);
    free_wmat(W); panel_free(P); panel_free(Py);
    cudaFree(d_act); cudaFree(d_x); cudaFree(d_y); cudaFree(d_out); cudaFree(d_aw); if (d_nw) cudaFree(d_nw);
    return pl.cl ? 1 : 0;
}

// out[tok][m] = W x[tok]  for n <= 256 rows at once through the wide (tcgen05) matmul; x is rounded to f16 first.
// geglu != 0: `blocks`/`blocks_up` are the gate and up matrices [m x k]; out[tok][m] = gelu(gate . x) * (up . x), rounded to f16.
extern "C" int lg_prefill_matmul_host(int type, const void *blocks, const void *blocks_up, int m, int k, const float *x, int n,
                                      float *out) {
    if (n < 1 || n > LG_PF_MAXN || k % 64 || (type != GGML_TYPE_Q4_0 && type != GGML_TYPE_Q4_K)) return -1;
    if (type == GGML_TYPE_Q4_K && k % 256) return -1;
    Engine *e = scratch_engine();
    struct gguf_tensor t, u;
    memset(&t, 0, sizeof t);
    char name[] = "lg_prefill_matmul_host";
    t.name = name; t.n_dims = 2; t.dims[0] = k; t.dims[1] = m; t.dims[2] = t.dims[3] = 1; t.type = type; t.data = (void *)blocks;
    u = t; u.data = (void *)blocks_up;
    const bool geglu = blocks_up != nullptr;
    WMat W = geglu ? build_wmat(e, {&t, &u}, true) : build_wmat(e, {&t});
    float *d_x = dalloc<float>((size_t)n * k);
    __half *d_xh = dalloc<__half>((size_t)LG_PF_MAXN * k);
    float *d_out = dalloc<float>((size_t)n * W.ldo);
    __half *d_act = dalloc<__half>((size_t)n * m);
    LG_CHECK(cudaMemcpyAsync(d_x, x, (size_t)n * k * 4, cudaMemcpyHostToDevice, e->stream));
    launch_k(e, lg_f32_to_f16_rows, dim3((k + 255) / 256, n), dim3(256), 0, (const float *)d_x, k, d_xh, k, k);
    LG_CHECK(cudaGetLastError());
    launch_pf_gemm(e, W, d_xh, LG_PF_MAXN, n, d_out, d_act, m, geglu ? LG_PF_GEGLU : LG_PF_STORE);
    LG_CHECK(cudaGetLastError());
    if (geglu) {
        std::vector<__half> h((size_t)n * m);
        LG_CHECK(cudaMemcpyAsync(h.data(), d_act, h.size() * 2, cudaMemcpyDeviceToHost, e->stream));
        check_err(e);
        for (size_t i = 0; i < h.size(); i++) out[i] = __half2float(h[i]);
    } else {
        std::vector<float> h((size_t)n * W.ldo);
        LG_CHECK(cudaMemcpyAsync(h.data(), d_out, h.size() * 4, cudaMemcpyDeviceToHost, e->stream));
        check_err(e);
        for (int tok = 0; tok < n; tok++)
            for (int r = 0; r < m; r++) out[(size_t)tok * m + r] = h[(size_t)tok * W.ldo + r];
    }
    free_wmat(W); cudaFree(d_x); cudaFree(d_xh); cudaFree(d_out); cudaFree(d_act);
    return 0;
}

static int flash_decode_host_impl(const float *q, const float *k, const float *v, int M, int H, int Hkv, int hd,
                                 int seq, int window, int pos, float *out, int cluster) {
    if (M < 1 || M > LG_MAXM || (hd != 64 && hd != 128 && hd != 256 && hd != 512) || H % Hkv) return -1;
    Engine *e = scratch_engine();
    const int kv_dim = Hkv * hd;
    std::vector<__half> hk((size_t)seq * kv_dim), hv((size_t)seq * kv_dim);
    for (size_t i = 0; i < hk.size(); i++) { hk[i] = __float2half_rn(k[i]); hv[i] = __float2half_rn(v[i]); }
    __half *d_k = dalloc<__half>(hk.size()), *d_v = dalloc<__half>(hv.size());
    float *d_q = dalloc<float>((size_t)M * H * hd), *d_o = dalloc<float>((size_t)M * H * hd);
    int *d_pos = dalloc<int>(1);
    int max_seq = pos + M > seq ? pos + M : seq;
    int slots = tiles_for(window, max_seq, M, hd);
    float *d_part = dalloc<float>((size_t)slots * M * H * hd);
    float2 *d_ml = dalloc<float2>((size_t)slots * M * H);
    LG_CHECK(cudaMemcpyAsync(d_k, hk.data(), hk.size() * 2, cudaMemcpyHostToDevice, e->stream));
    LG_CHECK(cudaMemcpyAsync(d_v, hv.data(), hv.size() * 2, cudaMemcpyHostToDevice, e->stream));
    LG_CHECK(cudaMemcpyAsync(d_q, q, (size_t)M * H * hd * 4, cudaMemcpyHostToDevice, e->stream));
    LG_CHECK(cudaMemcpyAsync(d_pos, &pos, 4, cudaMemcpyHostToDevice, e->stream));
    LgAttnArgs a{};
    a.qkv = d_q; a.ld = 0; a.q_ready = 1; a.has_v = 1; a.owns_kv = 0; a.eps = 0.0f; a.rope = nullptr;
    a.kc = d_k; a.vc = d_v; a.seq = seq; a.kv_dim = kv_dim; a.H = H; a.Hkv = Hkv; a.hd = hd; a.M = M;
    a.n_slots = slots; a.window = window; a.qpos_off = 0; a.win_shrink = 0; a.pos = d_pos;
    a.part = d_part; a.part_ml = d_ml; a.out.q = nullptr; a.out_f32 = d_o; a.err = e->err;
    int rc = 0;
    if (cluster) {
        const int C = attn_cluster_size(e, window, max_seq, seq, hd, H, Hkv);
        if (C) launch_attn_cluster(e, a, C); else rc = -3;         // more tiles than a cluster holds (or no cluster support)
    } else {
        launch_attn(e, a, slots);
    }
    if (!rc) LG_CHECK(cudaMemcpyAsync(out, d_o, (size_t)M * H * hd * 4, cudaMemcpyDeviceToHost, e->stream));
    LG_CHECK(cudaStreamSynchronize(e->stream));
    cudaFree(d_k); cudaFree(d_v); cudaFree(d_q); cudaFree(d_o); cudaFree(d_pos); cudaFree(d_part); cudaFree(d_ml);
    return rc;
}

extern "C" int lg_flash_decode_host(const float *q, const float *k, const float *v, int M, int H, int Hkv, int hd,
                                    int seq, int window, int pos, float *out) {
    return flash_decode_host_impl(q, k, v, M, H, Hkv, hd, seq, window, pos, out, 0);
}
extern "C" int lg_flash_decode_cluster_host(const float *q, const float *k, const float *v, int M, int H, int Hkv, int hd,
                                            int seq, int window, int pos, float *out) {
    return flash_decode_host_impl(q, k, v, M, H, Hkv, hd, seq, window, pos, out, 1);
}
