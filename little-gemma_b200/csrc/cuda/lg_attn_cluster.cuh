// lg_attn_cluster.cuh -- the decode step's attention with the tile merge inside a thread-block cluster.
//
// lg_attn_kernel sends every (query, tile) partial through global memory, takes a ticket, and lets the last CTA of
// a KV head read all partials back and merge them alone: a serial tail of several microseconds per layer.  Here
// the CTAs of one KV head form ONE cluster (one CTA per tile of 128 keys, up to 16 tiles).  A CTA keeps its
// partial (max, sum, accumulators) in its own shared memory; after a cluster barrier every CTA merges a share of
// the output -- one warp per (query, 32 output dims) -- reading the tiles' partials straight out of the peers'
// shared memory (ld.shared::cluster), and writes that share of the o-projection's panel.  No scratch in global
// memory, no atomics, no fence, and the merge is spread over the whole cluster instead of one CTA.
//
// Tile arithmetic (norm + rope of q/k/v, QK^T, softmax, PV) is that of lg_attn_kernel.  Tiles lie on absolute
// position boundaries; the merge walks a query's tiles in ascending order with exact zero weights for tiles
// outside its window, so a row's bits depend on its own position only -- not on the verify width or on the rows
// that share the launch.  Only plain distributed-shared-memory loads are used: no multicast, no remote stores.
#pragma once
#include "lg_kernels.cuh"

#define LG_ATTN_CL_MAX 16            // CTAs per cluster (non-portable size; 8 where 8 tiles are enough)

__device__ __forceinline__ uint32_t dsmem_addr(const void *local_addr, uint32_t rank) {
    uint32_t la = smem_u32(local_addr), ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(la), "r"(rank));
    return ra;
}
__device__ __forceinline__ float dsmem_ld_f32(uint32_t ra) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra) : "memory");
    return v;
}
__device__ __forceinline__ float2 dsmem_ld_f32x2(uint32_t ra) {
    float2 v;
    asm volatile("ld.shared::cluster.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(ra) : "memory");
    return v;
}

// grid (Hkv, C), cluster (1, C, 1): cluster rank r works on tile t_lo + r.
// dynamic smem: Qhi | Qlo [NQ16][HD+8] f16 | K [S][HD+8] (later: the tile's accumulators [NQ16][HD] f32) | V [S][HD+8]
//               | scores [NQ16][S] f32 | Phi | Plo [NQ16][S+8] f16 | ml [NQ16] float2
template <int HD>
__global__ void __launch_bounds__(LG_ATTN_THREADS) lg_attn_cluster_kernel(LgAttnArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ float s_qn[HD], s_kn[HD];
    pdl_launch();
    if (!a.q_ready)
        for (int i = threadIdx.x; i < HD; i += LG_ATTN_THREADS) { s_qn[i] = a.q_norm[i]; s_kn[i] = a.k_norm ? a.k_norm[i] : 1.0f; }
    if (!a.early_kv) pdl_wait();
    constexpr int S = lg_attn_tile(HD), LDH = HD + 8, LDP = S + 8, PER = HD / 64, HALF = HD / 2, NW = LG_ATTN_THREADS / 32;
    const int C = gridDim.y;
    const int kvh = blockIdx.x, gqa = a.H / a.Hkv, nq = gqa * a.M, nq16 = (nq + 15) & ~15;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rank = (int)cluster_rank();
    const int pos0 = *a.pos;
    const int p_first = pos0 + a.qpos_off, p_last = pos0 + a.M - 1 + a.qpos_off;
    const int lo_first = a.window > 0 ? max(0, p_first + a.win_shrink - a.window + 1) : 0;
    const int t_lo = lo_first / S, t_hi = p_last >= 0 ? p_last / S : -1;
    const int T = t_lo + rank;
    const bool live = p_last >= 0 && T <= t_hi;               // this CTA has a tile; the others only help with the merge
    const bool writes_kv = a.owns_kv && !a.q_ready;

    __half *qhi = (__half *)smem, *qlo = qhi + (size_t)nq16 * LDH;
    __half *sk = qlo + (size_t)nq16 * LDH, *sv = sk + (size_t)S * LDH;
    float *sc = (float *)(sv + (size_t)S * LDH);
    __half *phi = (__half *)(sc + (size_t)nq16 * S), *plo = phi + (size_t)nq16 * LDP;
    float2 *ml = (float2 *)(plo + (size_t)nq16 * LDP);
    float *opart = (float *)sk;                               // [nq16][HD] f32, written once the K tile has been consumed

    const int g = lane >> 2, t = lane & 3;
    if (live) {
        // ---- 1. cached K and V rows of the tile start streaming into shared memory at once ----
        constexpr int CH = HD / 8;
        for (int i = threadIdx.x; i < S * CH; i += LG_ATTN_THREADS) {
            const int key = i / CH, c = i % CH, p = T * S + key;
            __half *dk = sk + (size_t)key * LDH + c * 8, *dv = sv + (size_t)key * LDH + c * 8;
            if (p <= p_last && !(writes_kv && p >= pos0)) {
                const size_t off = (size_t)(p % a.seq) * a.kv_dim + (size_t)kvh * HD + c * 8;
                cp_async16(dk, a.kc + off);
                cp_async16(dv, a.vc + off);
            } else if (p > p_last) {
                *(uint4 *)dk = make_uint4(0, 0, 0, 0);
                *(uint4 *)dv = make_uint4(0, 0, 0, 0);
            }
        }
    }
    if (a.early_kv) pdl_wait();

    if (live) {
        // ---- 2. queries: per-head RMSNorm + RoPE, split into f16 hi + lo ----
        for (int qi = warp; qi < nq16; qi += NW) {
            float v0[PER], v1[PER];
            if (qi < nq) {
                const int tok = qi / gqa, hq = kvh * gqa + qi % gqa;
                if (a.q_ready) {
                    const float *src = a.qkv + ((size_t)tok * a.H + hq) * HD;
                    #pragma unroll
                    for (int e = 0; e < PER; e++) { v0[e] = src[lane * PER + e]; v1[e] = src[lane * PER + e + HALF]; }
                } else {
                    head_norm_rope<HD>(a.qkv + (size_t)tok * a.ld + (size_t)hq * HD, s_qn, a.rope + (size_t)tok * HALF, a.eps, lane, v0, v1);
                }
            } else {
                #pragma unroll
                for (int e = 0; e < PER; e++) v0[e] = v1[e] = 0.0f;
            }
            #pragma unroll
            for (int e = 0; e < PER; e++) {
                int i = lane * PER + e;
                __half h0 = __float2half_rn(v0[e]), h1 = __float2half_rn(v1[e]);
                qhi[(size_t)qi * LDH + i] = h0; qhi[(size_t)qi * LDH + i + HALF] = h1;
                qlo[(size_t)qi * LDH + i] = __float2half_rn(v0[e] - __half2float(h0));
                qlo[(size_t)qi * LDH + i + HALF] = __float2half_rn(v1[e] - __half2float(h1));
            }
        }
        if (writes_kv) {
            // rows of the new positions that fall into this tile: K (norm + rope) and V (plain norm), f16 RNE
            for (int j = warp; j < 2 * a.M; j += NW) {
                const int tok = j >> 1, isv = j & 1, p = pos0 + tok;
                if (p / S != T) continue;
                float v0[PER], v1[PER];
                const float *src = a.qkv + (size_t)tok * a.ld + (size_t)(a.H + ((isv && a.has_v) ? a.Hkv : 0) + kvh) * HD;
                head_norm_rope<HD>(src, isv ? nullptr : s_kn, isv ? nullptr : a.rope + (size_t)tok * HALF, a.eps, lane, v0, v1);
                __half *dst = (isv ? a.vc : a.kc) + (size_t)(p % a.seq) * a.kv_dim + (size_t)kvh * HD;
                __half *dsm = (isv ? sv : sk) + (size_t)(p - T * S) * LDH;
                #pragma unroll
                for (int e = 0; e < PER; e++) {
                    const __half h0 = __float2half_rn(v0[e]), h1 = __float2half_rn(v1[e]);
                    dst[lane * PER + e] = h0; dst[lane * PER + e + HALF] = h1;
                    dsm[lane * PER + e] = h0; dsm[lane * PER + e + HALF] = h1;
                }
            }
        }
        cp_async_wait_all();
        __syncthreads();

        // ---- 3. scores: warp w takes keys [w*S/8, (w+1)*S/8) ----
        constexpr int KPW = S / NW, NKT = KPW / 8;
        for (int mt = 0; mt < nq16 / 16; mt++) {
            float c0[NKT][4];
            #pragma unroll
            for (int n = 0; n < NKT; n++) c0[n][0] = c0[n][1] = c0[n][2] = c0[n][3] = 0.0f;
            const __half *qa_hi = qhi + (size_t)(mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDH + (lane >> 4) * 8;
            const __half *qa_lo = qlo + (size_t)(mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDH + (lane >> 4) * 8;
            const __half *kb = sk + (size_t)(warp * KPW + (lane & 7)) * LDH + (lane >> 3) * 8;
            #pragma unroll 2
            for (int k0 = 0; k0 < HD; k0 += 32) {
                uint32_t ah[4], al[4], ah2[4], al2[4];
                ldsm_x4(ah, qa_hi + k0); ldsm_x4(al, qa_lo + k0);
                ldsm_x4(ah2, qa_hi + k0 + 16); ldsm_x4(al2, qa_lo + k0 + 16);
                #pragma unroll
                for (int n = 0; n < NKT; n++) {
                    uint32_t b[4];
                    ldsm_x4(b, kb + (size_t)n * 8 * LDH + k0);
                    mma_f16(c0[n], ah, b[0], b[1]); mma_f16(c0[n], al, b[0], b[1]);
                    mma_f16(c0[n], ah2, b[2], b[3]); mma_f16(c0[n], al2, b[2], b[3]);
                }
            }
            #pragma unroll
            for (int h2 = 0; h2 < 2; h2++) {
                const int qi = mt * 16 + g + h2 * 8;
                const int pj = pos0 + qi / gqa + a.qpos_off;
                const int lo = a.window > 0 ? max(0, pj + a.win_shrink - a.window + 1) : 0;
                #pragma unroll
                for (int n = 0; n < NKT; n++)
                    #pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const int key = warp * KPW + n * 8 + t * 2 + e, p = T * S + key;
                        sc[(size_t)qi * S + key] = (qi < nq && p >= lo && p <= pj) ? c0[n][h2 * 2 + e] : -INFINITY;
                    }
            }
        }
        __syncthreads();

        // ---- 4. per-query softmax over the tile ----
        for (int qi = warp; qi < nq16; qi += NW) {
            float sv_[S / 32], mx = -INFINITY;
            #pragma unroll
            for (int j = 0; j < S / 32; j++) { sv_[j] = sc[(size_t)qi * S + lane + 32 * j]; mx = fmaxf(mx, sv_[j]); }
            mx = warp_max(mx);
            float sum = 0.0f;
            #pragma unroll
            for (int j = 0; j < S / 32; j++) {
                const float e = (sv_[j] == -INFINITY) ? 0.0f : expf(sv_[j] - mx);
                const __half h = __float2half_rn(e);
                phi[(size_t)qi * LDP + lane + 32 * j] = h;
                plo[(size_t)qi * LDP + lane + 32 * j] = __float2half_rn(e - __half2float(h));
                sum += e;
            }
            sum = warp_sum(sum);
            if (lane == 0) ml[qi] = make_float2(mx, sum);
        }
        __syncthreads();

        // ---- 5. O = P V: PVW warps split the head dims; the tile's accumulators go where the K tile was ----
        constexpr int PVW = HD / 16 < NW ? HD / 16 : NW, DW = HD / PVW, NT = DW / 8;
        if (warp < PVW) {
            for (int mt = 0; mt < nq16 / 16; mt++) {
                float o[NT][4];
                #pragma unroll
                for (int n = 0; n < NT; n++) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
                const __half *pa_hi = phi + (size_t)(mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDP + (lane >> 4) * 8;
                const __half *pa_lo = plo + (size_t)(mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDP + (lane >> 4) * 8;
                #pragma unroll
                for (int k0 = 0; k0 < S; k0 += 16) {
                    uint32_t ah[4], al[4];
                    ldsm_x4(ah, pa_hi + k0); ldsm_x4(al, pa_lo + k0);
                    const __half *vb = sv + (size_t)(k0 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDH + warp * DW + (lane >> 4) * 8;
                    #pragma unroll
                    for (int n = 0; n < NT; n += 2) {
                        uint32_t b[4];
                        ldsm_x4_t(b, vb + n * 8);
                        mma_f16(o[n], ah, b[0], b[1]); mma_f16(o[n], al, b[0], b[1]);
                        mma_f16(o[n + 1], ah, b[2], b[3]); mma_f16(o[n + 1], al, b[2], b[3]);
                    }
                }
                #pragma unroll
                for (int h2 = 0; h2 < 2; h2++) {
                    const int qi = mt * 16 + g + h2 * 8;
                    #pragma unroll
                    for (int n = 0; n < NT; n++)
                        *(float2 *)(opart + (size_t)qi * HD + warp * DW + n * 8 + t * 2) = make_float2(o[n][h2 * 2], o[n][h2 * 2 + 1]);
                }
            }
        }
    } else {
        for (int qi = threadIdx.x; qi < nq16; qi += LG_ATTN_THREADS) ml[qi] = make_float2(-INFINITY, 0.0f);
    }

    // ---- 6. every tile's partial is in place: merge across the cluster ----
    cluster_sync_all();
    // one warp per (query, group of 32 output dims), spread over all warps of the cluster
    const int n_items = nq * (HD / 32);
    for (int u = rank * NW + warp; u < n_items; u += C * NW) {
        const int qi = u / (HD / 32), d = (u % (HD / 32)) * 32 + lane;
        const int tok = qi / gqa, hq = kvh * gqa + qi % gqa;
        const int pj = pos0 + tok + a.qpos_off;
        float y = 0.0f;
        if (pj >= 0) {
            const int lo = a.window > 0 ? max(0, pj + a.win_shrink - a.window + 1) : 0;
            const int i0 = lo / S - t_lo, i1 = pj / S - t_lo;            // this query's tiles, as cluster ranks
            // lane i holds tile i's (max, sum) of this query
            float2 v = make_float2(-INFINITY, 0.0f);
            if (lane < C && lane >= i0 && lane <= i1) v = dsmem_ld_f32x2(dsmem_addr(ml + qi, (uint32_t)lane));
            const bool ok = v.y > 0.0f;
            const float mx = warp_max(ok ? v.x : -INFINITY);
            const float w = ok ? expf(v.x - mx) : 0.0f;
            // the tiles' accumulators of this lane's dim: all loads first, then the sums in ascending tile order
            float ov[LG_ATTN_CL_MAX];
            #pragma unroll
            for (int i = 0; i < LG_ATTN_CL_MAX; i++)
                ov[i] = (i < C && i >= i0 && i <= i1) ? dsmem_ld_f32(dsmem_addr(opart + (size_t)qi * HD + d, (uint32_t)i)) : 0.0f;
            float acc = 0.0f, lsum = 0.0f;
            #pragma unroll
            for (int i = 0; i < LG_ATTN_CL_MAX; i++) {
                const float wi = __shfl_sync(0xffffffffu, w, i), li = __shfl_sync(0xffffffffu, v.y, i);
                lsum = fmaf(wi, li, lsum);
                acc = fmaf(wi, ov[i], acc);
            }
            y = lsum > 0.0f ? acc * (1.0f / lsum) : 0.0f;
        }
        if (a.out_f32) a.out_f32[((size_t)tok * a.H + hq) * HD + d] = y;
        if (a.out_h) a.out_h[(size_t)tok * a.ld_h + hq * HD + d] = __float2half_rn(y);
        if (a.out.q) quant_group_store(y, lane, tok, (hq * HD + d) >> 5, a.out);
    }
    // nobody may leave while a peer can still read its shared memory
    cluster_sync_all();
}

inline size_t attn_cluster_smem(int nq, int hd) {
    size_t nq16 = (size_t)((nq + 15) & ~15), ldh = hd + 8, S = lg_attn_tile(hd);
    return 2 * nq16 * ldh * 2 + 2 * S * ldh * 2 + nq16 * S * 4 + 2 * nq16 * (S + 8) * 2 + nq16 * 8 + 64;
}
