// lg_attn_cluster.cuh -- the decode step's attention with the tile merge inside a thread-block cluster.
//
// lg_attn_kernel sends every (query, tile) partial through global memory, takes a ticket, and lets the last CTA of
// a KV head read all partials back and merge them alone: a serial tail of ~9 us per layer.  Here the CTAs of one
// KV head form ONE cluster.  Cluster rank r works on key tiles t_lo + r, t_lo + r + C, ... (one tile per CTA for a
// sliding-window layer; a few for a full-attention layer whose cache is longer than C tiles), keeps the running
// (max, sum, accumulators) of its tiles in registers / shared memory, and after a cluster barrier every CTA merges
// a share of the output -- one warp per (query, 32 output dims) -- reading the partials straight out of the peers'
// shared memory (ld.shared::cluster), and writes that share of the o-projection's panel.  No scratch in global
// memory, no atomics, no fence, and the merge is spread over the whole cluster instead of one CTA.
//
// A tile's K and V rows arrive by tiled TMA copies (cp.async.bulk.tensor.2d over a tensor map of the layer's cache,
// 128-byte swizzle, one elected thread issues HD/64 boxes per matrix): issuing 2 x 128 row copies per CTA one by
// one cost ~8 us, 16-byte cp.async loops ~3 us; the tiled copies cost one instruction per 64 columns.
//
// Bit-stability.  Tiles lie on absolute position boundaries.  A sliding-window layer always has one tile per CTA
// (the host picks C >= the tiles a block can touch), and the merge walks a query's tiles in ascending order with
// exact zero weights outside its window.  A full-attention layer has t_lo = 0, so the tiles a CTA folds together
// (T = r mod C) and their order are fixed by the absolute tile index; a tile past a query's position is an exact
// no-op for that query (weights 0, rescale 1).  So a row's bits depend on its own position only -- not on the
// verify width or on the rows that share the launch.  Only the CTA's own memory and plain loads from the peers'
// shared memory are used.
#pragma once
#include "lg_kernels.cuh"
#include "lg_prefill.cuh"            // tma_load_2d

#define LG_ATTN_CL_MAX 16            // CTAs per cluster (sizes above 8 are "non-portable": the host asks the device first)

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

// Element (row, col) of a K or V tile as the tiled copies leave it: blocks of 64 columns, each [S rows][128 bytes],
// the 16-byte chunk j of row r stored at chunk j ^ (r % 8) (128-byte swizzle; tile base 1024-byte aligned).
template <int S>
__device__ __forceinline__ __half *kv_at(__half *tile, int row, int col) {
    return tile + (col >> 6) * (S * 64) + row * 64 + ((((col & 63) >> 3) ^ (row & 7)) << 3) + (col & 7);
}

// grid (Hkv, C), cluster (1, C, 1).
// dynamic smem (1024-byte aligned): K tile | V tile [HD/64][S][64] f16 swizzled (K later: the CTA's accumulators [NQ16][HD] f32)
//               | Qhi | Qlo [NQ16][HD+8] f16 | scores [NQ16][S] f32 | Phi | Plo [NQ16][S+8] f16 | ml [NQ16] float2 | alpha [NQ16]
//               | new K / V rows [2 LG_MAXM][HD] f16
template <int HD>
__global__ void __launch_bounds__(LG_ATTN_THREADS)
lg_attn_cluster_kernel(const __grid_constant__ CUtensorMap tmk, const __grid_constant__ CUtensorMap tmv, LgAttnArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ float s_qn[HD], s_kn[HD];
    __shared__ __align__(8) uint64_t kv_bar;
    pdl_launch();
    LG_STAMP(a.tag, 0);
    LG_STAMP_KIND(a.tag, 6);
    constexpr int S = lg_attn_tile(HD), LDH = HD + 8, LDP = S + 8, PER = HD / 64, HALF = HD / 2, NW = LG_ATTN_THREADS / 32;
    constexpr uint32_t TILE_BYTES = (uint32_t)S * HD * 2;
    unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int C = gridDim.y;
    const int kvh = blockIdx.x, gqa = a.H / a.Hkv, nq = gqa * a.M, nq16 = (nq + 15) & ~15, nmt = nq16 / 16;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rank = (int)cluster_rank();

    __half *sk = (__half *)smem, *sv = sk + (size_t)S * HD;
    __half *qhi = sv + (size_t)S * HD, *qlo = qhi + (size_t)nq16 * LDH;
    float *sc = (float *)(qlo + (size_t)nq16 * LDH);
    __half *phi = (__half *)(sc + (size_t)nq16 * S), *plo = phi + (size_t)nq16 * LDP;
    float2 *ml = (float2 *)(plo + (size_t)nq16 * LDP);        // running (max, sum) of this CTA's tiles, per query
    float *row_a = (float *)(ml + nq16);
    __half *kvnew = (__half *)(row_a + nq16);                 // [2 LG_MAXM][HD]: the block's own K / V rows (row 2 tok + isv)
    float *opart = (float *)sk;                               // [nq16][HD] f32, written once the last K tile has been consumed

    if (threadIdx.x == 0) mbar_init(&kv_bar, 1);
    if (!a.q_ready)
        for (int i = threadIdx.x; i < HD; i += LG_ATTN_THREADS) { s_qn[i] = a.q_norm[i]; s_kn[i] = a.k_norm ? a.k_norm[i] : 1.0f; }
    for (int qi = threadIdx.x; qi < nq16; qi += LG_ATTN_THREADS) ml[qi] = make_float2(-INFINITY, 0.0f);
    // early_kv: the position and the cached rows below the block were written by earlier graph launches (this layer
    // writes its own rows, and only here), so the first tile may start streaming before the previous kernel has finished
    if (!a.early_kv) { pdl_wait(); if (a.skip && *a.skip) return; }     // called off: the whole cluster leaves before any copy or barrier
    const int pos0 = *a.pos;
    const int p_first = pos0 + a.qpos_off, p_last = pos0 + a.M - 1 + a.qpos_off;
    const int lo_first = a.window > 0 ? max(0, p_first + a.win_shrink - a.window + 1) : 0;
    const int t_lo = lo_first / S, t_hi = p_last >= 0 ? p_last / S : -1;
    const int T_first = t_lo + rank;
    const bool live = T_first <= t_hi;                        // this CTA has at least one tile; the others only help with the merge
    const bool writes_kv = a.owns_kv && !a.q_ready;

    // one elected thread sends a tile's K and V boxes; the copies complete on kv_bar
    auto load_tile = [&](int T) {
        mbar_expect_tx(&kv_bar, 2u * TILE_BYTES);
        const int y = (int)(((long long)T * S) % a.seq);
        #pragma unroll
        for (int c = 0; c < HD / 64; c++) {
            tma_load_2d(sk + (size_t)c * S * 64, &tmk, kvh * HD + c * 64, y, &kv_bar);
            tma_load_2d(sv + (size_t)c * S * 64, &tmv, kvh * HD + c * 64, y, &kv_bar);
        }
    };
    if (live && threadIdx.x == 0) load_tile(T_first);
    if (a.early_kv) pdl_wait();
    LG_STAMP(a.tag, 1);

    const int g = lane >> 2, t = lane & 3;
    // Both products run "transposed": keys (QK^T) or head dims (PV) are the 16-row M side of the tensor-core tile and the
    // queries its 8-column N side, so a block of up to 8 query rows -- the usual case: 4 tokens x 2 heads per KV head --
    // costs one tile column instead of a 16-row tile that is half padding.
    constexpr int KW = S / 16;                                 // warps that hold a 16-key row tile of the scores
    constexpr int PVW = HD / 16 < NW ? HD / 16 : NW, MTW = HD / 16 / PVW;      // warps on PV; 16-dim row tiles per such warp
    const int nq8 = (nq + 7) >> 3;                             // 8-query column tiles (at most 4)
    float o[MTW][4][4];                                        // O^T accumulators [dim tile][query tile][frag], kept across this CTA's tiles
    constexpr bool SPLIT = HD <= 256;                          // the lo half of P accumulates into a second set: two shorter chains
    float o2[SPLIT ? MTW : 1][4][4];
    #pragma unroll
    for (int mt = 0; mt < MTW; mt++)
        #pragma unroll
        for (int n = 0; n < 4; n++) {
            o[mt][n][0] = o[mt][n][1] = o[mt][n][2] = o[mt][n][3] = 0.0f;
            if (SPLIT) o2[mt][n][0] = o2[mt][n][1] = o2[mt][n][2] = o2[mt][n][3] = 0.0f;
        }

    __syncthreads();                                          // the norm weights, ml and the barrier are in place
    if (live) {
        // ---- queries (per-head RMSNorm + RoPE, split into f16 hi + lo) and the block's own K / V rows that fall into
        //      this CTA's tiles.  Every global load of a warp's first query row and of its K / V rows is issued before
        //      the first use, so the prologue holds one memory latency instead of one per row. ----
        auto store_q = [&](int qi, const float (&v0)[PER], const float (&v1)[PER]) {
            #pragma unroll
            for (int e = 0; e < PER; e++) {
                int i = lane * PER + e;
                __half h0 = __float2half_rn(v0[e]), h1 = __float2half_rn(v1[e]);
                qhi[(size_t)qi * LDH + i] = h0; qhi[(size_t)qi * LDH + i + HALF] = h1;
                qlo[(size_t)qi * LDH + i] = __float2half_rn(v0[e] - __half2float(h0));
                qlo[(size_t)qi * LDH + i + HALF] = __float2half_rn(v1[e] - __half2float(h1));
            }
        };
        auto q_src = [&](int qi) {
            const int tok = qi / gqa, hq = kvh * gqa + qi % gqa;
            return a.q_ready ? a.qkv + ((size_t)tok * a.H + hq) * HD : a.qkv + (size_t)tok * a.ld + (size_t)hq * HD;
        };
        float qv0[PER], qv1[PER]; float2 qcs[PER];
        float kv0[2][PER], kv1[2][PER]; float2 kcs[2][PER];
        bool hask[2];
        const bool hasq = warp < nq;
        if (hasq) head_load<HD>(q_src(warp), a.q_ready ? nullptr : a.rope + (size_t)(warp / gqa) * HALF, lane, qv0, qv1, qcs);
        #pragma unroll
        for (int u = 0; u < 2; u++) {
            const int j = warp + u * NW, tok = j >> 1, isv = j & 1, TT = (pos0 + tok) / S;
            hask[u] = writes_kv && j < 2 * a.M && TT >= T_first && TT <= t_hi && (TT - T_first) % C == 0;
            if (hask[u])
                head_load<HD>(a.qkv + (size_t)tok * a.ld + (size_t)(a.H + ((isv && a.has_v) ? a.Hkv : 0) + kvh) * HD,
                              isv ? nullptr : a.rope + (size_t)tok * HALF, lane, kv0[u], kv1[u], kcs[u]);
        }
        if (hasq) {
            if (!a.q_ready) head_finish<HD>(s_qn, true, a.eps, lane, qv0, qv1, qcs);
            store_q(warp, qv0, qv1);
        }
        #pragma unroll
        for (int u = 0; u < 2; u++) {
            if (!hask[u]) continue;
            const int j = warp + u * NW, tok = j >> 1, isv = j & 1, p = pos0 + tok;
            head_finish<HD>(isv ? nullptr : s_kn, !isv, a.eps, lane, kv0[u], kv1[u], kcs[u]);
            __half *dst = (isv ? a.vc : a.kc) + (size_t)(p % a.seq) * a.kv_dim + (size_t)kvh * HD;
            #pragma unroll
            for (int e = 0; e < PER; e++) {
                const __half h0 = __float2half_rn(kv0[u][e]), h1 = __float2half_rn(kv1[u][e]);
                dst[lane * PER + e] = h0; dst[lane * PER + e + HALF] = h1;
                kvnew[(size_t)j * HD + lane * PER + e] = h0; kvnew[(size_t)j * HD + lane * PER + e + HALF] = h1;
            }
        }
        for (int qi = warp + (hasq ? NW : 0); qi < nq16; qi += NW) {
            float v0[PER], v1[PER];
            if (qi < nq) {
                if (a.q_ready) {
                    const float *src = q_src(qi);
                    #pragma unroll
                    for (int e = 0; e < PER; e++) { v0[e] = src[lane * PER + e]; v1[e] = src[lane * PER + e + HALF]; }
                } else {
                    head_norm_rope<HD>(q_src(qi), s_qn, a.rope + (size_t)(qi / gqa) * HALF, a.eps, lane, v0, v1);
                }
            } else {
                #pragma unroll
                for (int e = 0; e < PER; e++) v0[e] = v1[e] = 0.0f;
            }
            store_q(qi, v0, v1);
        }
        LG_STAMP(a.tag, 2);

        uint32_t parity = 0;
        for (int T = T_first; T <= t_hi; T += C) {
            __syncthreads();                                    // first pass: barrier init and Q are visible; later: the previous tile is no longer read
            if (T > T_first && threadIdx.x == 0) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the tile was last touched through ordinary loads and stores
                load_tile(T);
            }
            // the tile has landed (bounded wait)
            if (!mbar_wait(&kv_bar, parity) && a.err && lane == 0) atomicOr(a.err, LG_ERR_MBAR_TIMEOUT);
            parity ^= 1;
            if (writes_kv) {
                // rows of the new positions that fall into this tile go over whatever the copy brought for them (the cache
                // itself was written in the prologue)
                for (int j = warp; j < 2 * a.M; j += NW) {
                    const int tok = j >> 1, isv = j & 1, p = pos0 + tok;
                    if (p / S != T) continue;
                    __half *tile = isv ? sv : sk;
                    const int row = p - T * S;
                    #pragma unroll
                    for (int e = 0; e < PER; e++) {
                        *kv_at<S>(tile, row, lane * PER + e) = kvnew[(size_t)j * HD + lane * PER + e];
                        *kv_at<S>(tile, row, lane * PER + e + HALF) = kvnew[(size_t)j * HD + lane * PER + e + HALF];
                    }
                }
                __syncthreads();
            }
            if (T == T_first) LG_STAMP(a.tag, 3);

            // ---- scores S^T = K Q^T: warp w < KW holds keys [16w, 16w + 16) as the tile's rows, 8 queries per column tile;
            //      keys past a query's position or before its window: -inf ----
            if (warp < KW) {
                // four independent chains per column tile (first / second 16 dims of a step x hi / lo half of q): a chain is
                // HD/32 dependent tensor-core instructions instead of HD/8
                float c0[4][4], c1[4][4], c2[4][4], c3[4][4];
                #pragma unroll
                for (int n = 0; n < 4; n++)
                    #pragma unroll
                    for (int f = 0; f < 4; f++) c0[n][f] = c1[n][f] = c2[n][f] = c3[n][f] = 0.0f;
                const int krow = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, kcol = (lane >> 4) * 8;
                #pragma unroll 2
                for (int k0 = 0; k0 < HD; k0 += 32) {
                    uint32_t ka[4], kb2[4];                    // A operands: 16 keys x dims k0..k0+15 and k0+16..k0+31
                    ldsm_x4(ka, kv_at<S>(sk, krow, k0 + kcol));
                    ldsm_x4(kb2, kv_at<S>(sk, krow, k0 + 16 + kcol));
                    #pragma unroll
                    for (int n = 0; n < 4; n++) {
                        if (n >= nq8) break;
                        uint32_t bh[4], bl[4];                  // B operands: 8 queries x dims k0, +8, +16, +24 (hi and lo halves of q)
                        ldsm_x4(bh, qhi + (size_t)(n * 8 + (lane & 7)) * LDH + k0 + (lane >> 3) * 8);
                        ldsm_x4(bl, qlo + (size_t)(n * 8 + (lane & 7)) * LDH + k0 + (lane >> 3) * 8);
                        mma_f16(c0[n], ka, bh[0], bh[1]); mma_f16(c1[n], ka, bl[0], bl[1]);
                        mma_f16(c2[n], kb2, bh[2], bh[3]); mma_f16(c3[n], kb2, bl[2], bl[3]);
                    }
                }
                #pragma unroll
                for (int n = 0; n < 4; n++)
                    #pragma unroll
                    for (int f = 0; f < 4; f++) c0[n][f] = (c0[n][f] + c2[n][f]) + (c1[n][f] + c3[n][f]);
                #pragma unroll
                for (int n = 0; n < 4; n++) {
                    if (n >= nq8) break;
                    #pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const int qi = n * 8 + t * 2 + e;
                        const int pj = pos0 + qi / gqa + a.qpos_off;
                        const int lo = a.window > 0 ? max(0, pj + a.win_shrink - a.window + 1) : 0;
                        #pragma unroll
                        for (int h2 = 0; h2 < 2; h2++) {
                            const int key = warp * 16 + g + h2 * 8, p = T * S + key;
                            sc[(size_t)qi * S + key] = (qi < nq && p >= lo && p <= pj) ? c0[n][h2 * 2 + e] : -INFINITY;
                        }
                    }
                }
            }
            __syncthreads();
            if (T == T_first) LG_STAMP(a.tag, 8);

            // ---- online softmax, one warp per query row: new running max, the tile's weights against it, the rescale of
            //      what was accumulated before (exactly 1 when the tile adds nothing for this row) ----
            for (int qi = warp; qi < nq8 * 8; qi += NW) {
                float sv_[S / 32], mx = -INFINITY;
                #pragma unroll
                for (int j = 0; j < S / 32; j++) { sv_[j] = sc[(size_t)qi * S + lane + 32 * j]; mx = fmaxf(mx, sv_[j]); }
                const float2 old = ml[qi];
                const float m_new = fmaxf(old.x, warp_max(mx));
                float sum = 0.0f;
                #pragma unroll
                for (int j = 0; j < S / 32; j++) {
                    const float e = (sv_[j] == -INFINITY) ? 0.0f : expf(sv_[j] - m_new);
                    const __half h = __float2half_rn(e);
                    phi[(size_t)qi * LDP + lane + 32 * j] = h;
                    plo[(size_t)qi * LDP + lane + 32 * j] = __float2half_rn(e - __half2float(h));
                    sum += e;
                }
                sum = warp_sum(sum);
                __syncwarp();
                if (lane == 0) {
                    const float alpha = (old.x == m_new) ? 1.0f : expf(old.x - m_new);      // old max -inf < new max: 0
                    row_a[qi] = alpha;
                    ml[qi] = make_float2(m_new, old.y * alpha + sum);
                }
            }
            __syncthreads();
            if (T == T_first) LG_STAMP(a.tag, 9);

            // ---- O^T = alpha O^T + V^T P^T: warp w < PVW holds MTW tiles of 16 head dims as rows, 8 queries per column tile ----
            if (warp < PVW) {
                #pragma unroll
                for (int n = 0; n < 4; n++) {
                    if (n >= nq8) break;
                    const float a0 = row_a[n * 8 + t * 2], a1 = row_a[n * 8 + t * 2 + 1];
                    #pragma unroll
                    for (int mt = 0; mt < MTW; mt++) {
                        o[mt][n][0] *= a0; o[mt][n][1] *= a1; o[mt][n][2] *= a0; o[mt][n][3] *= a1;
                        if (SPLIT) { o2[mt][n][0] *= a0; o2[mt][n][1] *= a1; o2[mt][n][2] *= a0; o2[mt][n][3] *= a1; }
                    }
                }
                #pragma unroll
                for (int k0 = 0; k0 < S; k0 += 32) {
                    uint32_t ph[4][4], pl[4][4];                // B operands: 8 queries x keys k0, +8, +16, +24 (hi and lo halves of P)
                    #pragma unroll
                    for (int n = 0; n < 4; n++) {
                        if (n >= nq8) break;
                        ldsm_x4(ph[n], phi + (size_t)(n * 8 + (lane & 7)) * LDP + k0 + (lane >> 3) * 8);
                        ldsm_x4(pl[n], plo + (size_t)(n * 8 + (lane & 7)) * LDP + k0 + (lane >> 3) * 8);
                    }
                    #pragma unroll
                    for (int mt = 0; mt < MTW; mt++) {
                        const int d0 = (warp * MTW + mt) * 16;
                        uint32_t va[4], vb[4];                  // A operands (transposed loads): 16 dims x keys k0..k0+15, k0+16..k0+31
                        ldsm_x4_t(va, kv_at<S>(sv, k0 + (lane & 7) + (lane >> 4) * 8, d0 + ((lane >> 3) & 1) * 8));
                        ldsm_x4_t(vb, kv_at<S>(sv, k0 + 16 + (lane & 7) + (lane >> 4) * 8, d0 + ((lane >> 3) & 1) * 8));
                        #pragma unroll
                        for (int n = 0; n < 4; n++) {
                            if (n >= nq8) break;
                            mma_f16(o[mt][n], va, ph[n][0], ph[n][1]); mma_f16(SPLIT ? o2[mt][n] : o[mt][n], va, pl[n][0], pl[n][1]);
                            mma_f16(o[mt][n], vb, ph[n][2], ph[n][3]); mma_f16(SPLIT ? o2[mt][n] : o[mt][n], vb, pl[n][2], pl[n][3]);
                        }
                    }
                }
            }
        }
        // ---- this CTA's accumulators go where the K tile was (every warp is past its last use of K) ----
        __syncthreads();
        LG_STAMP(a.tag, 10);
        if (warp < PVW) {
            #pragma unroll
            for (int mt = 0; mt < MTW; mt++) {
                const int d0 = (warp * MTW + mt) * 16;
                #pragma unroll
                for (int n = 0; n < 4; n++) {
                    if (n >= nq8) break;
                    #pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const int qi = n * 8 + t * 2 + e;
                        opart[(size_t)qi * HD + d0 + g] = SPLIT ? o[mt][n][e] + o2[mt][n][e] : o[mt][n][e];
                        opart[(size_t)qi * HD + d0 + g + 8] = SPLIT ? o[mt][n][2 + e] + o2[mt][n][2 + e] : o[mt][n][2 + e];
                    }
                }
            }
        }
    }

    // ---- every CTA's partial is in place: merge across the cluster ----
    LG_STAMP(a.tag, 4);
    cluster_sync_all();
    LG_STAMP(a.tag, 5);
    // one warp per (query, group of 32 output dims), spread over all warps of the cluster; rank i holds the query's
    // tiles t_lo + i, t_lo + i + C, ...: weights are exact zeros for ranks without a tile of this query
    const int n_items = nq * (HD / 32);
    for (int u = rank * NW + warp; u < n_items; u += C * NW) {
        const int qi = u / (HD / 32), d = (u % (HD / 32)) * 32 + lane;
        const int tok = qi / gqa, hq = kvh * gqa + qi % gqa;
        const int pj = pos0 + tok + a.qpos_off;
        float y = 0.0f;
        if (pj >= 0) {
            const int lo = a.window > 0 ? max(0, pj + a.win_shrink - a.window + 1) : 0;
            const int i0 = lo / S - t_lo, i1 = min(pj / S - t_lo, i0 + C - 1);      // ranks that hold tiles of this query
            // every remote load of this item -- the ranks' (max, sum) pairs and their accumulators of this lane's dim --
            // is issued before the first use; the sums then run in ascending rank order
            float2 v = make_float2(-INFINITY, 0.0f);
            if (lane < C && lane >= i0 && lane <= i1) v = dsmem_ld_f32x2(dsmem_addr(ml + qi, (uint32_t)lane));
            float ov[LG_ATTN_CL_MAX];
            #pragma unroll
            for (int i = 0; i < LG_ATTN_CL_MAX; i++)
                ov[i] = (i < C && i >= i0 && i <= i1) ? dsmem_ld_f32(dsmem_addr(opart + (size_t)qi * HD + d, (uint32_t)i)) : 0.0f;
            const bool ok = v.y > 0.0f;
            const float mx = warp_max(ok ? v.x : -INFINITY);
            const float w = ok ? expf(v.x - mx) : 0.0f;
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
    LG_STAMP(a.tag, 6);
    cluster_sync_all();
    LG_STAMP(a.tag, 7);
}

inline size_t attn_cluster_smem(int nq, int hd) {
    size_t nq16 = (size_t)((nq + 15) & ~15), ldh = hd + 8, S = lg_attn_tile(hd);
    return 1024 + 2 * S * hd * 2 + 2 * nq16 * ldh * 2 + nq16 * S * 4 + 2 * nq16 * (S + 8) * 2 + nq16 * 12 + 64 + (size_t)2 * LG_MAXM * hd * 2;
}
