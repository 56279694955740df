// lg_attn_deep.cuh -- split-KV flash-decode for full-attention layers of long-context sessions.
//
// The decode step's attention kernel (lg_attn_kernel) gives every tile of 128 keys its own CTA and
// lets the last CTA of a KV head merge all tiles: right at a few thousand keys, but at 32K keys that
// is 257 one-tile CTAs per head, one per SM at a time with its load and its math back to back, and a
// 2 MB merge by a single CTA.  Here a CTA walks a SPAN of G consecutive tiles of 64 keys with an
// online softmax (running max / sum per query, accumulators in registers), two CTAs fit an SM so one
// CTA's tile load overlaps the other's math, and the merge runs over spans, G times fewer partials.
//
// Spans, like tiles, lie on ABSOLUTE position boundaries (span s = keys [s*G*64, (s+1)*G*64)), G is a
// property of the session (the cache length), and a tile that is wholly outside a query's window is an
// exact no-op for that query (weights 0, rescale 1).  So a query row's result depends on its own
// position only -- not on the verify width or on which other rows share the launch -- which keeps the
// speculative stream byte-identical to plain decoding.
#pragma once
#include "lg_kernels.cuh"

#define LG_DEEP_S 64

// dynamic smem: Qhi | Qlo [NQ16][HD+8] f16 | K [64][HD+8] | V [64][HD+8] | scores 2 x [NQ16][64] f32 | Phi | Plo [NQ16][72] f16 | m, l, alpha [NQ16][3]
template <int HD, int MTM>      // MTM = 16-row query blocks the CTA carries accumulators for (>= nq16 / 16)
__global__ void __launch_bounds__(LG_ATTN_THREADS) lg_attn_deep_kernel(LgAttnArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ float s_qn[HD], s_kn[HD];
    pdl_launch();
    LG_STAMP_KIND(a.tag, 5);
    if (!a.q_ready)
        for (int i = threadIdx.x; i < HD; i += LG_ATTN_THREADS) { s_qn[i] = a.q_norm[i]; s_kn[i] = a.k_norm ? a.k_norm[i] : 1.0f; }
    if (!a.early_kv) pdl_wait();
    constexpr int S = LG_DEEP_S, LDH = HD + 8, LDP = S + 8, PER = HD / 64, HALF = HD / 2, NW = LG_ATTN_THREADS / 32;
    const int G = a.G;
    const int kvh = blockIdx.x, gqa = a.H / a.Hkv, nq = gqa * a.M, nq16 = (nq + 15) & ~15, nmt = nq16 / 16;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos0 = *a.pos;
    const int p_first = pos0 + a.qpos_off, p_last = pos0 + a.M - 1 + a.qpos_off;
    if (p_last < 0) return;
    const int lo_first = a.window > 0 ? max(0, p_first + a.win_shrink - a.window + 1) : 0;
    const int t_lo = lo_first / S, t_hi = p_last / S;
    const int s_lo = t_lo / G, s_hi = t_hi / G;                 // spans the block touches
    const int SP = s_lo + blockIdx.y;
    if (SP > s_hi) return;
    const int slot = SP % a.n_slots;
    const int T0 = max(SP * G, t_lo), T1 = min(SP * G + G - 1, t_hi);
    const bool writes_kv = a.owns_kv && !a.q_ready;

    __half *qhi = (__half *)smem, *qlo = qhi + (size_t)nq16 * LDH;
    __half *sk = qlo + (size_t)nq16 * LDH, *sv = sk + (size_t)S * LDH;
    float *sc = (float *)(sv + (size_t)S * LDH), *sc2 = sc + (size_t)nq16 * S;    // scores: lower / upper half of the head dims
    __half *phi = (__half *)(sc2 + (size_t)nq16 * S), *plo = phi + (size_t)nq16 * LDP;
    float *row_m = (float *)(plo + (size_t)nq16 * LDP), *row_l = row_m + nq16, *row_a = row_l + nq16;

    constexpr int CH = HD / 8;
    auto load_tile = [&](int T) {
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
    };
    load_tile(T0);
    if (a.early_kv) pdl_wait();

    // queries: per-head RMSNorm + RoPE, split into f16 hi + lo
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
    for (int r = threadIdx.x; r < nq16; r += LG_ATTN_THREADS) { row_m[r] = -INFINITY; row_l[r] = 0.0f; row_a[r] = 1.0f; }
    // rows past the last query only pad the 16-row tiles: their probabilities stay zero, the softmax skips them
    for (int i = threadIdx.x; i < (nq16 - nq) * LDP; i += LG_ATTN_THREADS) {
        phi[(size_t)nq * LDP + i] = __float2half_rn(0.0f); plo[(size_t)nq * LDP + i] = __float2half_rn(0.0f);
    }

    const int g = lane >> 2, t = lane & 3;
    // Both products run "transposed": keys (scores) or head dims (P V) are the 16-row side of the tensor-core tile and
    // the queries its 8-column side, so a block of up to 8 query rows costs one column tile, not a half-empty 16-row tile.
    constexpr int MTW = HD / 16 / NW;                            // 16-dim row tiles of O^T per warp
    static_assert(S == 64 && NW == 8 && HD % (16 * NW) == 0, "four 16-key row tiles x two halves of the head dims over eight warps");
    const int nq8 = (nq + 7) >> 3;                               // 8-query column tiles (at most 4)
    float o[MTW][4][4];                                          // O^T accumulators [dim tile][query tile][frag], kept across the span's tiles
    #pragma unroll
    for (int mt = 0; mt < MTW; mt++)
        #pragma unroll
        for (int n = 0; n < 4; n++) o[mt][n][0] = o[mt][n][1] = o[mt][n][2] = o[mt][n][3] = 0.0f;

    for (int T = T0; T <= T1; T++) {
        if (T > T0) {
            __syncthreads();                                     // the previous tile's K, V and P are no longer read
            if (T == T0 + 2) LG_STAMP(a.tag, 0);
            load_tile(T);
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
        if (T == T0 + 2) LG_STAMP(a.tag, 1);

        // scores S^T = K Q^T: warp w holds keys [16 (w & 3), +16) as the tile's rows and half (w >> 2) of the head dims,
        // 8 queries per column tile; the two halves land in two buffers the softmax adds
        {
            float c0[4][4], c1[4][4];
            #pragma unroll
            for (int n = 0; n < 4; n++)
                #pragma unroll
                for (int f = 0; f < 4; f++) c0[n][f] = c1[n][f] = 0.0f;
            const int kt = warp & 3, dh = warp >> 2;
            const __half *ka_p = sk + (size_t)(kt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDH + dh * (HD / 2) + (lane >> 4) * 8;
            #pragma unroll 2
            for (int k0 = 0; k0 < HD / 2; k0 += 16) {
                uint32_t ka[4];                                  // A operand: 16 keys x 16 dims
                ldsm_x4(ka, ka_p + k0);
                #pragma unroll
                for (int n = 0; n < 4; n++) {
                    if (n >= nq8) break;
                    uint32_t bq[4];                              // B operands: 8 queries x 16 dims, hi (bq[0..1]) and lo (bq[2..3])
                    const __half *qp = ((lane >> 4) ? qlo : qhi) + (size_t)(n * 8 + (lane & 7)) * LDH + dh * (HD / 2) + k0 + ((lane >> 3) & 1) * 8;
                    ldsm_x4(bq, qp);
                    mma_f16(c0[n], ka, bq[0], bq[1]); mma_f16(c1[n], ka, bq[2], bq[3]);
                }
            }
            float *dst = dh ? sc2 : sc;
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
                        const int key = kt * 16 + g + h2 * 8, p = T * S + key;
                        const float v = c0[n][h2 * 2 + e] + c1[n][h2 * 2 + e];
                        dst[(size_t)qi * S + key] = (dh || (qi < nq && p >= lo && p <= pj)) ? v : -INFINITY;
                    }
                }
            }
        }
        __syncthreads();
        if (T == T0 + 2) LG_STAMP(a.tag, 2);

        // online softmax, one warp per query row: new running max, the tile's weights against it, the rescale
        // of what was accumulated before (exactly 1 when the tile adds nothing for this row)
        for (int qi = warp; qi < nq; qi += NW) {
            const float s0 = sc[(size_t)qi * S + lane] + sc2[(size_t)qi * S + lane], s1 = sc[(size_t)qi * S + lane + 32] + sc2[(size_t)qi * S + lane + 32];
            const float m_old = row_m[qi];
            const float m_new = fmaxf(m_old, warp_max(fmaxf(s0, s1)));
            const float e0 = s0 == -INFINITY ? 0.0f : expf(s0 - m_new), e1 = s1 == -INFINITY ? 0.0f : expf(s1 - m_new);
            const __half h0 = __float2half_rn(e0), h1 = __float2half_rn(e1);
            phi[(size_t)qi * LDP + lane] = h0; phi[(size_t)qi * LDP + lane + 32] = h1;
            plo[(size_t)qi * LDP + lane] = __float2half_rn(e0 - __half2float(h0));
            plo[(size_t)qi * LDP + lane + 32] = __float2half_rn(e1 - __half2float(h1));
            const float sum = warp_sum(e0 + e1);
            if (lane == 0) {
                const float alpha = (m_old == m_new) ? 1.0f : expf(m_old - m_new);     // m_old = -inf < m_new: 0
                row_a[qi] = alpha;
                row_l[qi] = row_l[qi] * alpha + sum;
                row_m[qi] = m_new;
            }
        }
        __syncthreads();
        if (T == T0 + 2) LG_STAMP(a.tag, 3);

        // O^T = alpha O^T + V^T P^T: warp w holds MTW tiles of 16 head dims as rows, 8 queries per column tile
        {
            #pragma unroll
            for (int n = 0; n < 4; n++) {
                if (n >= nq8) break;
                const float a0 = row_a[n * 8 + t * 2], a1 = row_a[n * 8 + t * 2 + 1];
                #pragma unroll
                for (int mt = 0; mt < MTW; mt++) { o[mt][n][0] *= a0; o[mt][n][1] *= a1; o[mt][n][2] *= a0; o[mt][n][3] *= a1; }
            }
            #pragma unroll
            for (int k0 = 0; k0 < S; k0 += 32) {
                uint32_t ph[4][4], pl[4][4];                    // B operands: 8 queries x keys k0, +8, +16, +24 (hi and lo halves of P)
                #pragma unroll
                for (int n = 0; n < 4; n++) {
                    if (n >= nq8) break;
                    ldsm_x4(ph[n], phi + (size_t)(n * 8 + (lane & 7)) * LDP + k0 + (lane >> 3) * 8);
                    ldsm_x4(pl[n], plo + (size_t)(n * 8 + (lane & 7)) * LDP + k0 + (lane >> 3) * 8);
                }
                #pragma unroll
                for (int mt = 0; mt < MTW; mt++) {
                    const int d0 = (warp * MTW + mt) * 16;
                    uint32_t va[4], vb[4];                      // A operands (transposed loads): 16 dims x keys k0..k0+15, k0+16..k0+31
                    ldsm_x4_t(va, sv + (size_t)(k0 + (lane & 7) + (lane >> 4) * 8) * LDH + d0 + ((lane >> 3) & 1) * 8);
                    ldsm_x4_t(vb, sv + (size_t)(k0 + 16 + (lane & 7) + (lane >> 4) * 8) * LDH + d0 + ((lane >> 3) & 1) * 8);
                    #pragma unroll
                    for (int n = 0; n < 4; n++) {
                        if (n >= nq8) break;
                        mma_f16(o[mt][n], va, ph[n][0], ph[n][1]); mma_f16(o[mt][n], va, pl[n][0], pl[n][1]);
                        mma_f16(o[mt][n], vb, ph[n][2], ph[n][3]); mma_f16(o[mt][n], vb, pl[n][2], pl[n][3]);
                    }
                }
            }
        }
        if (T == T0 + 2) LG_STAMP(a.tag, 4);
    }

    // the span's partial (max, sum, accumulators) of every query row
    #pragma unroll
    for (int n = 0; n < 4; n++) {
        if (n >= nq8) break;
        #pragma unroll
        for (int e = 0; e < 2; e++) {
            const int qi = n * 8 + t * 2 + e;
            if (qi >= nq) continue;
            const int tok = qi / gqa, hq = kvh * gqa + qi % gqa;
            float *pp = a.part + (((size_t)slot * a.M + tok) * a.H + hq) * HD;
            #pragma unroll
            for (int mt = 0; mt < MTW; mt++) {
                const int d0 = (warp * MTW + mt) * 16;
                pp[d0 + g] = o[mt][n][e];
                pp[d0 + g + 8] = o[mt][n][2 + e];
            }
            if (warp == 0 && g == 0) a.part_ml[((size_t)slot * a.M + tok) * a.H + hq] = make_float2(row_m[qi], row_l[qi]);
        }
    }

    // the last CTA of this KV head merges the spans
    __shared__ int s_last;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        s_last = atomicAdd(a.tickets + kvh, 1) == s_hi - s_lo;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const int ns_all = s_hi - s_lo + 1;
    float2 *mls = (float2 *)sk;                               // [nq][ns_all]: (max, sum) then (weight, -); the K/V area is free now
    float *invl = row_l;                                      // [nq]
    for (int i = threadIdx.x; i < nq * ns_all; i += LG_ATTN_THREADS) {
        const int qi = i / ns_all, S2 = s_lo + i % ns_all;
        const int tok = qi / gqa, hq = kvh * gqa + qi % gqa;
        mls[i] = __ldcg(a.part_ml + ((size_t)(S2 % a.n_slots) * a.M + tok) * a.H + hq);
    }
    __syncthreads();
    for (int qi = warp; qi < nq; qi += NW) {
        const int pj = pos0 + qi / gqa + a.qpos_off;
        const int lo = a.window > 0 ? max(0, pj + a.win_shrink - a.window + 1) : 0;
        const int i0 = pj >= 0 ? (lo / S) / G - s_lo : 0, i1 = pj >= 0 ? (pj / S) / G - s_lo : -1;
        float mx = -INFINITY;
        for (int i = i0 + lane; i <= i1; i += 32) { float2 v = mls[qi * ns_all + i]; if (v.y > 0.0f) mx = fmaxf(mx, v.x); }
        mx = warp_max(mx);
        // a span always lands in lane (absolute span index % 32): the order of this sum is the same wherever the block's
        // first span lies (spans outside the query's window add exact zeros)
        float lsum = 0.0f;
        for (int S2 = (s_lo & ~31) + lane; S2 <= s_hi; S2 += 32) {
            if (S2 < s_lo) continue;
            const int i = S2 - s_lo;
            float2 v = mls[qi * ns_all + i];
            float w = (i >= i0 && i <= i1 && v.y > 0.0f) ? expf(v.x - mx) : 0.0f;
            mls[qi * ns_all + i].x = w;
            lsum += w * v.y;
        }
        lsum = warp_sum(lsum);
        if (lane == 0) invl[qi] = lsum > 0.0f ? 1.0f / lsum : 0.0f;
    }
    __syncthreads();
    float *ybuf = (float *)qhi;                                // [nq][HD] f32 (the query area is free now)
    const size_t slot_stride = (size_t)a.M * a.H * HD;
    for (int u = threadIdx.x; u < nq * (HD / 4); u += LG_ATTN_THREADS) {
        const int qi = u / (HD / 4), d4 = (u % (HD / 4)) * 4;
        const float *base = a.part + ((size_t)(qi / gqa) * a.H + kvh * gqa + qi % gqa) * HD + d4;
        const float2 *wq = mls + (size_t)qi * ns_all;
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int i = 0; i < ns_all; i += 8) {                  // ascending span order, 8 loads in flight
            float4 v[8];
            #pragma unroll
            for (int j = 0; j < 8; j++)
                if (i + j < ns_all) v[j] = __ldcg((const float4 *)(base + (size_t)((s_lo + i + j) % a.n_slots) * slot_stride));
            #pragma unroll
            for (int j = 0; j < 8; j++)
                if (i + j < ns_all) {
                    const float w = wq[i + j].x;
                    acc.x = fmaf(w, v[j].x, acc.x); acc.y = fmaf(w, v[j].y, acc.y);
                    acc.z = fmaf(w, v[j].z, acc.z); acc.w = fmaf(w, v[j].w, acc.w);
                }
        }
        const float il = invl[qi];
        *(float4 *)(ybuf + (size_t)qi * HD + d4) = make_float4(acc.x * il, acc.y * il, acc.z * il, acc.w * il);
    }
    __syncthreads();
    for (int u = warp; u < nq * (HD / 32); u += NW) {
        const int qi = u / (HD / 32), d = (u % (HD / 32)) * 32 + lane;
        const int tok = qi / gqa, hq = kvh * gqa + qi % gqa;
        const float y = ybuf[(size_t)qi * HD + d];
        if (a.out_f32) a.out_f32[((size_t)tok * a.H + hq) * HD + d] = y;
        if (a.out_h) a.out_h[(size_t)tok * a.ld_h + hq * HD + d] = __float2half_rn(y);
        if (a.out.q) quant_group_store(y, lane, tok, (hq * HD + d) >> 5, a.out);
    }
    if (threadIdx.x == 0) a.tickets[kvh] = 0;
}

inline size_t attn_deep_smem(int nq, int hd) {
    size_t nq16 = (size_t)((nq + 15) & ~15), ldh = hd + 8, S = LG_DEEP_S;
    return 2 * nq16 * ldh * 2 + 2 * S * ldh * 2 + 2 * nq16 * S * 4 + 2 * nq16 * (S + 8) * 2 + nq16 * 12 + 64;
}
