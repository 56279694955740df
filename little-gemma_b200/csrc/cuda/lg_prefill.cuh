// lg_prefill.cuh -- the wide (prompt) matmul on the 5th-generation tensor cores.
//
// out[tok][row] = sum_k W[row][k] * X[tok][k] for a block of up to 256 prompt tokens at once.
// W is the same tile-major q4 matrix the decode step streams (16 rows x 64 columns per 512-byte
// tile, nibbles stored as two's-complement q-8); X is an f16 row-major activation block.  The
// weights are expanded to f16 on the fly -- d*(q-8) rounded once to f16, i.e. the f16 rounding of
// the exact dequantised value -- so each weight byte leaves HBM once per token block and the
// multiply-accumulate runs as tcgen05.mma (kind::f16, f32 accumulate in tensor memory).
//
// One CTA owns 128 weight rows (8 row tiles = the 128 TMEM lanes) x NT tokens (TMEM columns) and
// walks k in blocks of 64 (one tile position = one 128-byte swizzle row of f16):
//   warp 8 (one thread)  streams the raw q4 tiles + scales of two k blocks per stage with bulk copies;
//   warp 9 (one thread)  loads the X block [NT tokens x 64] with a tiled TMA copy (128-byte swizzle);
//   warps 0-7            expand a raw k block to the f16 A operand [128 rows x 64] (one row tile per
//                        warp) in the same swizzled K-major layout, then fence it to the async proxy;
//   warp 10 (one thread) issues four tcgen05.mma (M=128, N=NT, K=16) per k block and commits the
//                        stage back to the producers; after the last block it commits the accumulator;
//   warps 0-7            read the accumulator with tcgen05.ld (lane quarter = warp % 4, column half =
//                        warp / 4) and store f32 rows, or apply GeGLU on interleaved gate/up rows and
//                        store the f16 input of the down projection.
// blockIdx.z cuts k into slices whose partial sums go to separate planes of `out` (matrices with
// few rows would otherwise fill a fraction of the SMs); the consumer adds the planes.
// Every mbarrier wait is bounded; a timeout raises LG_ERR_MBAR_TIMEOUT, the CTA stops waiting,
// drains its own copies, frees its tensor memory and returns.
#pragma once
#include <cuda.h>
#include "lg_kernels.cuh"

#define LG_PF_BM 128
#define LG_PF_BK 64
#define LG_PF_A_STAGES 4        // expanded weight (A operand) stages: a multiple of LG_PF_GROUPS, so a stage belongs to ONE
                                // expand group and its empty-barrier phases are observed in order by the same threads
                                // (a parity wait cannot tell "two completions behind" from "done")
#define LG_PF_SMEM_MAX 232448   // 227 KB: the most dynamic shared memory a CTA can have
#define LG_PF_DQ_WARPS 8
#define LG_PF_GROUPS 4          // expand-warp groups working on different k blocks
#define LG_PF_THREADS ((LG_PF_DQ_WARPS + 3) * 32)
#define LG_PF_MAXN 256

enum { LG_PF_STORE = 0, LG_PF_GEGLU = 1 };

struct LgPfGemmArgs {
    const uint4 *wq; const uint2 *ws; const uint2 *wd;
    int nkp, n_row_tiles;
    int n_tok;                  // valid tokens of the block (columns beyond are computed and dropped)
    float *out; int ldo;        // STORE: out[slice][tok][ldo], slice = blockIdx.z
    size_t part_stride;         // floats between the planes of two k slices
    int n_rows;                 // rows >= n_rows are padding and are not stored
    __half *act; int ld_act;    // GEGLU: act[tok][ld_act], element j = gelu(gate_j) * up_j
    int *err;
};

// raw stage: 8 row tiles x 2 tile positions of nibbles, then their scales, then (q4_K) their {d,dmin}
template <int FMT> __host__ __device__ constexpr int pf_raw_stage_bytes() {
    return 8 * 2 * (512 + 64 + (FMT == LG_FMT_Q4_K ? 64 : 0));
}
template <int NT> __host__ __device__ constexpr int pf_a_stages() { return LG_PF_A_STAGES; }
// activation (B operand) stages (3 stages with a deeper raw ring measured slower at a 256-wide token tile)
template <int NT> __host__ __device__ constexpr int pf_b_stages() { return 4; }
// raw q4 stages of two k blocks each: as many as fit beside the operand stages, at most 8 -- the bytes in flight
// from HBM per SM, which is what keeps the weight stream moving
template <int NT, int FMT> __host__ __device__ constexpr int pf_raw_stages() {
    int left = LG_PF_SMEM_MAX - 1024 - 512 - pf_a_stages<NT>() * LG_PF_BM * 128 - pf_b_stages<NT>() * NT * 128;
    int n = left / pf_raw_stage_bytes<FMT>();
    return n > 8 ? 8 : n;
}
template <int NT, int FMT> __host__ __device__ constexpr size_t pf_smem_bytes() {
    return 1024 + (size_t)pf_a_stages<NT>() * LG_PF_BM * 128 + (size_t)pf_b_stages<NT>() * NT * 128
         + (size_t)pf_raw_stages<NT, FMT>() * pf_raw_stage_bytes<FMT>() + 512;
}

// mbar_wait on a shared-space address that is already in a register
__device__ __forceinline__ bool mbar_wait_u32(uint32_t bar, uint32_t parity) {
    for (int it = 0; it < LG_SPIN_LIMIT; ++it) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 :: "r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
// K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc_k128(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// two stored nibbles (bytes b0,b1 of `n`, already q = stored ^ 8) -> half2 (q0-8, q1-8) * d
__device__ __forceinline__ uint32_t pf_pair_q4_0(uint32_t n, uint32_t sel, __half2 d2) {
    uint32_t v;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(v) : "r"(n), "r"(0x64646464u), "r"(sel));        // (1024+q0, 1024+q1)
    __half2 h = __hsub2(*(__half2 *)&v, __half2half2(__ushort_as_half((unsigned short)0x6408)));   // - 1032
    h = __hmul2(h, d2);
    return *(uint32_t *)&h;
}
// q4_K: d*sc*q - dmin*m with the two products rounded to f16 first
__device__ __forceinline__ uint32_t pf_pair_q4_K(uint32_t n, uint32_t sel, __half2 dsc2, __half2 negdm2) {
    uint32_t v;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(v) : "r"(n), "r"(0x64646464u), "r"(sel));
    __half2 h = __hsub2(*(__half2 *)&v, __half2half2(__ushort_as_half((unsigned short)0x6400)));   // - 1024 = q
    h = __hfma2(h, dsc2, negdm2);
    return *(uint32_t *)&h;
}

template <int NT, int FMT, int EPI>
__global__ void __launch_bounds__(LG_PF_THREADS) lg_pf_gemm_kernel(const __grid_constant__ CUtensorMap tmx, LgPfGemmArgs a) {
    extern __shared__ unsigned char pf_smem_raw[];
    constexpr int STA = pf_a_stages<NT>(), STB = pf_b_stages<NT>(), RS = pf_raw_stages<NT, FMT>(), RAW = pf_raw_stage_bytes<FMT>();
    constexpr int A_BYTES = LG_PF_BM * 128, B_BYTES = NT * 128;
    constexpr int RAW_SC = 16 * 512, RAW_DD = RAW_SC + 16 * 64;
    unsigned char *base = (unsigned char *)(((uintptr_t)pf_smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char *sA = base, *sB = sA + STA * A_BYTES, *sRaw = sB + STB * B_BYTES;
    uint64_t *bars = (uint64_t *)(sRaw + RS * RAW);
    static_assert(STA == STB, "an operand stage is one A tile and one B tile behind the same pair of barriers");
    // full[s]: the expand group's arrivals + the activation copy's bytes; empty[s]: one commit frees both tiles
    uint64_t *raw_full = bars, *raw_empty = raw_full + RS, *full = raw_empty + RS, *empty = full + STA, *acc_full = empty + STA;
    uint32_t *tmem_slot = (uint32_t *)(acc_full + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rt0 = blockIdx.x * 8, tok0 = blockIdx.y * NT;
    const int kb_lo = (int)((long long)a.nkp * blockIdx.z / gridDim.z), kb_hi = (int)((long long)a.nkp * (blockIdx.z + 1) / gridDim.z);
    const int nkb = kb_hi - kb_lo, n_raw = (nkb + 1) >> 1;     // this CTA's k blocks: kb_lo + [0, nkb)
    constexpr int DQT = LG_PF_DQ_WARPS * 32;

    pdl_launch();
    if (threadIdx.x == 0) {
        for (int i = 0; i < RS; i++) { mbar_init(raw_full + i, 1); mbar_init(raw_empty + i, 2 * DQT / LG_PF_GROUPS); }
        for (int i = 0; i < STA; i++) { mbar_init(full + i, DQT / LG_PF_GROUPS + 1); mbar_init(empty + i, 1); }
        mbar_init(acc_full, 1);
    }
    if (warp == LG_PF_DQ_WARPS + 2) {        // tensor memory: NT f32 columns x 128 lanes
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(tmem_slot)), "r"(NT) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    if (warp == LG_PF_DQ_WARPS) {
        // ---------------- raw weight producer ----------------
        if (lane == 0) {
            bool ok = true;
            int issued = 0;
            for (int r = 0; r < n_raw && ok; r++) {
                const int rs = r % RS;
                if (r >= RS && !mbar_wait(raw_empty + rs, ((r / RS) & 1) ^ 1)) { atomicOr(a.err, LG_ERR_MBAR_TIMEOUT | 2); ok = false; break; }
                const int np = min(2, nkb - 2 * r);
                unsigned char *st = sRaw + rs * RAW;
                mbar_expect_tx(raw_full + rs, 8u * np * (512 + 64 + (FMT == LG_FMT_Q4_K ? 64 : 0)));
                #pragma unroll
                for (int ti = 0; ti < 8; ti++) {
                    const int rt = min(rt0 + ti, a.n_row_tiles - 1);
                    const size_t tile = (size_t)rt * a.nkp + kb_lo + 2 * r;
                    bulk_g2s(st + ti * 1024, a.wq + tile * 32, np * 512, raw_full + rs);
                    bulk_g2s(st + RAW_SC + ti * 128, a.ws + tile * 8, np * 64, raw_full + rs);
                    if (FMT == LG_FMT_Q4_K) bulk_g2s(st + RAW_DD + ti * 128, a.wd + tile * 8, np * 64, raw_full + rs);
                }
                issued = r + 1;
            }
            if (!ok)      // drain: the copies already issued must land before the CTA's shared memory is released
                for (int r = max(0, issued - RS); r < issued; r++) mbar_wait(raw_full + r % RS, (r / RS) & 1);
        }
    } else if (warp == LG_PF_DQ_WARPS + 1) {
        // ---------------- activation producer ----------------
        if (lane == 0) {
            pdl_wait();
            bool ok = true;
            int issued = 0;
            for (int kb = 0; kb < nkb && ok; kb++) {
                const int s = kb % STB;
                if (kb >= STB && !mbar_wait(empty + s, ((kb / STB) & 1) ^ 1)) { atomicOr(a.err, LG_ERR_MBAR_TIMEOUT | 4); ok = false; break; }
                mbar_expect_tx(full + s, B_BYTES);
                tma_load_2d(sB + s * B_BYTES, &tmx, (kb_lo + kb) * LG_PF_BK, tok0, full + s);
                issued = kb + 1;
            }
            if (!ok)
                for (int kb = max(0, issued - STB); kb < issued; kb++) mbar_wait(full + kb % STB, (kb / STB) & 1);
        }
    } else if (warp == LG_PF_DQ_WARPS + 2) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(LG_PF_BM >> 4) << 24);
            // This one thread is the pipeline's pacemaker: everything it does per k block is a serial chain of dependent
            // instructions, so the loop is unrolled over the stages (static stage index: descriptors and barrier
            // addresses live in registers) and carries as little arithmetic as possible.
            uint64_t adesc[STA], bdesc[STB];
            uint32_t ufull[STA], uempty[STA];
            #pragma unroll
            for (int st = 0; st < STA; st++) {
                adesc[st] = umma_desc_k128(smem_u32(sA + st * A_BYTES)); bdesc[st] = umma_desc_k128(smem_u32(sB + st * B_BYTES));
                ufull[st] = smem_u32(full + st); uempty[st] = smem_u32(empty + st);
            }
            bool ok = true;
            uint32_t ph = 0, acc = 0;
            for (int kb0 = 0; kb0 < nkb && ok; kb0 += STA, ph ^= 1) {
                #pragma unroll
                for (int st = 0; st < STA; st++) {
                    if (kb0 + st >= nkb || !ok) break;
                    if (!mbar_wait_u32(ufull[st], ph)) { atomicOr(a.err, LG_ERR_MBAR_TIMEOUT | 8); ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    #pragma unroll
                    for (int j = 0; j < LG_PF_BK / 16; j++) { umma_f16(tmem, adesc[st] + 2 * j, bdesc[st] + 2 * j, idesc, acc); acc = 1u; }
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(uempty[st]) : "memory");
                }
            }
            umma_commit(acc_full);                   // arrives when every MMA above has completed
        }
    } else {
        // ---------------- expand q4 -> f16 A operand (one row tile per warp), then the epilogue ----------------
        // The expand warps form LG_PF_GROUPS groups; group gi takes the k blocks kb = gi (mod LG_PF_GROUPS), so
        // several k blocks are being expanded at once and a group's latency chain (wait, expand, proxy fence,
        // arrive) overlaps the other groups'.  Within a group the warps split the 8 row tiles.
        // All shared-memory traffic of this loop uses explicit shared-space addresses (32-bit).
        constexpr int NG = LG_PF_GROUPS, WPG = LG_PF_DQ_WARPS / NG, TPW = 8 / WPG;   // warps per group, tiles per warp
        static_assert(STA % NG == 0, "a stage must belong to one expand group");
        const int g = lane >> 2, t = lane & 3;
        const int gi = warp / WPG, wi = warp % WPG;
        const uint32_t raw0 = smem_u32(sRaw) + lane * 16;
        const uint32_t rsc0 = smem_u32(sRaw) + RAW_SC + g * 8, rdd0 = smem_u32(sRaw) + RAW_DD + g * 8;
        // row ti*16 + g (+8): 8-row group (2 ti) (+1), row-in-group g; 16-byte chunk c of a row sits at c ^ g
        const uint32_t dst0 = smem_u32(sA) + g * 128 + (t & 1) * 8;
        uint32_t coff[4];                                                            // [sub-block][low / high nibbles]
        #pragma unroll
        for (int i = 0; i < 4; i++) coff[i] = (uint32_t)(((4 * (i >> 1) + (t >> 1) + 2 * (i & 1)) ^ g) << 4);
        bool ok = true;
        for (int kb = gi; kb < nkb; kb += NG) {
            const int s = kb % STA, r = kb >> 1, rs = r % RS, half = kb & 1;
            if (ok && !mbar_wait(raw_full + rs, (r / RS) & 1)) { ok = false; atomicOr(a.err, 32); }
            if (ok && kb >= STA && !mbar_wait(empty + s, ((kb / STA) & 1) ^ 1)) { ok = false; atomicOr(a.err, 64); }
            if (!ok) break;
            #pragma unroll
            for (int q = 0; q < TPW; q++) {
                const int ti = wi * TPW + q;                                         // row tile of the CTA's 8
                const uint32_t roff = rs * RAW + ti * 1024 + half * 512, soff = rs * RAW + ti * 128 + half * 64;
                uint4 w; uint2 sc, dd = make_uint2(0, 0);
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w) : "r"(raw0 + roff));
                asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(sc.x), "=r"(sc.y) : "r"(rsc0 + soff));
                if (FMT == LG_FMT_Q4_K) asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(dd.x), "=r"(dd.y) : "r"(rdd0 + soff));
                const uint32_t dstS = dst0 + s * A_BYTES + (2 * ti) * 1024;
                #pragma unroll
                for (int sbk = 0; sbk < 2; sbk++)
                    #pragma unroll
                    for (int h8 = 0; h8 < 2; h8++) {
                        const uint32_t word = sbk ? (h8 ? w.w : w.z) : (h8 ? w.y : w.x);
                        const uint32_t sw = sbk ? sc.y : sc.x;
                        const uint32_t lo = (word & 0x0F0F0F0Fu) ^ 0x08080808u, hi = ((word >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;
                        uint2 vlo, vhi;
                        if (FMT == LG_FMT_Q4_0) {
                            uint32_t dbits;                                           // the row's scale in both halves
                            asm("prmt.b32 %0, %1, %1, %2;" : "=r"(dbits) : "r"(sw), "r"(h8 ? 0x3232u : 0x1010u));
                            const __half2 d2 = *(const __half2 *)&dbits;
                            vlo = make_uint2(pf_pair_q4_0(lo, 0x4140u, d2), pf_pair_q4_0(lo, 0x4342u, d2));
                            vhi = make_uint2(pf_pair_q4_0(hi, 0x4140u, d2), pf_pair_q4_0(hi, 0x4342u, d2));
                        } else {
                            const uint32_t sm = h8 ? (sw >> 16) : (sw & 0xffff);
                            const float2 dm = __half22float2(*(const __half2 *)(h8 ? &dd.y : &dd.x));
                            const __half2 dsc2 = __float2half2_rn(dm.x * (float)(sm & 0xff));
                            const __half2 ndm2 = __float2half2_rn(-dm.y * (float)(sm >> 8));
                            vlo = make_uint2(pf_pair_q4_K(lo, 0x4140u, dsc2, ndm2), pf_pair_q4_K(lo, 0x4342u, dsc2, ndm2));
                            vhi = make_uint2(pf_pair_q4_K(hi, 0x4140u, dsc2, ndm2), pf_pair_q4_K(hi, 0x4342u, dsc2, ndm2));
                        }
                        const uint32_t rowa = dstS + h8 * 1024;
                        asm volatile("st.shared.v2.u32 [%0], {%1,%2};" :: "r"(rowa + coff[2 * sbk]), "r"(vlo.x), "r"(vlo.y) : "memory");
                        asm volatile("st.shared.v2.u32 [%0], {%1,%2};" :: "r"(rowa + coff[2 * sbk + 1]), "r"(vhi.x), "r"(vhi.y) : "memory");
                    }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");           // generic-proxy stores -> visible to the MMA
            mbar_arrive(full + s);
            mbar_arrive(raw_empty + rs);           // every expand thread arrives once per k block it takes
        }
        if (!ok && lane == 0) atomicOr(a.err, LG_ERR_MBAR_TIMEOUT);

        // ---------------- epilogue: lane l of warp w holds accumulator row 32 (w % 4) + l ----------------
        if (ok) { ok = mbar_wait(acc_full, 0); if (!ok) atomicOr(a.err, 128); }
        if (!ok && lane == 0) atomicOr(a.err, LG_ERR_MBAR_TIMEOUT);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            const int lq = warp & 3, ch = warp >> 2;                     // TMEM lane quarter, column half
            const int lrow = lq * 32 + lane;                            // row within the CTA's 128
            const int rt = rt0 + (lrow >> 4);
            float *outp = a.out + (size_t)blockIdx.z * a.part_stride;
            for (int c0 = ch * (NT / 2); c0 < (ch + 1) * (NT / 2); c0 += 32) {
                if (tok0 + c0 >= a.n_tok) break;                          // uniform per CTA
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)(lq * 32) << 16) + c0, v);
                if (EPI == LG_PF_STORE) {
                    const int row = rt0 * 16 + lrow;
                    if (rt < a.n_row_tiles && row < a.n_rows) {
                        #pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (tok0 + c0 + j < a.n_tok) outp[(size_t)(tok0 + c0 + j) * a.ldo + row] = __uint_as_float(v[j]);
                    }
                } else {
                    // tile rows 0-7 are gate rows, rows 8-15 the matching up rows: lane l pairs with lane l+8
                    const int r16 = lrow & 15;
                    #pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const float mine = __uint_as_float(v[j]);
                        const float other = __shfl_xor_sync(0xffffffffu, mine, 8);
                        if (r16 < 8 && rt < a.n_row_tiles && tok0 + c0 + j < a.n_tok) {
                            const float y = __fmul_rn(gelu_tanh(mine), other);
                            a.act[(size_t)(tok0 + c0 + j) * a.ld_act + rt * 8 + r16] = __float2half_rn(y);
                        }
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (warp == LG_PF_DQ_WARPS + 2) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(NT) : "memory");
    }
}

// y = gelu_tanh(gate) * up as f16 rows (per-layer-embedding gate of a prompt block)
__global__ void lg_pf_geglu_rows(const float *__restrict__ gate, const float *__restrict__ up, int ld_g, int ld_u, int n,
                                 __half *__restrict__ out, int ld_out) {
    pdl_launch(); pdl_wait();
    const int tok = blockIdx.y;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        out[(size_t)tok * ld_out + i] = __float2half_rn(__fmul_rn(gelu_tanh(gate[(size_t)tok * ld_g + i]), up[(size_t)tok * ld_u + i]));
}

// Media positions of a prompt block: x[tok] = rows[ridx[tok]] where ridx[tok] >= 0 (the row replaces the token embedding as it is)
__global__ void lg_inject_rows(float *__restrict__ x, int ldx, const float *__restrict__ rows, const int *__restrict__ ridx, int n) {
    pdl_launch(); pdl_wait();
    const int tok = blockIdx.x, r = ridx[tok];
    if (r < 0) return;
    for (int i = threadIdx.x; i < n; i += blockDim.x) x[(size_t)tok * ldx + i] = rows[(size_t)r * n + i];
}

// f32 rows -> f16 rows (the B operand of the wide matmul)
__global__ void lg_f32_to_f16_rows(const float *__restrict__ src, int ld_src, __half *__restrict__ dst, int ld_dst, int n) {
    pdl_launch(); pdl_wait();
    const int tok = blockIdx.y;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        dst[(size_t)tok * ld_dst + i] = __float2half_rn(src[(size_t)tok * ld_src + i]);
}

// ---------------------------------------------------------------------------------------------
// attention of a prompt block: all query rows of the block in one launch per layer
// ---------------------------------------------------------------------------------------------
// Step 1 (lg_pf_qkv_prep_kernel): per token, per-head RMSNorm + NeoX RoPE of the raw projection
// rows.  Queries go to an f16 hi + lo pair [tok][H][hd]; K (norm + rope) and V (plain norm) rows go
// to the f16 cache of the owning layer (round to nearest even) at row (pos % seq).  The cache ring
// of a sliding-window layer has more spare rows than a block has tokens, so writing the whole block
// first does not overwrite a row an earlier query of the block still attends to.
struct LgPfPrepArgs {
    const float *qkv; int ld;            // [n][ld] = [q (H*hd) | k (Hkv*hd) | v (Hkv*hd)], the sum of n_parts planes
    int n_parts; size_t part_stride;
    int has_v, owns_kv;
    const float *q_norm, *k_norm; float eps;
    const float2 *rope;                  // [n][hd/2]
    __half *kc, *vc; int seq, kv_dim;
    int H, Hkv;
    const int *pos;                      // position of the block's first token
    __half *q_hi, *q_lo;                 // [n][H][hd]
};

template <int HD>
__global__ void __launch_bounds__(256) lg_pf_qkv_prep_kernel(LgPfPrepArgs a) {
    __shared__ float s_qn[HD], s_kn[HD];
    __shared__ float s_row[8][HD];       // a warp's head vector with the k-slice planes added
    pdl_launch();
    for (int i = threadIdx.x; i < HD; i += 256) { s_qn[i] = a.q_norm[i]; s_kn[i] = a.k_norm ? a.k_norm[i] : 1.0f; }
    pdl_wait();
    __syncthreads();
    constexpr int PER = HD / 64, HALF = HD / 2;
    const int tok = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int p = *a.pos + tok;
    const int jobs = a.H + (a.owns_kv ? 2 * a.Hkv : 0);
    const float2 *rope = a.rope + (size_t)tok * HALF;
    for (int j = blockIdx.y * 8 + warp; j < jobs; j += 8 * gridDim.y) {     // one head vector per warp
        float v0[PER], v1[PER];
        const int jj = j - a.H, isv = jj >= a.Hkv, kvh = isv ? jj - a.Hkv : jj;
        const float *src = a.qkv + (size_t)tok * a.ld
                         + (size_t)(j < a.H ? j : a.H + ((isv && a.has_v) ? a.Hkv : 0) + kvh) * HD;
        if (a.n_parts > 1) {
            __syncwarp();
            for (int i = lane; i < HD; i += 32) {
                float v = src[i];
                for (int p = 1; p < a.n_parts; p++) v += src[(size_t)p * a.part_stride + i];
                s_row[warp][i] = v;
            }
            __syncwarp();
            src = s_row[warp];
        }
        if (j < a.H) {
            head_norm_rope<HD>(src, s_qn, rope, a.eps, lane, v0, v1);
            __half *dh = a.q_hi + ((size_t)tok * a.H + j) * HD, *dl = a.q_lo + ((size_t)tok * a.H + j) * HD;
            #pragma unroll
            for (int e = 0; e < PER; e++) {
                const int i = lane * PER + e;
                const __half h0 = __float2half_rn(v0[e]), h1 = __float2half_rn(v1[e]);
                dh[i] = h0; dh[i + HALF] = h1;
                dl[i] = __float2half_rn(v0[e] - __half2float(h0)); dl[i + HALF] = __float2half_rn(v1[e] - __half2float(h1));
            }
        } else {
            head_norm_rope<HD>(src, isv ? nullptr : s_kn, isv ? nullptr : rope, a.eps, lane, v0, v1);
            __half *dst = (isv ? a.vc : a.kc) + (size_t)(p % a.seq) * a.kv_dim + (size_t)kvh * HD;
            #pragma unroll
            for (int e = 0; e < PER; e++) {
                dst[lane * PER + e] = __float2half_rn(v0[e]);
                dst[lane * PER + e + HALF] = __float2half_rn(v1[e]);
            }
        }
    }
}

// Step 2 (lg_pf_attn_kernel): one CTA = one KV head x LG_PFA_Q query rows (LG_PFA_Q / gqa consecutive
// tokens x the gqa query heads of that KV head).  It walks the keys of its causal / sliding window
// in tiles of 64 with an online softmax: S = Q K^T and O += P V on mma.sync.m16n8k16 (f16 operands,
// f32 accumulate), Q and P as f16 hi + lo pairs like the decode kernel, scale 1.0.  The normalised
// rows are written as f16 -- the o-projection's input.
struct LgPfAttnArgs {
    const __half *q_hi, *q_lo;           // [n][H][hd]
    const __half *kc, *vc; int seq, kv_dim;
    int H, Hkv, n;
    int window;                          // <= 0: full causal
    const int *pos;
    __half *out; int ld_out;             // [n][ld_out], head hq at column hq*hd
};
#define LG_PFA_Q 32
#define LG_PFA_S 64

template <int HD>
__global__ void __launch_bounds__(256) lg_pf_attn_kernel(LgPfAttnArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int NQ = LG_PFA_Q, S = LG_PFA_S, LDH = HD + 8, LDP = S + 8, LDS = S + 4;
    __half *qhi = (__half *)smem, *qlo = qhi + NQ * LDH;
    __half *sk = qlo + NQ * LDH;                              // two buffers of [K tile | V tile], each [S][LDH]
    float *sc = (float *)(sk + 4 * S * LDH);                  // [NQ][LDS]
    __half *phi = (__half *)(sc + NQ * LDS), *plo = phi + NQ * LDP;
    float *row_m = (float *)(plo + NQ * LDP), *row_l = row_m + NQ, *row_a = row_l + NQ;
    pdl_launch(); pdl_wait();

    const int kvh = blockIdx.x, gqa = a.H / a.Hkv, qb = NQ / gqa;           // qb tokens per CTA
    const int t0 = blockIdx.y * qb;
    if (t0 >= a.n) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int pos0 = *a.pos;
    const int nt = min(qb, a.n - t0);                                       // valid tokens of this CTA
    const int p_first = pos0 + t0, p_last = pos0 + t0 + nt - 1;
    const int lo_first = a.window > 0 ? max(0, p_first - a.window + 1) : 0;

    // queries: row r = (token r / gqa, head kvh*gqa + r % gqa)
    constexpr int CH = HD / 8;
    for (int i = threadIdx.x; i < NQ * CH; i += 256) {
        const int r = i / CH, c = i % CH, tok = t0 + r / gqa, hq = kvh * gqa + r % gqa;
        uint4 vh = make_uint4(0, 0, 0, 0), vl = vh;
        if (r / gqa < nt) {
            vh = *(const uint4 *)(a.q_hi + ((size_t)tok * a.H + hq) * HD + c * 8);
            vl = *(const uint4 *)(a.q_lo + ((size_t)tok * a.H + hq) * HD + c * 8);
        }
        *(uint4 *)(qhi + (size_t)r * LDH + c * 8) = vh;
        *(uint4 *)(qlo + (size_t)r * LDH + c * 8) = vl;
    }
    for (int r = threadIdx.x; r < NQ; r += 256) { row_m[r] = -INFINITY; row_l[r] = 0.0f; }

    // warp roles: m-tile mt (16 query rows) x slice hf of the tile's keys (scores) or of the head dims (output)
    constexpr int MT = NQ / 16, WK = 8 / MT, KPW = S / WK, NKT = KPW / 8;
    const int mt = warp % MT, hf = warp / MT;
    constexpr int DW = HD / WK, NT = DW / 8;                   // output dims per warp, 8-wide n tiles
    static_assert(NT % 2 == 0 && NKT >= 1, "tile split");
    float o[NT][4];
    #pragma unroll
    for (int n2 = 0; n2 < NT; n2++) o[n2][0] = o[n2][1] = o[n2][2] = o[n2][3] = 0.0f;

    // K/V tiles are double-buffered: tile i+1 streams in (cp.async) while tile i is being used
    auto load_tile = [&](int k0, int buf) {
        __half *bk = sk + (size_t)buf * 2 * S * LDH, *bv = bk + S * LDH;
        for (int i = threadIdx.x; i < S * CH; i += 256) {
            const int key = i / CH, c = i % CH, p = k0 + key;
            __half *dk = bk + (size_t)key * LDH + c * 8, *dv = bv + (size_t)key * LDH + c * 8;
            if (p <= p_last) {
                const size_t off = (size_t)(p % a.seq) * a.kv_dim + (size_t)kvh * HD + c * 8;
                cp_async16(dk, a.kc + off);
                cp_async16(dv, a.vc + off);
            } else {
                *(uint4 *)dk = make_uint4(0, 0, 0, 0);
                *(uint4 *)dv = make_uint4(0, 0, 0, 0);
            }
        }
    };
    const int k_first = (lo_first / S) * S;
    load_tile(k_first, 0);
    int buf = 0;
    for (int k0 = k_first; k0 <= p_last; k0 += S, buf ^= 1) {
        cp_async_wait_all();
        __syncthreads();                                        // tile k0 has landed; the other buffer and P are no longer read
        if (k0 + S <= p_last) load_tile(k0 + S, buf ^ 1);
        const __half *sk_t = sk + (size_t)buf * 2 * S * LDH, *sv_t = sk_t + S * LDH;

        // ---- scores of 16 rows x KPW keys per warp ----
        {
            float c0[NKT][4];
            #pragma unroll
            for (int n2 = 0; n2 < NKT; n2++) c0[n2][0] = c0[n2][1] = c0[n2][2] = c0[n2][3] = 0.0f;
            const __half *qa_hi = qhi + (size_t)(mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDH + (lane >> 4) * 8;
            const __half *qa_lo = qlo + (size_t)(mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDH + (lane >> 4) * 8;
            const __half *kb = sk_t + (size_t)(hf * KPW + (lane & 7)) * LDH + (lane >> 3) * 8;
            #pragma unroll 2
            for (int d0 = 0; d0 < HD; d0 += 32) {
                uint32_t ah[4], al[4], ah2[4], al2[4];
                ldsm_x4(ah, qa_hi + d0); ldsm_x4(al, qa_lo + d0);
                ldsm_x4(ah2, qa_hi + d0 + 16); ldsm_x4(al2, qa_lo + d0 + 16);
                #pragma unroll
                for (int n2 = 0; n2 < NKT; n2++) {
                    uint32_t b[4];
                    ldsm_x4(b, kb + (size_t)n2 * 8 * LDH + d0);
                    mma_f16(c0[n2], ah, b[0], b[1]); mma_f16(c0[n2], al, b[0], b[1]);
                    mma_f16(c0[n2], ah2, b[2], b[3]); mma_f16(c0[n2], al2, b[2], b[3]);
                }
            }
            #pragma unroll
            for (int h2 = 0; h2 < 2; h2++) {
                const int r = mt * 16 + g + h2 * 8;
                const int pj = pos0 + t0 + r / gqa;
                const int lo = a.window > 0 ? max(0, pj - a.window + 1) : 0;
                const bool rv = r / gqa < nt;
                #pragma unroll
                for (int n2 = 0; n2 < NKT; n2++)
                    #pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const int key = hf * KPW + n2 * 8 + t * 2 + e, p = k0 + key;
                        sc[r * LDS + key] = (rv && p >= lo && p <= pj) ? c0[n2][h2 * 2 + e] : -INFINITY;
                    }
            }
        }
        __syncthreads();

        // ---- online softmax: warp w owns NQ/8 consecutive rows ----
        for (int r = warp * (NQ / 8); r < (warp + 1) * (NQ / 8); r++) {
            const float s0 = sc[r * LDS + lane], s1 = sc[r * LDS + lane + 32];
            const float m_old = row_m[r];
            const float m_new = fmaxf(m_old, warp_max(fmaxf(s0, s1)));
            const float e0 = s0 == -INFINITY ? 0.0f : expf(s0 - m_new), e1 = s1 == -INFINITY ? 0.0f : expf(s1 - m_new);
            const __half h0 = __float2half_rn(e0), h1 = __float2half_rn(e1);
            phi[r * LDP + lane] = h0; phi[r * LDP + lane + 32] = h1;
            plo[r * LDP + lane] = __float2half_rn(e0 - __half2float(h0));
            plo[r * LDP + lane + 32] = __float2half_rn(e1 - __half2float(h1));
            const float sum = warp_sum(e0 + e1);
            if (lane == 0) {
                const float alpha = m_old == -INFINITY ? 0.0f : expf(m_old - m_new);     // m_new == -inf: nothing seen yet
                row_a[r] = alpha;
                row_l[r] = row_l[r] * alpha + sum;
                row_m[r] = m_new;
            }
        }
        __syncthreads();

        // ---- O = alpha O + P V: 16 rows x DW dims per warp ----
        {
            const float a0 = row_a[mt * 16 + g], a1 = row_a[mt * 16 + g + 8];
            #pragma unroll
            for (int n2 = 0; n2 < NT; n2++) { o[n2][0] *= a0; o[n2][1] *= a0; o[n2][2] *= a1; o[n2][3] *= a1; }
            const __half *pa_hi = phi + (size_t)(mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDP + (lane >> 4) * 8;
            const __half *pa_lo = plo + (size_t)(mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDP + (lane >> 4) * 8;
            #pragma unroll
            for (int kk = 0; kk < S; kk += 16) {
                uint32_t ah[4], al[4];
                ldsm_x4(ah, pa_hi + kk); ldsm_x4(al, pa_lo + kk);
                const __half *vb = sv_t + (size_t)(kk + (lane & 7) + ((lane >> 3) & 1) * 8) * LDH + hf * DW + (lane >> 4) * 8;
                #pragma unroll
                for (int n2 = 0; n2 < NT; n2 += 2) {
                    uint32_t b[4];
                    ldsm_x4_t(b, vb + n2 * 8);
                    mma_f16(o[n2], ah, b[0], b[1]); mma_f16(o[n2], al, b[0], b[1]);
                    mma_f16(o[n2 + 1], ah, b[2], b[3]); mma_f16(o[n2 + 1], al, b[2], b[3]);
                }
            }
        }
    }
    __syncthreads();
    #pragma unroll
    for (int h2 = 0; h2 < 2; h2++) {
        const int r = mt * 16 + g + h2 * 8;
        if (r / gqa < nt) {
            const float l = row_l[r], inv = l > 0.0f ? 1.0f / l : 0.0f;
            __half *dst = a.out + (size_t)(t0 + r / gqa) * a.ld_out + (size_t)(kvh * gqa + r % gqa) * HD + hf * DW;
            #pragma unroll
            for (int n2 = 0; n2 < NT; n2++)
                *(__half2 *)(dst + n2 * 8 + t * 2) = __floats2half2_rn(o[n2][h2 * 2] * inv, o[n2][h2 * 2 + 1] * inv);
        }
    }
}

template <int HD> constexpr size_t pf_attn_smem() {
    return (size_t)2 * LG_PFA_Q * (HD + 8) * 2 + (size_t)4 * LG_PFA_S * (HD + 8) * 2 + (size_t)LG_PFA_Q * (LG_PFA_S + 4) * 4
         + (size_t)2 * LG_PFA_Q * (LG_PFA_S + 8) * 2 + 3 * LG_PFA_Q * 4;
}
