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
//   warp 4 (one thread)  streams the raw q4 tiles + scales of two k blocks per stage with bulk copies;
//   warp 5 (one thread)  loads the X block [NT tokens x 64] with a tiled TMA copy (128-byte swizzle);
//   warps 0-3            expand a raw k block to the f16 A operand [128 rows x 64] in the same
//                        swizzled K-major layout, then fence it to the async proxy;
//   warp 6 (one thread)  issues four tcgen05.mma (M=128, N=NT, K=16) per k block and commits the
//                        stage back to the producers; after the last block it commits the accumulator;
//   warps 0-3            read the accumulator with tcgen05.ld and store f32 rows, or apply GeGLU on
//                        interleaved gate/up rows and store the f16 input of the down projection.
// Every mbarrier wait is bounded; a timeout raises LG_ERR_MBAR_TIMEOUT, the CTA stops waiting,
// drains its own copies, frees its tensor memory and returns.
#pragma once
#include <cuda.h>
#include "lg_kernels.cuh"

#define LG_PF_BM 128
#define LG_PF_BK 64
#define LG_PF_STAGES 4          // A / B operand stages
#define LG_PF_RAW_STAGES 3      // raw q4 stages of two k blocks each
#define LG_PF_THREADS 224
#define LG_PF_MAXN 256

enum { LG_PF_STORE = 0, LG_PF_GEGLU = 1 };

struct LgPfGemmArgs {
    const uint4 *wq; const uint2 *ws; const uint2 *wd;
    int nkp, n_row_tiles;
    int n_tok;                  // valid tokens of the block (columns beyond are computed and dropped)
    float *out; int ldo;        // STORE: out[tok][ldo]
    int n_rows;                 // rows >= n_rows are padding and are not stored
    __half *act; int ld_act;    // GEGLU: act[tok][ld_act], element j = gelu(gate_j) * up_j
    int *err;
};

// raw stage: 8 row tiles x 2 tile positions of nibbles, then their scales, then (q4_K) their {d,dmin}
template <int FMT> __host__ __device__ constexpr int pf_raw_stage_bytes() {
    return 8 * 2 * (512 + 64 + (FMT == LG_FMT_Q4_K ? 64 : 0));
}
template <int NT, int FMT> __host__ __device__ constexpr size_t pf_smem_bytes() {
    return 1024 + (size_t)LG_PF_STAGES * (LG_PF_BM * 128 + NT * 128) + (size_t)LG_PF_RAW_STAGES * pf_raw_stage_bytes<FMT>() + 256;
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
    constexpr int ST = LG_PF_STAGES, RS = LG_PF_RAW_STAGES, RAW = pf_raw_stage_bytes<FMT>();
    constexpr int A_BYTES = LG_PF_BM * 128, B_BYTES = NT * 128;
    constexpr int RAW_SC = 16 * 512, RAW_DD = RAW_SC + 16 * 64;
    unsigned char *base = (unsigned char *)(((uintptr_t)pf_smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char *sA = base, *sB = sA + ST * A_BYTES, *sRaw = sB + ST * B_BYTES;
    uint64_t *bars = (uint64_t *)(sRaw + RS * RAW);
    uint64_t *raw_full = bars, *raw_empty = raw_full + RS, *a_full = raw_empty + RS, *b_full = a_full + ST,
             *empty = b_full + ST, *acc_full = empty + ST;
    uint32_t *tmem_slot = (uint32_t *)(acc_full + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rt0 = blockIdx.x * 8, tok0 = blockIdx.y * NT;
    const int nkb = a.nkp, n_raw = (nkb + 1) >> 1;

    pdl_launch();
    if (threadIdx.x == 0) {
        for (int i = 0; i < RS; i++) { mbar_init(raw_full + i, 1); mbar_init(raw_empty + i, 128); }
        for (int i = 0; i < ST; i++) { mbar_init(a_full + i, 128); mbar_init(b_full + i, 1); mbar_init(empty + i, 1); }
        mbar_init(acc_full, 1);
    }
    if (warp == 6) {                         // tensor memory: NT f32 columns x 128 lanes
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(tmem_slot)), "r"(NT) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    if (warp == 4) {
        // ---------------- raw weight producer ----------------
        if (lane == 0) {
            bool ok = true;
            int issued = 0;
            for (int r = 0; r < n_raw && ok; r++) {
                const int rs = r % RS;
                if (r >= RS && !mbar_wait(raw_empty + rs, ((r / RS) & 1) ^ 1)) { atomicOr(a.err, LG_ERR_MBAR_TIMEOUT); ok = false; break; }
                const int np = min(2, nkb - 2 * r);
                unsigned char *st = sRaw + rs * RAW;
                mbar_expect_tx(raw_full + rs, 8u * np * (512 + 64 + (FMT == LG_FMT_Q4_K ? 64 : 0)));
                #pragma unroll
                for (int ti = 0; ti < 8; ti++) {
                    const int rt = min(rt0 + ti, a.n_row_tiles - 1);
                    const size_t tile = (size_t)rt * a.nkp + 2 * r;
                    bulk_g2s(st + ti * 1024, a.wq + tile * 32, np * 512, raw_full + rs);
                    bulk_g2s(st + RAW_SC + ti * 128, a.ws + tile * 8, np * 64, raw_full + rs);
                    if (FMT == LG_FMT_Q4_K) bulk_g2s(st + RAW_DD + ti * 128, a.wd + tile * 8, np * 64, raw_full + rs);
                }
                issued = r + 1;
            }
            if (!ok)      // drain: the copies already issued must land before the CTA's shared memory is released
                for (int r = max(0, issued - RS); r < issued; r++) mbar_wait(raw_full + r % RS, (r / RS) & 1);
        }
    } else if (warp == 5) {
        // ---------------- activation producer ----------------
        if (lane == 0) {
            pdl_wait();
            bool ok = true;
            int issued = 0;
            for (int kb = 0; kb < nkb && ok; kb++) {
                const int s = kb % ST;
                if (kb >= ST && !mbar_wait(empty + s, ((kb / ST) & 1) ^ 1)) { atomicOr(a.err, LG_ERR_MBAR_TIMEOUT); ok = false; break; }
                mbar_expect_tx(b_full + s, B_BYTES);
                tma_load_2d(sB + s * B_BYTES, &tmx, kb * LG_PF_BK, tok0, b_full + s);
                issued = kb + 1;
            }
            if (!ok)
                for (int kb = max(0, issued - ST); kb < issued; kb++) mbar_wait(b_full + kb % ST, (kb / ST) & 1);
        }
    } else if (warp == 6) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(LG_PF_BM >> 4) << 24);
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; kb++) {
                const int s = kb % ST; const uint32_t ph = (kb / ST) & 1;
                if (!mbar_wait(a_full + s, ph) || !mbar_wait(b_full + s, ph)) { atomicOr(a.err, LG_ERR_MBAR_TIMEOUT); ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t ad = umma_desc_k128(smem_u32(sA + s * A_BYTES)), bd = umma_desc_k128(smem_u32(sB + s * B_BYTES));
                #pragma unroll
                for (int j = 0; j < LG_PF_BK / 16; j++)
                    umma_f16(tmem, ad + 2 * j, bd + 2 * j, idesc, (kb | j) ? 1u : 0u);
                umma_commit(empty + s);              // the stage is free once these MMAs have read it
            }
            umma_commit(acc_full);                   // arrives when every MMA above has completed
        }
    } else {
        // ---------------- expand q4 -> f16 A operand (warps 0-3), then the epilogue ----------------
        const int g = lane >> 2, t = lane & 3;
        bool ok = true;
        for (int kb = 0; kb < nkb; kb++) {
            const int s = kb % ST, r = kb >> 1, rs = r % RS, half = kb & 1;
            if (ok && !half && !mbar_wait(raw_full + rs, (r / RS) & 1)) ok = false;
            if (ok && kb >= ST && !mbar_wait(empty + s, ((kb / ST) & 1) ^ 1)) ok = false;
            if (!ok) break;
            const unsigned char *raw = sRaw + rs * RAW;
            unsigned char *dstA = sA + s * A_BYTES;
            #pragma unroll
            for (int q = 0; q < 2; q++) {
                const int ti = warp * 2 + q;                                         // row tile of the CTA's 8
                const uint4 w = *(const uint4 *)(raw + ti * 1024 + half * 512 + lane * 16);
                const uint2 sc = *(const uint2 *)(raw + RAW_SC + ti * 128 + half * 64 + g * 8);
                uint2 dd = make_uint2(0, 0);
                if (FMT == LG_FMT_Q4_K) dd = *(const uint2 *)(raw + RAW_DD + ti * 128 + half * 64 + g * 8);
                #pragma unroll
                for (int sbk = 0; sbk < 2; sbk++)
                    #pragma unroll
                    for (int h8 = 0; h8 < 2; h8++) {
                        const uint32_t word = sbk ? (h8 ? w.w : w.z) : (h8 ? w.y : w.x);
                        const uint32_t sw = sbk ? sc.y : sc.x;
                        const uint32_t lo = (word & 0x0F0F0F0Fu) ^ 0x08080808u, hi = ((word >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;
                        uint2 vlo, vhi;
                        if (FMT == LG_FMT_Q4_0) {
                            const __half d = __ushort_as_half((unsigned short)(h8 ? (sw >> 16) : (sw & 0xffff)));
                            const __half2 d2 = __half2half2(d);
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
                        // row (ti*16 + g + 8*h8): row % 8 == g; 16-byte chunk c of the row sits at c ^ g
                        const int row = ti * 16 + g + 8 * h8;
                        unsigned char *rowp = dstA + (row >> 3) * 1024 + g * 128 + (t & 1) * 8;
                        const int c_lo = 4 * sbk + (t >> 1), c_hi = c_lo + 2;
                        *(uint2 *)(rowp + ((c_lo ^ g) << 4)) = vlo;
                        *(uint2 *)(rowp + ((c_hi ^ g) << 4)) = vhi;
                    }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");           // generic-proxy stores -> visible to the MMA
            mbar_arrive(a_full + s);
            if (half || kb == nkb - 1) mbar_arrive(raw_empty + rs);
        }
        if (!ok && lane == 0) atomicOr(a.err, LG_ERR_MBAR_TIMEOUT);

        // ---------------- epilogue: lane l of warp w holds accumulator row 32w + l ----------------
        if (ok) ok = mbar_wait(acc_full, 0);
        if (!ok && lane == 0) atomicOr(a.err, LG_ERR_MBAR_TIMEOUT);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            const int lrow = warp * 32 + lane;                          // row within the CTA's 128
            const int rt = rt0 + (lrow >> 4);
            for (int c0 = 0; c0 < NT; c0 += 32) {
                if (tok0 + c0 >= a.n_tok) break;                          // uniform per CTA
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + c0, v);
                if (EPI == LG_PF_STORE) {
                    const int row = rt0 * 16 + lrow;
                    if (rt < a.n_row_tiles && row < a.n_rows) {
                        #pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (tok0 + c0 + j < a.n_tok) a.out[(size_t)(tok0 + c0 + j) * a.ldo + row] = __uint_as_float(v[j]);
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
    if (warp == 6) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(NT) : "memory");
    }
}

// f32 rows -> f16 rows (the B operand of the wide matmul)
__global__ void lg_f32_to_f16_rows(const float *__restrict__ src, int ld_src, __half *__restrict__ dst, int ld_dst, int n) {
    pdl_launch(); pdl_wait();
    const int tok = blockIdx.y;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        dst[(size_t)tok * ld_dst + i] = __float2half_rn(src[(size_t)tok * ld_src + i]);
}
