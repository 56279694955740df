// lg_kernels.cuh -- sm_100a device code of the speculative-decode step.
//
// Data layouts (all in HBM, produced once at load or by the kernels below):
//
//  * q4 weight matrix [m rows x k], "tile-major": the matrix is cut into tiles of 16 rows x 64
//    columns (two 32-element quantisation sub-blocks).  One tile is 512 bytes of nibbles, stored
//    so that lane l of a warp reads ONE 16-byte word = exactly its mma.m16n8k32 A-fragment
//    source for both sub-blocks: {row g sb0, row g+8 sb0, row g sb1, row g+8 sb1}, g = l/4, and
//    within a 4-byte word byte i holds element 4t+i in the low nibble and 16+4t+i in the high
//    nibble (t = l%4).  Nibbles are stored as two's-complement (q-8), so "(w<<4)&0xF0F0F0F0"
//    and "w&0xF0F0F0F0" are the signed bytes 16*(q-8).  Tiles of one row-tile are contiguous
//    along k.  Scales travel in a parallel array (64 bytes per tile for q4_0).
//    Same 0.5625 bytes per weight as the file format.
//
//  * activation panel: the M<=8 token rows entering a matmul, quantised per 32-element group
//    to 16-bit integers split into two signed bytes (value = 256*hi + lo, |value| <= 32639) with
//    one f32 scale per (token, group).  Per group the panel holds 8 columns x 32 bytes:
//    column 2j = hi bytes of token j, column 2j+1 = lo bytes, in mma B-fragment order, so one
//    m16n8k32 s8 MMA yields the hi and lo integer dot products of token j for 16 weight rows.
//    Tokens 4..7 live in a second panel.  Integer dots are exact; f32 enters only when a
//    sub-block's integer sum is scaled and accumulated.  Column j never depends on M or on the
//    other columns, which is what makes a verify row bit-identical to a plain decode step.
//
//  * KV cache: per owning layer K and V [seq rows][kv_dim] f16, row(p) = p % seq.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>

#define LG_MAXM 8              // widest verify block
#define LG_QMAX 32639.0f       // 127*256 + 127: keeps both bytes of the split in [-128,127]
#define LG_SPIN_LIMIT (1 << 20)

// error bits a kernel may raise in the engine's status word
#define LG_ERR_MBAR_TIMEOUT 1

struct LgPanel {               // quantised activations of <= 8 tokens, k = 32*nsb columns
    int8_t *q;                 // [2][nsb][256]
    float2 *s;                 // [2][nsb][4]   (scale, scale * sum of the group's integers)
    int nsb;
};

// ---------------------------------------------------------------------------------------------
// small helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Sum over the block in a fixed order (independent of anything but blockDim). `red` >= 32 floats.
__device__ __forceinline__ float block_sum(float v, float *red) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    int nw = (blockDim.x + 31) >> 5;
    float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.0f;
    if (threadIdx.x < 32) t = warp_sum(t);
    if (threadIdx.x == 0) red[0] = t;
    __syncthreads();
    return red[0];
}

__device__ __forceinline__ float gelu_tanh(float x) {
    return 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}

// byte offset of element kk (0..31) inside one 32-byte panel column (B-fragment order)
__device__ __forceinline__ int panel_elem(int kk) { return ((kk & 15) >> 2) * 8 + (kk >> 4) * 4 + (kk & 3); }

// One warp quantises one 32-element group of token `tok`: lane holds element `lane`.
__device__ __forceinline__ void quant_group_store(float y, int lane, int tok, int sb, const LgPanel &P) {
    float amax = warp_max(fabsf(y));
    float d = amax * (1.0f / LG_QMAX);
    float inv = amax > 0.0f ? LG_QMAX / amax : 0.0f;
    int q = __float2int_rn(y * inv);
    q = max(-32639, min(32639, q));
    int lo = ((q + 128) & 255) - 128;
    int hi = (q - lo) >> 8;
    int isum = q;
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) isum += __shfl_xor_sync(0xffffffffu, isum, o);
    size_t base = ((size_t)(tok >> 2) * P.nsb + sb) * 256 + (size_t)((tok & 3) * 2) * 32 + panel_elem(lane);
    P.q[base] = (int8_t)hi;
    P.q[base + 32] = (int8_t)lo;
    if (lane == 0) P.s[((size_t)(tok >> 2) * P.nsb + sb) * 4 + (tok & 3)] = make_float2(d, d * (float)isum);
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// streaming 16-byte weight load: read-only path, do not keep in L1
__device__ __forceinline__ uint4 ldg_stream16(const uint4 *p) {
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_stream8(const uint2 *p) {
    uint2 v;
    asm("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- bulk (TMA, non-tensor) global -> shared copy completed on an mbarrier --------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// dst, src 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// Bounded wait: returns false (and the caller raises LG_ERR_MBAR_TIMEOUT) instead of spinning forever.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    for (int it = 0; it < LG_SPIN_LIMIT; ++it) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

// ---------------------------------------------------------------------------------------------
// weight repack (runs once per tensor at load)
// ---------------------------------------------------------------------------------------------
// q4_0 file blocks [m][k/32][18 B]  ->  tile-major nibbles + f16 scales.  One thread per (tile, lane).
__global__ void lg_repack_q4_0(const uint8_t *__restrict__ src, uint4 *__restrict__ wq, uint2 *__restrict__ ws,
                               int m, int nsb, int n_row_tiles) {
    int nkp = nsb >> 1;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t total = (size_t)n_row_tiles * nkp * 32;
    if (idx >= total) return;
    int lane = idx & 31;
    size_t tile = idx >> 5;
    int kp = (int)(tile % nkp), rt = (int)(tile / nkp);
    int g = lane >> 2, t = lane & 3;
    uint32_t w[4];
    uint16_t d[4];
    #pragma unroll
    for (int j = 0; j < 4; j++) {
        int row = rt * 16 + g + (j & 1) * 8, sb = kp * 2 + (j >> 1);
        w[j] = 0; d[j] = 0;
        if (row < m) {
            const uint8_t *b = src + ((size_t)row * nsb + sb) * 18;
            d[j] = (uint16_t)(b[0] | (b[1] << 8));
            const uint8_t *qs = b + 2 + 4 * t;
            w[j] = ((uint32_t)qs[0] | ((uint32_t)qs[1] << 8) | ((uint32_t)qs[2] << 16) | ((uint32_t)qs[3] << 24)) ^ 0x88888888u;
        }
    }
    wq[idx] = make_uint4(w[0], w[1], w[2], w[3]);
    if (t == 0) ws[tile * 8 + g] = make_uint2((uint32_t)d[0] | ((uint32_t)d[1] << 16), (uint32_t)d[2] | ((uint32_t)d[3] << 16));
}

// 6-bit (scale, min) pair j of a q4_K super-block's 12 packed bytes
__device__ __forceinline__ void q4k_pair(const uint8_t *p, int j, int &sc, int &mn) {
    if (j < 4) { sc = p[j] & 63; mn = p[j + 4] & 63; }
    else { sc = (p[j + 4] & 15) | ((p[j - 4] >> 6) << 4); mn = (p[j + 4] >> 4) | ((p[j] >> 6) << 4); }
}
// q4_K file super-blocks [m][k/256][144 B] -> the same tile-major nibbles; per (row, sub-block) the
// scales array holds {f16 d, f16 dmin, u8 sc, u8 mn} spread over two arrays: ws (uint2 per tile
// lane-group: 4 x (sc | mn<<8) as u16) and wd (uint2 per (tile, g): {d,dmin} of row g and row g+8).
__global__ void lg_repack_q4_K(const uint8_t *__restrict__ src, uint4 *__restrict__ wq, uint2 *__restrict__ ws,
                               uint2 *__restrict__ wd, int m, int nsb, int n_row_tiles) {
    int nkp = nsb >> 1;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t total = (size_t)n_row_tiles * nkp * 32;
    if (idx >= total) return;
    int lane = idx & 31;
    size_t tile = idx >> 5;
    int kp = (int)(tile % nkp), rt = (int)(tile / nkp);
    int g = lane >> 2, t = lane & 3;
    uint32_t w[4], dd[2] = {0, 0};
    uint16_t sm[4];
    #pragma unroll
    for (int j = 0; j < 4; j++) {
        int row = rt * 16 + g + (j & 1) * 8, sb = kp * 2 + (j >> 1);
        w[j] = 0; sm[j] = 0;
        if (row < m) {
            const uint8_t *b = src + ((size_t)row * (nsb >> 3) + (sb >> 3)) * 144;
            int js = sb & 7, sc, mn;
            q4k_pair(b + 4, js, sc, mn);
            sm[j] = (uint16_t)(sc | (mn << 8));
            dd[j & 1] = (uint32_t)b[0] | ((uint32_t)b[1] << 8) | ((uint32_t)b[2] << 16) | ((uint32_t)b[3] << 24);
            const uint8_t *qs = b + 16 + 32 * (js >> 1);
            int sh = (js & 1) * 4;
            uint32_t word = 0;
            #pragma unroll
            for (int i = 0; i < 4; i++) {
                uint32_t lo = (qs[4 * t + i] >> sh) & 15, hi = (qs[16 + 4 * t + i] >> sh) & 15;
                word |= (lo | (hi << 4)) << (8 * i);
            }
            w[j] = word ^ 0x88888888u;
        }
    }
    wq[idx] = make_uint4(w[0], w[1], w[2], w[3]);
    if (t == 0) {
        ws[tile * 8 + g] = make_uint2((uint32_t)sm[0] | ((uint32_t)sm[1] << 16), (uint32_t)sm[2] | ((uint32_t)sm[3] << 16));
        wd[tile * 8 + g] = make_uint2(dd[0], dd[1]);
    }
}

// ---------------------------------------------------------------------------------------------
// exact dequantisation of file-format rows (embedding gather; also the bit-exactness gate)
// ---------------------------------------------------------------------------------------------
// out[i][0..k) = scale * decode(row ids[i]) for q4_0 (type 2) / q4_K (type 12) / f32 (0) / f16 (1)
__global__ void lg_dequant_rows(const uint8_t *__restrict__ src, int type, int k, const int *__restrict__ ids,
                                int n_rows, int row0, float scale, float *__restrict__ out, int ldo) {
    int r = blockIdx.x;
    long long row = ids ? (long long)ids[r] : (long long)row0 + r;
    row = row < 0 ? 0 : (row >= n_rows ? n_rows - 1 : row);        // an out-of-range id must not read outside the table
    float *o = out + (size_t)r * ldo;
    if (type == 2) {
        const uint8_t *base = src + (size_t)row * (k / 32) * 18;
        for (int e = threadIdx.x; e < k; e += blockDim.x) {
            const uint8_t *b = base + (size_t)(e >> 5) * 18;
            float d = __half2float(__ushort_as_half((unsigned short)(b[0] | (b[1] << 8))));
            int j = e & 31;
            int nib = j < 16 ? (b[2 + j] & 15) : (b[2 + j - 16] >> 4);
            o[e] = __fmul_rn(__fmul_rn(d, (float)(nib - 8)), scale);
        }
    } else if (type == 12) {
        const uint8_t *base = src + (size_t)row * (k / 256) * 144;
        for (int e = threadIdx.x; e < k; e += blockDim.x) {
            const uint8_t *b = base + (size_t)(e >> 8) * 144;
            float d = __half2float(__ushort_as_half((unsigned short)(b[0] | (b[1] << 8))));
            float dmin = __half2float(__ushort_as_half((unsigned short)(b[2] | (b[3] << 8))));
            int j = (e & 255) >> 5, l = e & 31, sc, mn;
            q4k_pair(b + 4, j, sc, mn);
            int nib = (b[16 + 32 * (j >> 1) + l] >> ((j & 1) * 4)) & 15;
            float v = __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)nib), __fmul_rn(dmin, (float)mn));
            o[e] = __fmul_rn(v, scale);
        }
    } else if (type == 1) {
        const __half *h = (const __half *)src + (size_t)row * k;
        for (int e = threadIdx.x; e < k; e += blockDim.x) o[e] = __fmul_rn(__half2float(h[e]), scale);
    } else {
        const float *f = (const float *)src + (size_t)row * k;
        for (int e = threadIdx.x; e < k; e += blockDim.x) o[e] = __fmul_rn(f[e], scale);
    }
}

// ---------------------------------------------------------------------------------------------
// the small-M matmul: out[tok][row] = sum_k W[row][k] * x[tok][k]
// ---------------------------------------------------------------------------------------------
struct LgGemvArgs {
    const uint4 *wq;           // tile-major nibbles
    const uint2 *ws;           // q4_0: 4 f16 scales per (tile, g); q4_K: 4 x (sc|mn<<8)
    const uint2 *wd;           // q4_K only: {d,dmin} for rows g and g+8 per (tile, g)
    LgPanel x;
    int nkp;                   // 64-column tile count along k (whole matrix)
    int n_row_tiles;
    int kslices;               // gridDim.y; slice s covers tile columns [s*nkp/kslices, (s+1)*nkp/kslices)
    float *out;                // [kslices][LG_MAXM][ldo] partial sums
    int ldo;
    int M;
    // head epilogue
    float softcap;
    float *logits;             // optional [M][ldo] (n_vocab) when the caller wants the rows
    int n_valid_rows;          // rows >= this are padding
    float *amax_val;           // [gridDim.x][LG_MAXM] per-CTA best logit
    int *amax_idx;
    int *err;
};

enum { LG_FMT_Q4_0 = 0, LG_FMT_Q4_K = 1 };
enum { LG_EPI_STORE = 0, LG_EPI_HEAD = 1 };

#define LG_GEMV_WARPS 8

// One weight fetch of a warp: R row tiles at the same 64-column tile position.
template <int R, int FMT> struct LgWFrag {
    uint4 w[R];
    uint2 sc[R];
    uint2 dd[FMT == LG_FMT_Q4_K ? R : 1];
};

template <int R, int FMT>
__device__ __forceinline__ void gemv_fetch(LgWFrag<R, FMT> &f, const LgGemvArgs &a, int rt0, int kp, int lane, int g) {
    #pragma unroll
    for (int r = 0; r < R; r++) {
        int rt = rt0 + r;
        if (rt < a.n_row_tiles) {
            size_t tile = (size_t)rt * a.nkp + kp;
            f.w[r] = ldg_stream16(a.wq + tile * 32 + lane);
            f.sc[r] = ldg_stream8(a.ws + tile * 8 + g);
            if (FMT == LG_FMT_Q4_K) f.dd[r] = ldg_stream8(a.wd + tile * 8 + g);
        } else {
            f.w[r] = make_uint4(0, 0, 0, 0); f.sc[r] = make_uint2(0, 0);
            if (FMT == LG_FMT_Q4_K) f.dd[r] = make_uint2(0, 0);
        }
    }
}

// A CTA works on items = (group of R consecutive row tiles) x (its k slice, blockIdx.y).  Its 8
// warps split the slice's 64-column tile positions; for each position a warp loads the B fragment
// once from shared memory and applies it to the R row tiles (R independent 16-byte weight loads in
// flight per lane, the next position's loads issued before the current one is consumed).  The
// activation panel slice is staged once per CTA by a bulk copy whose completion is awaited only
// after the first weight loads are in flight.  Partial sums of the 8 warps are added in warp order.
// Dynamic shared memory: [NP][nsb_s][256] int8 | [NP][nsb_s][4] float2 | [8][R*NP*64] f32 | mbarrier
template <int R, int NP, int FMT, int EPI>
__global__ void __launch_bounds__(LG_GEMV_WARPS * 32, 2)
lg_gemv_kernel(LgGemvArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int ks = blockIdx.y;
    const int kp0 = (int)((long long)a.nkp * ks / a.kslices), kp1 = (int)((long long)a.nkp * (ks + 1) / a.kslices);
    const int nsb_s = (kp1 - kp0) * 2;
    int8_t *sq = (int8_t *)smem;
    float2 *ss = (float2 *)(smem + (size_t)NP * nsb_s * 256);
    float *red = (float *)(ss + (size_t)NP * nsb_s * 4);
    uint64_t *bar = (uint64_t *)(red + LG_GEMV_WARPS * R * NP * 64);
    constexpr int SLOTS = (R * NP * 64 + LG_GEMV_WARPS * 32 - 1) / (LG_GEMV_WARPS * 32);
    const int n_groups = (a.n_row_tiles + R - 1) / R;

    if (threadIdx.x == 0) mbar_init(bar, 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t qb = (uint32_t)nsb_s * 256, sb = (uint32_t)nsb_s * 32;
        mbar_expect_tx(bar, NP * (qb + sb));
        #pragma unroll
        for (int p = 0; p < NP; p++) {
            bulk_g2s(sq + (size_t)p * qb, a.x.q + ((size_t)p * a.x.nsb + kp0 * 2) * 256, qb, bar);
            bulk_g2s(ss + (size_t)p * nsb_s * 4, a.x.s + ((size_t)p * a.x.nsb + kp0 * 2) * 4, sb, bar);
        }
    }
    bool staged = false;

    float best_v[SLOTS]; int best_i[SLOTS];
    #pragma unroll
    for (int j = 0; j < SLOTS; j++) { best_v[j] = -INFINITY; best_i[j] = 0x7fffffff; }

    for (int grp = blockIdx.x; grp < n_groups; grp += gridDim.x) {
        const int rt0 = grp * R;
        float acc[R][NP][2];
        #pragma unroll
        for (int r = 0; r < R; r++)
            #pragma unroll
            for (int p = 0; p < NP; p++) acc[r][p][0] = acc[r][p][1] = 0.0f;

        LgWFrag<R, FMT> cur, nxt;
        int kp = kp0 + warp;
        if (kp < kp1) gemv_fetch<R, FMT>(cur, a, rt0, kp, lane, g);
        if (!staged) {
            if (!mbar_wait(bar, 0)) { if (threadIdx.x == 0) atomicOr(a.err, LG_ERR_MBAR_TIMEOUT); }
            staged = true;
        }
        for (; kp < kp1; kp += LG_GEMV_WARPS) {
            const bool more = kp + LG_GEMV_WARPS < kp1;
            if (more) gemv_fetch<R, FMT>(nxt, a, rt0, kp + LG_GEMV_WARPS, lane, g);
            #pragma unroll
            for (int s = 0; s < 2; s++) {
                const int sbl = (kp - kp0) * 2 + s;
                uint2 b[NP]; float2 xs[NP];
                #pragma unroll
                for (int p = 0; p < NP; p++) {
                    b[p] = *(const uint2 *)(sq + ((size_t)p * nsb_s + sbl) * 256 + lane * 8);
                    xs[p] = ss[((size_t)p * nsb_s + sbl) * 4 + t];
                }
                #pragma unroll
                for (int r = 0; r < R; r++) {
                    uint32_t wg = s ? cur.w[r].z : cur.w[r].x, wh = s ? cur.w[r].w : cur.w[r].y;
                    uint32_t a0 = (wg << 4) & 0xF0F0F0F0u, a2 = wg & 0xF0F0F0F0u;
                    uint32_t a1 = (wh << 4) & 0xF0F0F0F0u, a3 = wh & 0xF0F0F0F0u;
                    float d0, d1, m0 = 0.0f, m1 = 0.0f;
                    uint32_t sw = s ? cur.sc[r].y : cur.sc[r].x;
                    if (FMT == LG_FMT_Q4_0) {
                        float2 f = __half22float2(*(const __half2 *)&sw);
                        d0 = f.x; d1 = f.y;
                    } else {
                        float2 r0 = __half22float2(*(const __half2 *)&cur.dd[r].x), r1 = __half22float2(*(const __half2 *)&cur.dd[r].y);
                        d0 = r0.x * (float)(sw & 0xff); m0 = 16.0f * (8.0f * d0 - r0.y * (float)((sw >> 8) & 0xff));
                        d1 = r1.x * (float)((sw >> 16) & 0xff); m1 = 16.0f * (8.0f * d1 - r1.y * (float)(sw >> 24));
                    }
                    #pragma unroll
                    for (int p = 0; p < NP; p++) {
                        int c[4] = {0, 0, 0, 0};
                        mma_s8(c, a0, a1, a2, a3, b[p].x, b[p].y);
                        float v0 = (float)((c[0] << 8) + c[1]) * xs[p].x;      // row g,   token 4p+t
                        float v1 = (float)((c[2] << 8) + c[3]) * xs[p].x;      // row g+8
                        acc[r][p][0] = fmaf(v0, d0, acc[r][p][0]);
                        acc[r][p][1] = fmaf(v1, d1, acc[r][p][1]);
                        if (FMT == LG_FMT_Q4_K) {     // nibbles are stored as (q-8): add back (8 d sc - dmin m) * sum(x)
                            acc[r][p][0] = fmaf(m0, xs[p].y, acc[r][p][0]);
                            acc[r][p][1] = fmaf(m1, xs[p].y, acc[r][p][1]);
                        }
                    }
                }
            }
            if (more) cur = nxt;
        }

        // fixed-order sum over the 8 warps
        #pragma unroll
        for (int r = 0; r < R; r++)
            #pragma unroll
            for (int p = 0; p < NP; p++) {
                red[(warp * R * NP + r * NP + p) * 64 + t * 16 + g] = acc[r][p][0];
                red[(warp * R * NP + r * NP + p) * 64 + t * 16 + g + 8] = acc[r][p][1];
            }
        __syncthreads();
        #pragma unroll
        for (int j = 0; j < SLOTS; j++) {
            int idx = threadIdx.x + j * LG_GEMV_WARPS * 32;
            if (idx < R * NP * 64) {
                int rp = idx >> 6, r = rp / NP, p = rp % NP, tok = p * 4 + ((idx >> 4) & 3);
                float sum = 0.0f;
                #pragma unroll
                for (int w2 = 0; w2 < LG_GEMV_WARPS; w2++) sum += red[w2 * R * NP * 64 + idx];
                sum *= 0.0625f;
                int row = (rt0 + r) * 16 + (idx & 15);
                if (rt0 + r < a.n_row_tiles && tok < a.M) {
                    if (EPI == LG_EPI_STORE) {
                        a.out[((size_t)ks * LG_MAXM + tok) * a.ldo + row] = sum;
                    } else if (row < a.n_valid_rows) {
                        if (a.softcap > 0.0f) sum = a.softcap * tanhf(sum / a.softcap);
                        if (a.logits) a.logits[(size_t)tok * a.ldo + row] = sum;
                        if (sum > best_v[j]) { best_v[j] = sum; best_i[j] = row; }   // rows ascend per slot: first max wins
                    }
                }
            }
        }
        __syncthreads();
    }

    if (EPI == LG_EPI_HEAD) {
        // candidates of this CTA: one per (slot, thread); merge per token (larger value, lower index on ties)
        float *cv = red; int *ci = (int *)(red + R * NP * 64);
        #pragma unroll
        for (int j = 0; j < SLOTS; j++) {
            int idx = threadIdx.x + j * LG_GEMV_WARPS * 32;
            if (idx < R * NP * 64) { cv[idx] = best_v[j]; ci[idx] = best_i[j]; }
        }
        __syncthreads();
        if (threadIdx.x < a.M) {
            int tok = threadIdx.x, p = tok >> 2, tl = tok & 3;
            float bv = -INFINITY; int bi = 0x7fffffff;
            for (int r = 0; r < R; r++)
                for (int row = 0; row < 16; row++) {
                    int idx = ((r * NP + p) * 4 + tl) * 16 + row;
                    float v = cv[idx]; int i2 = ci[idx];
                    if (v > bv || (v == bv && i2 < bi)) { bv = v; bi = i2; }
                }
            a.amax_val[(size_t)blockIdx.x * LG_MAXM + tok] = bv;
            a.amax_idx[(size_t)blockIdx.x * LG_MAXM + tok] = bi;
        }
    }
}

// Merge the per-CTA argmax candidates: out[tok] = index of the largest logit, lowest index on ties.
__global__ void lg_argmax_final(const float *__restrict__ val, const int *__restrict__ idx, int n_parts, int *out) {
    int tok = blockIdx.x;
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < n_parts; i += blockDim.x) {
        float v = val[(size_t)i * LG_MAXM + tok]; int x = idx[(size_t)i * LG_MAXM + tok];
        if (v > bv || (v == bv && x < bi)) { bv = v; bi = x; }
    }
    __shared__ float sv[32]; __shared__ int si[32];
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        int nw = blockDim.x >> 5;
        bv = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY; bi = threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
        #pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (threadIdx.x == 0) out[tok] = bi == 0x7fffffff ? 0 : bi;
    }
}

// ---------------------------------------------------------------------------------------------
// embedding gather
// ---------------------------------------------------------------------------------------------
// x[tok][0..ne) = decode(token_embd row toks[tok]) * sqrt(ne) from the TILE-MAJOR copy (the same
// matrix is the output head).  Bit-identical to decoding the file row: value = d * (nibble-8).
__global__ void lg_embed_rows(const uint4 *__restrict__ wq, const uint2 *__restrict__ ws, const uint2 *__restrict__ wd,
                              int fmt, int nkp, int n_rows, const int *__restrict__ toks, float scale,
                              float *__restrict__ out, int ldo) {
    int tok = blockIdx.x;
    int row = min(max(toks[tok], 0), n_rows - 1);               // an out-of-range id must not read outside the table
    int rt = row >> 4, r = row & 15, g = r & 7, hi8 = r >> 3;
    const uint32_t *wq32 = (const uint32_t *)wq;
    for (int e = threadIdx.x; e < nkp * 64; e += blockDim.x) {
        int kp = e >> 6, s = (e >> 5) & 1, kk = e & 31;
        int t = (kk & 15) >> 2, i = kk & 3;
        size_t tile = (size_t)rt * nkp + kp;
        uint32_t word = wq32[(tile * 32 + g * 4 + t) * 4 + s * 2 + hi8];
        int nib = (word >> (8 * i + (kk >> 4) * 4)) & 15;
        int qv = (nib ^ 8) - 8;                               // stored two's complement of (q-8)
        uint2 sc = ws[tile * 8 + g];
        uint32_t sw = s ? sc.y : sc.x;
        float v;
        if (fmt == LG_FMT_Q4_0) {
            float d = __half2float(__ushort_as_half((unsigned short)(hi8 ? (sw >> 16) : (sw & 0xffff))));
            v = __fmul_rn(d, (float)qv);
        } else {
            uint2 dd = wd[tile * 8 + g];
            uint32_t dw = hi8 ? dd.y : dd.x;
            float d = __half2float(__ushort_as_half((unsigned short)(dw & 0xffff)));
            float dmin = __half2float(__ushort_as_half((unsigned short)(dw >> 16)));
            uint32_t sm = hi8 ? (sw >> 16) : (sw & 0xffff);
            v = __fsub_rn(__fmul_rn(__fmul_rn(d, (float)(sm & 0xff)), (float)(qv + 8)), __fmul_rn(dmin, (float)(sm >> 8)));
        }
        out[(size_t)tok * ldo + e] = __fmul_rn(v, scale);
    }
}

// ---------------------------------------------------------------------------------------------
// norms
// ---------------------------------------------------------------------------------------------
// One CTA per token row.
//   if (add_src)  x += rmsnorm(sum of n_parts partials of add_src) * add_w ; x *= out_scale
//   if (norm_w)   y  = rmsnorm(x) * norm_w  -> panel (quantised) and/or y_f32
// Either half may be absent.  rmsnorm(v) = v * (1/sqrt(mean(v^2) + eps)).
struct LgNormArgs {
    float *x; int ldx;                   // residual stream rows [M][ldx]
    const float *add_src; int n_parts; size_t part_stride; int ld_add;   // partial p at add_src + p*part_stride + tok*ld_add
    const float *add_w; float out_scale;
    const float *norm_w;
    LgPanel panel; int want_panel;
    float *y; int ldy;                   // optional f32 copy of the normed row
    int n; float eps;
};
__global__ void lg_norm_kernel(LgNormArgs a) {
    extern __shared__ float row[];       // n floats + 32
    float *red = row + a.n;
    const int tok = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float *x = a.x + (size_t)tok * a.ldx;
    if (a.add_src) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < a.n; i += blockDim.x) {
            float v = 0.0f;
            for (int p = 0; p < a.n_parts; p++) v += a.add_src[(size_t)p * a.part_stride + (size_t)tok * a.ld_add + i];
            row[i] = v;
            ss += v * v;
        }
        ss = block_sum(ss, red);
        float s = 1.0f / sqrtf(ss / (float)a.n + a.eps);
        for (int i = threadIdx.x; i < a.n; i += blockDim.x) {
            float v = __fadd_rn(x[i], __fmul_rn(__fmul_rn(row[i], s), a.add_w[i]));
            v = __fmul_rn(v, a.out_scale);
            x[i] = v;
            row[i] = v;
        }
    } else {
        for (int i = threadIdx.x; i < a.n; i += blockDim.x) row[i] = x[i];
    }
    if (!a.norm_w && !a.want_panel && !a.y) return;
    __syncthreads();
    float s = 1.0f;
    if (a.norm_w) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < a.n; i += blockDim.x) ss += row[i] * row[i];
        ss = block_sum(ss, red);
        s = 1.0f / sqrtf(ss / (float)a.n + a.eps);
    }
    for (int sb = warp; sb * 32 < a.n; sb += nw) {
        int i = sb * 32 + lane;
        float yv = a.norm_w ? __fmul_rn(__fmul_rn(row[i], s), a.norm_w[i]) : row[i];   // no norm_w: the row itself
        if (a.y) a.y[(size_t)tok * a.ldy + i] = yv;
        if (a.want_panel) quant_group_store(yv, lane, tok, sb, a.panel);
    }
}

// Quantise f32 rows into a panel (used where the producer is not one of the fused kernels).
__global__ void lg_quant_rows(const float *__restrict__ x, int ldx, int n, LgPanel P) {
    int tok = blockIdx.y, lane = threadIdx.x & 31;
    int sb = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (sb * 32 >= n) return;
    quant_group_store(x[(size_t)tok * ldx + sb * 32 + lane], lane, tok, sb, P);
}

// ---------------------------------------------------------------------------------------------
// per-head q/k/v post-processing: rmsnorm, NeoX RoPE at pos+tok, f16 KV write
// ---------------------------------------------------------------------------------------------
// qkv: [M][ld] rows = [q (H*hd) | k (Hkv*hd) | v (Hkv*hd)] from the matmul (v absent: v = k projection).
// grid (H + 2*Hkv, M), block hd/2 threads ... each thread owns the pair (i, i+hd/2).
struct LgQkvArgs {
    const float *qkv; int ld;
    int H, Hkv, hd; int has_v; int owns_kv;
    const float *q_norm, *k_norm;        // [hd]
    const float *rope_div;               // [hd/2] or null
    float rope_base; float eps;
    const int *pos;                      // device position of token 0
    float *q_out;                        // [M][H*hd] f32 (normed + rotated)
    __half *kc, *vc; int seq, kv_dim;    // cache of this layer
};
__global__ void lg_qkv_post_kernel(LgQkvArgs a) {
    __shared__ float red[32];
    const int head = blockIdx.x, tok = blockIdx.y, i = threadIdx.x, half = a.hd >> 1;
    const int pos = *a.pos + tok;
    int kind = head < a.H ? 0 : (head < a.H + a.Hkv ? 1 : 2);   // q, k, v
    if (kind && !a.owns_kv) return;
    int hh = kind == 0 ? head : (kind == 1 ? head - a.H : head - a.H - a.Hkv);
    size_t col = kind == 0 ? (size_t)hh * a.hd
               : (kind == 1 || !a.has_v) ? (size_t)(a.H + hh) * a.hd
               : (size_t)(a.H + a.Hkv + hh) * a.hd;
    const float *src = a.qkv + (size_t)tok * a.ld + col;
    float v0 = src[i], v1 = src[i + half];
    float ss = block_sum(v0 * v0 + v1 * v1, red);
    float s = 1.0f / sqrtf(ss / (float)a.hd + a.eps);
    if (kind == 2) {
        size_t r = (size_t)(pos % a.seq) * a.kv_dim + (size_t)hh * a.hd;
        a.vc[r + i] = __float2half_rn(__fmul_rn(v0, s));
        a.vc[r + i + half] = __float2half_rn(__fmul_rn(v1, s));
        return;
    }
    const float *w = kind == 0 ? a.q_norm : a.k_norm;
    v0 = __fmul_rn(__fmul_rn(v0, s), w[i]);
    v1 = __fmul_rn(__fmul_rn(v1, s), w[i + half]);
    float freq = powf(a.rope_base, -2.0f * (float)i / (float)a.hd);
    float ang = (float)pos * freq / (a.rope_div ? a.rope_div[i] : 1.0f);
    float c = cosf(ang), sn = sinf(ang);
    float r0 = __fsub_rn(__fmul_rn(v0, c), __fmul_rn(v1, sn));
    float r1 = __fadd_rn(__fmul_rn(v0, sn), __fmul_rn(v1, c));
    if (kind == 0) {
        float *q = a.q_out + ((size_t)tok * a.H + hh) * a.hd;
        q[i] = r0; q[i + half] = r1;
    } else {
        size_t r = (size_t)(pos % a.seq) * a.kv_dim + (size_t)hh * a.hd;
        a.kc[r + i] = __float2half_rn(r0);
        a.kc[r + i + half] = __float2half_rn(r1);
    }
}

// ---------------------------------------------------------------------------------------------
// split-KV flash-decode over the f16 cache
// ---------------------------------------------------------------------------------------------
// Keys are partitioned on ABSOLUTE position boundaries: tile T covers positions [T*S, (T+1)*S).
// Query j (token j of the block, position p_j = pos + j + qpos_off) attends positions
// [max(0, p_j - window + 1), p_j]  (window <= 0: from 0).  A CTA handles one KV head and one tile
// for all queries of the block (gqa heads x M tokens); per (query, tile) it emits the partial
// (max, sum, acc[hd]) of an online softmax.  The combine kernel merges a query's tiles in
// ascending order.  A partial depends only on (query position, tile), never on M or on which
// other queries share the launch.
struct LgAttnArgs {
    const float *q;            // [M][H][hd]
    const __half *kc, *vc; int seq, kv_dim;
    int H, Hkv, hd, M;
    int S;                     // tile size (keys)
    int n_slots;               // tile slots in the scratch (>= tiles a block can touch)
    int window;                // <=0: full causal
    int qpos_off;              // 0 for the target; -1 for the draft head (query at pos sees keys < pos)
    int win_shrink;            // draft head: window start stays pos-W+1 (one fewer key)
    const int *pos;
    float *part;               // [n_slots][M][H][hd+2]  (acc[hd], max, sum)
    LgPanel out; float *out_f32;   // combine output: panel of [M][H*hd] and/or f32
};

#define LG_ATTN_THREADS 256
// dynamic smem: q [nq][hd] f32 | kv tile [S][hd+8] f16 | scores [nq][S] f32
__global__ void __launch_bounds__(LG_ATTN_THREADS) lg_attn_split_kernel(LgAttnArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int kvh = blockIdx.x, gqa = a.H / a.Hkv, nq = gqa * a.M, hd = a.hd, S = a.S;
    const int pos0 = *a.pos;
    // tile range touched by this block of queries
    int p_first = pos0 + a.qpos_off, p_last = pos0 + a.M - 1 + a.qpos_off;
    if (p_last < 0) return;
    int lo_first = a.window > 0 ? max(0, p_first + a.win_shrink - a.window + 1) : 0;
    int t_lo = lo_first / S, t_hi = p_last / S;
    int T = t_lo + blockIdx.y;
    if (T > t_hi) return;
    const int slot = T % a.n_slots;

    float *sq = (float *)smem;                                   // [nq][hd]
    __half *skv = (__half *)(sq + (size_t)nq * hd);              // [S][hd+8]
    float *sc = (float *)(skv + (size_t)S * (hd + 8));           // [nq][S]
    const int ldk = hd + 8;

    for (int i = threadIdx.x; i < nq * hd; i += blockDim.x) {
        int qi = i / hd, d = i % hd, tok = qi / gqa, hq = kvh * gqa + qi % gqa;
        sq[i] = a.q[((size_t)tok * a.H + hq) * hd + d];
    }
    // K tile -> smem (16-byte chunks)
    const int chunks = hd / 8;
    for (int i = threadIdx.x; i < S * chunks; i += blockDim.x) {
        int key = i / chunks, c = i % chunks;
        int p = T * S + key;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (p <= p_last) v = *(const uint4 *)(a.kc + (size_t)(p % a.seq) * a.kv_dim + (size_t)kvh * hd + c * 8);
        *(uint4 *)(skv + (size_t)key * ldk + c * 8) = v;
    }
    __syncthreads();
    // scores
    for (int i = threadIdx.x; i < nq * S; i += blockDim.x) {
        int qi = i / S, key = i % S;
        int p = T * S + key;
        int pj = pos0 + qi / gqa + a.qpos_off;
        int lo = a.window > 0 ? max(0, pj + a.win_shrink - a.window + 1) : 0;
        float s = -INFINITY;
        if (p >= lo && p <= pj) {
            s = 0.0f;
            const float *qv = sq + (size_t)qi * hd;
            const __half *kr = skv + (size_t)key * ldk;
            for (int d = 0; d < hd; d += 8) {
                uint4 kk = *(const uint4 *)(kr + d);
                const __half2 *h2 = (const __half2 *)&kk;
                float4 qa = *(const float4 *)(qv + d), qb = *(const float4 *)(qv + d + 4);
                float2 k0 = __half22float2(h2[0]), k1 = __half22float2(h2[1]), k2 = __half22float2(h2[2]), k3 = __half22float2(h2[3]);
                s = fmaf(qa.x, k0.x, s); s = fmaf(qa.y, k0.y, s); s = fmaf(qa.z, k1.x, s); s = fmaf(qa.w, k1.y, s);
                s = fmaf(qb.x, k2.x, s); s = fmaf(qb.y, k2.y, s); s = fmaf(qb.z, k3.x, s); s = fmaf(qb.w, k3.y, s);
            }
        }
        sc[i] = s;
    }
    __syncthreads();
    // V tile -> smem (reuses the K buffer)
    for (int i = threadIdx.x; i < S * chunks; i += blockDim.x) {
        int key = i / chunks, c = i % chunks;
        int p = T * S + key;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (p <= p_last) v = *(const uint4 *)(a.vc + (size_t)(p % a.seq) * a.kv_dim + (size_t)kvh * hd + c * 8);
        *(uint4 *)(skv + (size_t)key * ldk + c * 8) = v;
    }
    // per-query tile softmax: one warp per query
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int qi = warp; qi < nq; qi += nw) {
        float mx = -INFINITY;
        for (int k2 = lane; k2 < S; k2 += 32) mx = fmaxf(mx, sc[qi * S + k2]);
        mx = warp_max(mx);
        float sum = 0.0f;
        for (int k2 = lane; k2 < S; k2 += 32) {
            float s = sc[qi * S + k2];
            float e = (s == -INFINITY) ? 0.0f : expf(s - mx);
            sc[qi * S + k2] = e;
            sum += e;
        }
        sum = warp_sum(sum);
        if (lane == 0) {
            int tok = qi / gqa, hq = kvh * gqa + qi % gqa;
            float *pp = a.part + (((size_t)slot * a.M + tok) * a.H + hq) * (hd + 2);
            pp[hd] = mx; pp[hd + 1] = sum;
        }
    }
    __syncthreads();
    // P V: thread owns a dim pair for a subset of queries
    const int npair = hd / 2, qstep = blockDim.x / npair;      // hd 256: 128 pairs, 2 query lanes; hd 64: 32 pairs, 8
    const int dp = threadIdx.x % npair;
    for (int qi = threadIdx.x / npair; qi < nq; qi += qstep) {
        float a0 = 0.0f, a1 = 0.0f;
        const float *pr = sc + (size_t)qi * S;
        for (int key = 0; key < S; key++) {
            float2 vv = __half22float2(*(const __half2 *)(skv + (size_t)key * ldk + dp * 2));
            float pw = pr[key];
            a0 = fmaf(pw, vv.x, a0); a1 = fmaf(pw, vv.y, a1);
        }
        int tok = qi / gqa, hq = kvh * gqa + qi % gqa;
        float *pp = a.part + (((size_t)slot * a.M + tok) * a.H + hq) * (hd + 2);
        pp[dp * 2] = a0; pp[dp * 2 + 1] = a1;
    }
}

// grid (H, M), block hd threads: merge the tiles of one (token, head) in ascending tile order.
__global__ void lg_attn_combine_kernel(LgAttnArgs a) {
    const int hq = blockIdx.x, tok = blockIdx.y, d = threadIdx.x, hd = a.hd, S = a.S;
    const int pj = *a.pos + tok + a.qpos_off;
    float acc = 0.0f, m = -INFINITY, l = 0.0f;
    if (pj >= 0) {
        int lo = a.window > 0 ? max(0, pj + a.win_shrink - a.window + 1) : 0;
        for (int T = lo / S; T <= pj / S; T++) {
            const float *pp = a.part + (((size_t)(T % a.n_slots) * a.M + tok) * a.H + hq) * (hd + 2);
            float pm = pp[hd], pl = pp[hd + 1];
            if (pl <= 0.0f) continue;
            float nm = fmaxf(m, pm);
            float s_old = (m == -INFINITY) ? 0.0f : expf(m - nm), s_new = expf(pm - nm);
            acc = acc * s_old + pp[d] * s_new;
            l = l * s_old + pl * s_new;
            m = nm;
        }
    }
    float y = l > 0.0f ? acc / l : 0.0f;
    if (a.out_f32) a.out_f32[((size_t)tok * a.H + hq) * hd + d] = y;
    if (a.out.q) quant_group_store(y, d & 31, tok, (hq * hd + d) >> 5, a.out);
}

// ---------------------------------------------------------------------------------------------
// GeGLU and the per-layer-embedding elementwise pieces
// ---------------------------------------------------------------------------------------------
// y = gelu_tanh(gate) * up -> panel.  gate/up are f32 rows; `up` may be a per-token vector (PLE).
__global__ void lg_geglu_kernel(const float *__restrict__ gate, const float *__restrict__ up, int ld_g, int ld_u,
                                int n, LgPanel P) {
    int tok = blockIdx.y, lane = threadIdx.x & 31;
    int sb = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (sb * 32 >= n) return;
    int i = sb * 32 + lane;
    float y = __fmul_rn(gelu_tanh(gate[(size_t)tok * ld_g + i]), up[(size_t)tok * ld_u + i]);
    quant_group_store(y, lane, tok, sb, P);
}

// Per-layer inputs: ipl[tok][L][ple] = (rmsnorm(proj[tok][L][:] / sqrt(ne)) * w + tokrow[tok][L][:]) / sqrt(2)
// grid (n_layer, M), block = ple threads (ple % 32 == 0, <= 1024)
__global__ void lg_ple_build_kernel(const float *__restrict__ proj, const float *__restrict__ tokrow,
                                    const float *__restrict__ w, float *__restrict__ ipl, int ple, int total,
                                    float inv_sqrt_ne, float eps) {
    __shared__ float red[32];
    int L = blockIdx.x, tok = blockIdx.y, i = threadIdx.x;
    size_t o = (size_t)tok * total + (size_t)L * ple + i;
    float v = __fmul_rn(proj[o], inv_sqrt_ne);
    float ss = block_sum(v * v, red);
    float s = 1.0f / sqrtf(ss / (float)ple + eps);
    float y = __fmul_rn(__fmul_rn(v, s), w[i]);
    ipl[o] = __fmul_rn(__fadd_rn(y, tokrow[o]), 0.70710678118654752f);
}

// ---------------------------------------------------------------------------------------------
// greedy acceptance, position advance and hand-off to the next round -- all on the device
// ---------------------------------------------------------------------------------------------
struct LgRoundState {          // lives in device memory; one per session
    int pos;                   // position of toks[0] of the round being built
    int toks[LG_MAXM];         // toks[0] = chosen token, toks[1..] = drafts
    int out[LG_MAXM];          // greedy successors of toks[j]
    int adv;                   // tokens advanced by the last verify (1..M)
    int n_emitted;             // tokens appended to the log so far
    int n_draft, n_accept;
    int dpos;                  // position the draft head is drafting for
};
// After a verify of M rows: adv = 1 + run of out[j-1] == toks[j]; append toks[1..adv-1] and
// out[adv-1] to the token log; next round starts at pos+adv with toks[0] = out[adv-1];
// h_prev <- normed hidden of row adv-1.  (The cache needs no rollback: rows past pos+adv are
// overwritten by the next round before any query can read them.)
__global__ void lg_accept_kernel(LgRoundState *st, int M, const float *__restrict__ hidden, int ld, int ne,
                                 float *__restrict__ h_prev, int *__restrict__ log, int log_cap,
                                 int advance_state) {
    __shared__ int s_adv;
    if (threadIdx.x == 0) {
        int adv = 1;
        while (adv < M && st->out[adv - 1] == st->toks[adv]) adv++;
        s_adv = adv;
        st->adv = adv;
        if (advance_state) {
            int n = st->n_emitted;
            for (int j = 1; j < adv; j++) { if (n < log_cap) log[n] = st->toks[j]; n++; }
            if (n < log_cap) log[n] = st->out[adv - 1];
            n++;
            st->n_emitted = n;
            st->n_draft += M - 1; st->n_accept += adv - 1;
            st->pos += adv;
            st->toks[0] = st->out[adv - 1];
        }
    }
    __syncthreads();
    const float *src = hidden + (size_t)(s_adv - 1) * ld;
    for (int i = threadIdx.x; i < ne; i += blockDim.x) h_prev[i] = src[i];
}

// drafts for the coming round: slot j <- replay[n_emitted + j - 1] (oracle-replayed drafts)
__global__ void lg_replay_drafts_kernel(LgRoundState *st, int M, const int *__restrict__ replay, int n_replay) {
    int j = threadIdx.x + 1;
    if (j < M) { int i = st->n_emitted + j - 1; st->toks[j] = i < n_replay ? replay[i] : 0; }
}

// draft-head input: cat = [ embed(tok)*sqrt(nb) , h_prev ] is assembled by lg_embed_rows + this copy
__global__ void lg_copy_f32(float *__restrict__ dst, const float *__restrict__ src, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = src[i];
}
__global__ void lg_set_draft_pos(LgRoundState *st, int j) { st->dpos = st->pos + j; }
// slots a head cannot draft repeat the previous token, so the verify simply rejects them
__global__ void lg_pad_drafts(LgRoundState *st, int from, int M) { for (int j = from; j < M; j++) st->toks[j] = st->toks[j - 1]; }
__global__ void lg_store_draft(LgRoundState *st, int j, const int *best) { st->toks[j] = *best; }
