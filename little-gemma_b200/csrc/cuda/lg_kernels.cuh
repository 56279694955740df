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
#include "lg_formats.h"

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

// Programmatic dependent launch: every kernel of a forward may be started before its predecessor
// has finished.  pdl_launch() lets the successor begin its own prologue; pdl_wait() blocks until the
// predecessor grid has completed and its writes are visible.  Nothing produced by an earlier kernel
// may be read, and nothing may be written, before pdl_wait().  (No-ops for a plain launch.)
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- phase time stamps (profiling builds only: -DLG_STAMPS) ------------------------------------
// Thread 0 of a CTA records the global nanosecond timer at named points of a kernel into
// lg_stamps[launch tag][CTA][slot]; the host reads the array back after a forward and lays the launches of a
// layer on one time axis (lg_debug_stamps).  Compiled out of the product build.
#define LG_STAMP_LAUNCHES 96
#define LG_STAMP_CTAS 320
#define LG_STAMP_SLOTS 12
#ifdef LG_STAMPS
__device__ long long lg_stamps[LG_STAMP_LAUNCHES][LG_STAMP_CTAS][LG_STAMP_SLOTS];
__device__ __forceinline__ void lg_stamp(int tag, int slot) {
    if (threadIdx.x == 0 && tag >= 0 && tag < LG_STAMP_LAUNCHES) {
        const int cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
        if (cta < LG_STAMP_CTAS) {
            long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            lg_stamps[tag][cta][slot] = t;
        }
    }
}
#define LG_STAMP(tag, slot) lg_stamp(tag, slot)
// the last slot of CTA 0 names the kernel (1 matmul store, 2 head, 3 GeGLU, 4 matmul with sums, 5 attention/ticket, 6 attention/cluster, 7 norm / residual update)
#define LG_STAMP_KIND(tag, kind) do { if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && (tag) >= 0 && (tag) < LG_STAMP_LAUNCHES) lg_stamps[tag][0][LG_STAMP_SLOTS - 1] = (kind); } while (0)
#else
#define LG_STAMP(tag, slot) do { } while (0)
#define LG_STAMP_KIND(tag, kind) do { } while (0)
#endif

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

__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void dsmem_store(float *local_addr, uint32_t rank, float v) {
    uint32_t la = smem_u32(local_addr), ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(la), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" :: "r"(ra), "f"(v) : "memory");
}
// One f32 into a peer CTA's shared memory, counted (4 bytes) on that peer's mbarrier: the receiver waits for the byte
// count instead of a cluster-wide barrier, so threads that never join a barrier (a producer warp) are no obstacle.
__device__ __forceinline__ void dsmem_st_async_f32(float *local_addr, uint64_t *local_bar, uint32_t rank, float v) {
    uint32_t ra, rb;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(smem_u32(local_addr)), "r"(rank));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rb) : "r"(smem_u32(local_bar)), "r"(rank));
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.f32 [%0], %1, [%2];" :: "r"(ra), "f"(v), "r"(rb) : "memory");
}
// Bounded wait with cluster-scope acquire: the data counted on the barrier came from peer CTAs.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t *bar, uint32_t parity) {
    for (int it = 0; it < LG_SPIN_LIMIT; ++it) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

// Bounded-wait probe: waits on an mbarrier nobody completes, for at most `polls` polls, then reports like the kernels do.
__global__ void lg_wait_probe_kernel(int *err, int polls) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        bool done = false;
        for (int it = 0; it < polls && !done; ++it) {
            uint32_t ok;
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(ok) : "r"(smem_u32(&bar)), "r"(0u) : "memory");
            done = ok != 0;
        }
        if (!done) atomicOr(err, LG_ERR_MBAR_TIMEOUT);
    }
}

// ---------------------------------------------------------------------------------------------
// weight repack (runs once per tensor at load)
// ---------------------------------------------------------------------------------------------
// q4_0 file blocks [m][k/32][18 B]  ->  tile-major nibbles + f16 scales.  One thread per (tile, lane).
// With src_b set, tile rt is made of rows [8rt, 8rt+8) of src followed by the same rows of src_b
// (gate and up interleaved, so one thread's two accumulators are gate_i and up_i).
__global__ void lg_repack_q4_0(const uint8_t *__restrict__ src, const uint8_t *__restrict__ src_b,
                               uint4 *__restrict__ wq, uint2 *__restrict__ ws, int m, int nsb, int n_row_tiles) {
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
        int row = src_b ? rt * 8 + g : rt * 16 + g + (j & 1) * 8, sb = kp * 2 + (j >> 1);
        w[j] = 0; d[j] = 0;
        if (row < m) {
            const uint8_t *b = ((src_b && (j & 1)) ? src_b : src) + ((size_t)row * nsb + sb) * 18;
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
__global__ void lg_repack_q4_K(const uint8_t *__restrict__ src, const uint8_t *__restrict__ src_b,
                               uint4 *__restrict__ wq, uint2 *__restrict__ ws,
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
        int row = src_b ? rt * 8 + g : rt * 16 + g + (j & 1) * 8, sb = kp * 2 + (j >> 1);
        w[j] = 0; sm[j] = 0;
        if (row < m) {
            const uint8_t *b = ((src_b && (j & 1)) ? src_b : src) + ((size_t)row * (nsb >> 3) + (sb >> 3)) * 144;
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

// File blocks of q8_0 / q6_K / q5_K / q3_K [m][k/blk][bytes] -> i8 tiles.  One thread per (tile, lane, sub-block): its 16
// bytes are {row g, row g+8} x {columns 4t..4t+3, 16+4t..16+4t+3} of that sub-block = the A operands of the two k16 MMAs.
// wq: [tile][2 sub-blocks][32 lanes] uint4;  ws: f16 d {row g sb0, row g+8 sb0, row g sb1, row g+8 sb1} per (tile, g);
// wd: integer scales, .x = row g {sb0 cols 0-15, sb0 16-31, sb1 0-15, sb1 16-31}, .y = row g+8;  wm: f32 dmin*m (q5_K).
// With src_b: the two tensors woven 8 rows at a time, as in lg_repack_q4_0.
__global__ void lg_repack_i8(const uint8_t *__restrict__ src, const uint8_t *__restrict__ src_b, int type,
                             uint4 *__restrict__ wq, uint2 *__restrict__ ws, uint2 *__restrict__ wd, uint4 *__restrict__ wm,
                             int m, int nsb, int n_row_tiles) {
    const int nkp = nsb >> 1;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)n_row_tiles * nkp * 64;
    if (idx >= total) return;
    const int lane = idx & 31, sb_in = (idx >> 5) & 1;
    const size_t tile = idx >> 6;
    const int kp = (int)(tile % nkp), rt = (int)(tile / nkp);
    const int g = lane >> 2, t = lane & 3;
    const int blk = lg_fmt_block(type), bytes = lg_fmt_bytes(type), k = nsb * 32;
    uint32_t w[4] = {0, 0, 0, 0};
    uint32_t dsc[2] = {0, 0}, isc[2] = {0, 0}; float mo[2] = {0.0f, 0.0f};
    #pragma unroll
    for (int hi8 = 0; hi8 < 2; hi8++) {
        const int row = src_b ? rt * 8 + g : rt * 16 + g + hi8 * 8;
        if (row >= m) continue;
        const uint8_t *base = ((src_b && hi8) ? src_b : src) + (size_t)row * (k / blk) * bytes;
        #pragma unroll
        for (int half = 0; half < 2; half++) {
            uint32_t word = 0;
            #pragma unroll
            for (int i = 0; i < 4; i++) {
                const int col = kp * 64 + sb_in * 32 + half * 16 + 4 * t + i;
                int q, sc, mi; uint16_t db, mb;
                lg_fmt_elem(type, base + (size_t)(col / blk) * bytes, col % blk, &q, &sc, &db, &mb, &mi);
                word |= (uint32_t)(uint8_t)(int8_t)q << (8 * i);
                if (t == 0 && i == 0) {
                    dsc[hi8] = db;
                    isc[hi8] |= (uint32_t)(uint8_t)(int8_t)sc << (8 * half);
                    mo[hi8] = __fmul_rn(__half2float(__ushort_as_half(mb)), (float)mi);
                }
            }
            w[half * 2 + hi8] = word;
        }
    }
    wq[idx] = make_uint4(w[0], w[1], w[2], w[3]);
    if (t == 0) {
        // two threads (sub-block 0 and 1) share each scale record: each writes its half
        uint16_t *dp = (uint16_t *)(ws + tile * 8 + g);
        dp[sb_in * 2 + 0] = (uint16_t)dsc[0]; dp[sb_in * 2 + 1] = (uint16_t)dsc[1];
        uint16_t *ip = (uint16_t *)(wd + tile * 8 + g);
        ip[0 * 2 + sb_in] = (uint16_t)isc[0]; ip[1 * 2 + sb_in] = (uint16_t)isc[1];
        if (wm) { float *mp = (float *)(wm + tile * 8 + g); mp[sb_in * 2 + 0] = mo[0]; mp[sb_in * 2 + 1] = mo[1]; }
    }
}

// ---------------------------------------------------------------------------------------------
// exact dequantisation of file-format rows (embedding gather; also the bit-exactness gate)
// ---------------------------------------------------------------------------------------------
// out[i][0..k) = scale * decode(row ids[i]) for q4_0 (type 2) / q4_K (type 12) / f32 (0) / f16 (1)
__global__ void lg_dequant_rows(const uint8_t *__restrict__ src, int type, int k, const int *__restrict__ ids,
                                int n_rows, int row0, float scale, float *__restrict__ out, int ldo) {
    pdl_launch(); pdl_wait();
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
    } else if (lg_fmt_is_i8(type)) {
        const int blk = lg_fmt_block(type), bytes = lg_fmt_bytes(type);
        const uint8_t *base = src + (size_t)row * (k / blk) * bytes;
        for (int e = threadIdx.x; e < k; e += blockDim.x) {
            int q, sc, mi; uint16_t db, mb;
            lg_fmt_elem(type, base + (size_t)(e / blk) * bytes, e % blk, &q, &sc, &db, &mb, &mi);
            float v = __fmul_rn(__fmul_rn(__half2float(__ushort_as_half(db)), (float)sc), (float)q);
            if (type == LG_T_Q5_K) v = __fsub_rn(v, __fmul_rn(__half2float(__ushort_as_half(mb)), (float)mi));
            o[e] = __fmul_rn(v, scale);
        }
    } else if (type == 30) {
        const unsigned short *h = (const unsigned short *)src + (size_t)row * k;      // bf16: the upper half of an f32
        for (int e = threadIdx.x; e < k; e += blockDim.x) o[e] = __fmul_rn(__uint_as_float((uint32_t)h[e] << 16), scale);
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
    __half *yh; int ldyh;                // optional f16 copy (input of the wide prompt matmul; single-CTA kernel only)
    int tag;                             // launch index for LG_STAMP (profiling builds)
    const int *skip;                     // optional: non-zero -> the launch does nothing (a draft that was called off)
};

struct LgGemvArgs {
    const uint4 *wq;           // tile-major nibbles
    const uint2 *ws;           // q4_0: 4 f16 scales per (tile, g); q4_K: 4 x (sc|mn<<8)
    const uint2 *wd;           // q4_K: {d,dmin} for rows g and g+8 per (tile, g); i8 tiles: 2 x 4 integer scales (rows g, g+8; 16-column groups)
    const uint4 *wm;           // LG_FMT_I8M: f32 offsets {row g sb0, row g+8 sb0, row g sb1, row g+8 sb1} per (tile, g)
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
    float *amax_val2;          // optional [gridDim.x][LG_MAXM] per-CTA second-best logit (the draft head's confidence margin)
    const int *skip;           // optional: non-zero -> the launch does nothing (a draft that was called off)
    int *err;
    // GeGLU epilogue: rows are interleaved (tile = 8 gate rows then the 8 matching up rows);
    // y = gelu_tanh(gate) * up goes straight into the next matmul's panel
    LgPanel outp;
    // cl_ks: the kslices CTAs of a row group are one thread-block cluster (1, kslices, 1); ranks > 0 send their partial
    // sums into rank 0's shared memory, so rank 0 holds the complete rows and runs the epilogue (one item per CTA)
    int cl_ks;
    // SUMS epilogue (complete rows only): besides out[tok][row], per item and token the four partial sums
    //   A = sum o^2,  B = sum x (w o),  C = sum (w o)^2,  D = sum x^2      (x = xres, the residual row; w = add_w)
    // from which the consumer forms 1/rms(o) and 1/rms(x + rmsnorm(o) w) without another pass over the row
    const float *xres; int ldx;
    const float *add_w; int n_cols;
    // GATE epilogue (R = 2: an item's 32 rows are one panel group; complete rows): y = gelu_tanh(out) * mul[tok][row] -> outp
    const float *mul; int ld_mul;
    float4 *sums;              // [LG_MAXM][LG_SUMS_ITEMS]: a token's partials lie side by side (one coalesced read for the consumer)
    int tag;                   // launch index for LG_STAMP (profiling builds)
    int ns;                    // ring stages (LG_GEMV_STAGES .. LG_GEMV_STAGES_MAX)
};

// Weight formats of the tile-major copies.  The two q4 formats keep 4 bits per weight.  Every other block format the
// reference reads (q8_0, q6_K, q5_K, q3_K) is expanded at load to "i8 tiles": one signed byte per weight (q8_0: the file's;
// the K formats: q - 32, q, q - 4.. as their decode defines them), the block scale d as f16 per (row, 32 columns), an
// integer scale per (row, 16 columns), and for q5_K (LG_FMT_I8M) the f32 offset dmin * m per (row, 32 columns); the decode
// (d * s) * q - m is the file's, bit for bit.  More bytes than the file for the K formats (1.125 B per weight against
// 0.82 for q6_K): the price of one kernel for all of them.
enum { LG_FMT_Q4_0 = 0, LG_FMT_Q4_K = 1, LG_FMT_I8 = 2, LG_FMT_I8M = 3 };
__host__ __device__ constexpr int lg_tile_bytes(int fmt) { return fmt >= LG_FMT_I8 ? 1024 : 512; }              // weights of one 16x64 tile
__host__ __device__ constexpr int lg_tile_extra(int fmt) { return fmt == LG_FMT_Q4_0 ? 64 : fmt == LG_FMT_I8M ? 256 : 128; }   // its scale bytes
enum { LG_EPI_STORE = 0, LG_EPI_HEAD = 1, LG_EPI_GEGLU = 2, LG_EPI_SUMS = 3, LG_EPI_GATE = 4 };
// partial sums one lane adds when a row's norms are assembled from per-item partials: 32 lanes x 10 cover 320 items
// (the host uses the SUMS epilogue only for matrices of at most that many items)
#define LG_SS_PER_LANE 10
#define LG_SUMS_ITEMS (32 * LG_SS_PER_LANE)
#define LG_GEMV_CL_MAX 8               // most k slices a cluster-reduced matmul may have (the portable cluster size)

#define LG_GEMV_CW 8                    // consumer warps per CTA
#define LG_GEMV_THREADS ((LG_GEMV_CW + 1) * 32)   // + one producer warp
#define LG_GEMV_STAGES 3               // ring depth: 3 stages, 4 (LG_GEMV_STAGES_MAX) where two CTAs per SM still fit
#define LG_GEMV_STAGES_MAX 4
#define LG_GEMV_STAGE_TILES 32         // 16x64 q4 weight tiles per stage (R row tiles x 32/R positions); i8 tiles: 16
template <int FMT> __host__ __device__ constexpr int gemv_stage_tiles() { return FMT >= LG_FMT_I8 ? 16 : LG_GEMV_STAGE_TILES; }

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumer_sync() {       // the consumer warps only; the producer warp never joins
    asm volatile("bar.sync 1, %0;" :: "n"(LG_GEMV_CW * 32) : "memory");
}

// Bytes of one ring stage: nibbles, scales (and the {d,dmin} pairs of q4_K)
template <int FMT> __host__ __device__ constexpr int gemv_stage_bytes() {
    return gemv_stage_tiles<FMT>() * (lg_tile_bytes(FMT) + lg_tile_extra(FMT));
}
__device__ __forceinline__ void mma_s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(b0));
}

// The small-M matmul.  A CTA walks items = (group of R consecutive row tiles) x (its k slice,
// blockIdx.y), item after item (blockIdx.x, +gridDim.x, ...).
//   * One producer thread streams the items' weight tiles HBM -> shared memory with bulk copies
//     (cp.async.bulk, TMA) into a ring of LG_GEMV_STAGES stages of 32 tiles (18 KB); each stage is
//     R row tiles x P = 32/R consecutive tile positions, completed on a "full" mbarrier and handed
//     back on an "empty" one.  The producer runs ahead of the consumers across item boundaries, so
//     up to 55 KB per CTA is in flight without occupying a single register.
//   * The activation panel slice is staged once per CTA by the same thread (after the first weight
//     stages are in flight -- they do not depend on the previous kernel).
//   * LG_GEMV_CW consumer warps split a stage's positions; for each position a warp reads the B
//     fragment once and applies it to the R row tiles: A fragments are one conflict-free 16-byte
//     shared load per lane, `mma.sync.m16n8k32.s8`, f32 scale-accumulate.  Partial sums of the
//     warps are added in warp order.
// Every wait is bounded; a timeout raises LG_ERR_MBAR_TIMEOUT and the kernel runs to its end.
//   * k slices (gridDim.y > 1) either leave one partial result per slice for the consumer to add, or -- cl_ks -- form
//     a thread-block cluster whose ranks 1.. send their sums into rank 0's shared memory (st.async, counted on an
//     mbarrier of rank 0), so that rank 0 runs the epilogue on complete rows.
// Dynamic shared memory: panel q | panel s | ring | warp partials | item sums | peers' sums (cluster) | mbarriers
template <int R, int NP, int FMT, int EPI>
__global__ void __launch_bounds__(LG_GEMV_THREADS)
lg_gemv_kernel(LgGemvArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int ST = gemv_stage_tiles<FMT>();
    constexpr int P = ST / R;                                // tile positions per stage
    constexpr int TB = lg_tile_bytes(FMT);
    // fewer positions than consumer warps (i8 tiles with R = 4): the warps also split the row tiles of a position
    constexpr int PW = P < LG_GEMV_CW ? P : LG_GEMV_CW, RS = LG_GEMV_CW / PW;
    const int NS = a.ns;                                     // ring depth chosen by the host (3 or 4)
    constexpr int EB = EPI;
    constexpr int RN = R * NP * 64;                          // outputs of one item: R row tiles x 16 rows x NP panels x 4 tokens
    constexpr int STAGE = gemv_stage_bytes<FMT>();
    constexpr int SC_OFF = ST * TB;                          // scales after the weights, {d,dmin} / integer scales after them, offsets last
    constexpr int DD_OFF = SC_OFF + ST * 64;
    constexpr int MM_OFF = DD_OFF + ST * 64;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int ks = blockIdx.y;
    const int kp0 = (int)((long long)a.nkp * ks / a.kslices), kp1 = (int)((long long)a.nkp * (ks + 1) / a.kslices);
    const int nkp_s = kp1 - kp0, nsb_s = nkp_s * 2;
    const int n_chunks = (nkp_s + P - 1) / P;
    const int n_groups = (a.n_row_tiles + R - 1) / R;
    const bool cl = a.cl_ks != 0;                            // cluster (1, kslices, 1): cluster rank == blockIdx.y

    int8_t *sq = (int8_t *)smem;
    float2 *ss = (float2 *)(smem + (size_t)NP * nsb_s * 256);
    unsigned char *ring = (unsigned char *)(ss + (size_t)NP * nsb_s * 4);
    ring = (unsigned char *)(((uintptr_t)ring + 127) & ~(uintptr_t)127);
    float *red = (float *)(ring + (size_t)NS * STAGE);
    float *fin = red + LG_GEMV_CW * RN;                      // [RN] complete sums of the item (GeGLU, SUMS)
    float *cred = fin + RN;                                  // cluster reduce: [kslices - 1][RN] partials of ranks 1.. (rank 0's copy is used)
    uint64_t *full = (uint64_t *)(cred + (cl ? (a.kslices - 1) * RN : 0));
    uint64_t *empty = full + NS, *pbar = empty + NS, *cbar = pbar + 1;

    pdl_launch();
    LG_STAMP(a.tag, 0);
    LG_STAMP_KIND(a.tag, 1 + EB);
    if (threadIdx.x == 0) {
        for (int i = 0; i < NS; i++) { mbar_init(full + i, 1); mbar_init(empty + i, LG_GEMV_CW); }
        mbar_init(pbar, 1);
        mbar_init(cbar, 1);
        // rank 0 of a cluster expects every peer's RN partial sums (once: a cluster-reduced launch has one item per CTA)
        if (cl && ks == 0) mbar_expect_tx(cbar, (uint32_t)(a.kslices - 1) * RN * 4);
    }
    __syncthreads();
    // no peer may send before the receiving barrier exists: every thread arrives at the cluster barrier here; the consumer
    // warps complete it (wait) only just before the exchange, microseconds later, so the start of the kernel does not stall
    if (cl) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");

    if (warp == LG_GEMV_CW) {
        // ---------------- producer ----------------
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0; bool panel_sent = false, ok = true;
            // stages this CTA will stream in all, and how many of them go out before the dependency wait: a full ring
            const int my_groups = blockIdx.x < n_groups ? (n_groups - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
            const int total_stages = my_groups * n_chunks, early = min(NS, total_stages);
            int issued = 0;
            for (int grp = blockIdx.x; grp < n_groups && ok; grp += gridDim.x) {
                const size_t tile_base = (size_t)grp * R * a.nkp + kp0;
                for (int c = 0; c < n_chunks && ok; c++) {
                    if (!mbar_wait(empty + stage, phase ^ 1)) { atomicOr(a.err, LG_ERR_MBAR_TIMEOUT); ok = false; break; }
                    const int np = min(P, nkp_s - c * P);
                    const uint32_t tile_bytes = (uint32_t)np * (TB + lg_tile_extra(FMT));
                    unsigned char *st = ring + (size_t)stage * STAGE;
                    mbar_expect_tx(full + stage, R * tile_bytes);
                    #pragma unroll
                    for (int r = 0; r < R; r++) {
                        const size_t tile = tile_base + (size_t)r * a.nkp + (size_t)c * P;
                        bulk_g2s(st + (size_t)r * P * TB, a.wq + tile * (TB / 16), (uint32_t)np * TB, full + stage);
                        bulk_g2s(st + SC_OFF + (size_t)r * P * 64, a.ws + tile * 8, (uint32_t)np * 64, full + stage);
                        if (FMT != LG_FMT_Q4_0)
                            bulk_g2s(st + DD_OFF + (size_t)r * P * 64, a.wd + tile * 8, (uint32_t)np * 64, full + stage);
                        if (FMT == LG_FMT_I8M)
                            bulk_g2s(st + MM_OFF + (size_t)r * P * 128, a.wm + tile * 8, (uint32_t)np * 128, full + stage);
                    }
                    if (++stage == NS) { stage = 0; phase ^= 1; }
                    if (!panel_sent && ++issued == early) {
                        // a ring of weights is in flight; now the activations, which the previous kernel produced
                        pdl_wait();
                        if (a.skip && *a.skip) {
                            // called off: let the copies already in flight land (shared memory must not be released under
                            // them), then leave; the consumers have left on the same word
                            for (int i = 0; i < issued; i++) mbar_wait(full + (i % NS), 0);
                            ok = false;
                            break;
                        }
                        uint32_t qb = (uint32_t)nsb_s * 256, sb = (uint32_t)nsb_s * 32;
                        mbar_expect_tx(pbar, NP * (qb + sb));
                        #pragma unroll
                        for (int p = 0; p < NP; p++) {
                            bulk_g2s(sq + (size_t)p * qb, a.x.q + ((size_t)p * a.x.nsb + kp0 * 2) * 256, qb, pbar);
                            bulk_g2s(ss + (size_t)p * nsb_s * 4, a.x.s + ((size_t)p * a.x.nsb + kp0 * 2) * 4, sb, pbar);
                        }
                        panel_sent = true;
                    }
                }
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    constexpr int CT = LG_GEMV_CW * 32;
    constexpr int SLOTS = (RN + CT - 1) / CT;
    float best_v[SLOTS], sec_v[SLOTS]; int best_i[SLOTS];
    #pragma unroll
    for (int j = 0; j < SLOTS; j++) { best_v[j] = -INFINITY; sec_v[j] = -INFINITY; best_i[j] = 0x7fffffff; }

    pdl_wait();
    LG_STAMP(a.tag, 1);
    if (a.skip && *a.skip) return;
    bool ok = mbar_wait(pbar, 0);
    if (!ok && threadIdx.x == 0) atomicOr(a.err, LG_ERR_MBAR_TIMEOUT);
    LG_STAMP(a.tag, 2);
    int stage = 0; uint32_t phase = 0;

    for (int grp = blockIdx.x; grp < n_groups; grp += gridDim.x) {
        const int rt0 = grp * R;
        // SUMS: this thread's residual elements and norm weights, fetched now and used after the main loop
        float x_v[SLOTS], w_v[SLOTS];
        if (EB == LG_EPI_SUMS && ks == 0) {
            #pragma unroll
            for (int j = 0; j < SLOTS; j++) {
                const int idx = threadIdx.x + j * CT;
                const int rp = idx >> 6, r = rp / NP, p = rp % NP, tok = p * 4 + ((idx >> 4) & 3), row = (rt0 + r) * 16 + (idx & 15);
                const bool live = idx < RN && tok < a.M && row < a.n_cols;
                x_v[j] = live ? __ldcg(a.xres + (size_t)tok * a.ldx + row) : 0.0f;
                w_v[j] = live ? a.add_w[row] : 0.0f;
            }
        }
        float acc[R][NP][2];
        #pragma unroll
        for (int r = 0; r < R; r++)
            #pragma unroll
            for (int p = 0; p < NP; p++) acc[r][p][0] = acc[r][p][1] = 0.0f;

        for (int c = 0; c < n_chunks; c++) {
            if (ok && !mbar_wait(full + stage, phase)) { ok = false; if (lane == 0) atomicOr(a.err, LG_ERR_MBAR_TIMEOUT); }
            const int np = min(P, nkp_s - c * P);
            const unsigned char *st = ring + (size_t)stage * STAGE;
            for (int pp = warp % PW; pp < np; pp += PW) {
                uint2 b[2][NP]; float2 xs[2][NP];
                #pragma unroll
                for (int s = 0; s < 2; s++)
                    #pragma unroll
                    for (int p = 0; p < NP; p++) {
                        const int sbl = (c * P + pp) * 2 + s;
                        b[s][p] = *(const uint2 *)(sq + ((size_t)p * nsb_s + sbl) * 256 + lane * 8);
                        xs[s][p] = ss[((size_t)p * nsb_s + sbl) * 4 + t];
                    }
                #pragma unroll
                for (int r = 0; r < R; r++) {
                    if (RS > 1 && (r % RS) != warp / PW) continue;          // another warp's row tile
                    if (FMT >= LG_FMT_I8) {
                        // i8 tile: per sub-block this lane's 16 bytes are {row g, row g+8} x {columns 4t.., 16+4t..}; one
                        // k16 MMA per 16-column group, whose integer scale joins the block's f16 d (x16: the common
                        // epilogue divides by the 16 the q4 tiles carry)
                        const unsigned char *tp = st + (size_t)(r * P + pp) * TB;
                        const uint2 sw2 = *(const uint2 *)(st + SC_OFF + (size_t)(r * P + pp) * 64 + g * 8);
                        const uint2 is2 = *(const uint2 *)(st + DD_OFF + (size_t)(r * P + pp) * 64 + g * 8);
                        uint4 mm = make_uint4(0, 0, 0, 0);
                        if (FMT == LG_FMT_I8M) mm = *(const uint4 *)(st + MM_OFF + (size_t)(r * P + pp) * 128 + g * 16);
                        #pragma unroll
                        for (int s = 0; s < 2; s++) {
                            const uint4 w = *(const uint4 *)(tp + s * 512 + lane * 16);
                            const float2 fd = __half22float2(*(const __half2 *)(s ? &sw2.y : &sw2.x));
                            #pragma unroll
                            for (int h = 0; h < 2; h++) {
                                const int i0 = (int)(int8_t)((is2.x >> (8 * (2 * s + h))) & 0xff), i1 = (int)(int8_t)((is2.y >> (8 * (2 * s + h))) & 0xff);
                                const float e0 = 16.0f * __fmul_rn(fd.x, (float)i0), e1 = 16.0f * __fmul_rn(fd.y, (float)i1);
                                #pragma unroll
                                for (int p = 0; p < NP; p++) {
                                    int cc[4] = {0, 0, 0, 0};
                                    mma_s8_k16(cc, h ? w.z : w.x, h ? w.w : w.y, h ? b[s][p].y : b[s][p].x);
                                    const float v0 = (float)((cc[0] << 8) + cc[1]) * xs[s][p].x;
                                    const float v1 = (float)((cc[2] << 8) + cc[3]) * xs[s][p].x;
                                    acc[r][p][0] = fmaf(v0, e0, acc[r][p][0]);
                                    acc[r][p][1] = fmaf(v1, e1, acc[r][p][1]);
                                }
                            }
                            if (FMT == LG_FMT_I8M) {
                                const float m0 = -16.0f * __uint_as_float(s ? mm.z : mm.x), m1 = -16.0f * __uint_as_float(s ? mm.w : mm.y);
                                #pragma unroll
                                for (int p = 0; p < NP; p++) {
                                    acc[r][p][0] = fmaf(m0, xs[s][p].y, acc[r][p][0]);
                                    acc[r][p][1] = fmaf(m1, xs[s][p].y, acc[r][p][1]);
                                }
                            }
                        }
                        continue;
                    }
                    // this lane's 16 bytes: {row g, row g+8} words of sub-block 0, then of sub-block 1
                    const uint4 w = *(const uint4 *)(st + (size_t)(r * P + pp) * 512 + lane * 16);
                    const uint2 sw2 = *(const uint2 *)(st + SC_OFF + (size_t)(r * P + pp) * 64 + g * 8);
                    uint2 dd = make_uint2(0, 0);
                    if (FMT == LG_FMT_Q4_K) dd = *(const uint2 *)(st + DD_OFF + (size_t)(r * P + pp) * 64 + g * 8);
                    #pragma unroll
                    for (int s = 0; s < 2; s++) {
                        const uint32_t wg = s ? w.z : w.x, wh = s ? w.w : w.y, sw = s ? sw2.y : sw2.x;
                        uint32_t a0 = (wg << 4) & 0xF0F0F0F0u, a2 = wg & 0xF0F0F0F0u;
                        uint32_t a1 = (wh << 4) & 0xF0F0F0F0u, a3 = wh & 0xF0F0F0F0u;
                        float d0, d1, m0 = 0.0f, m1 = 0.0f;
                        if (FMT == LG_FMT_Q4_0) {
                            float2 fd = __half22float2(*(const __half2 *)&sw);
                            d0 = fd.x; d1 = fd.y;
                        } else {
                            float2 r0 = __half22float2(*(const __half2 *)&dd.x), r1 = __half22float2(*(const __half2 *)&dd.y);
                            d0 = r0.x * (float)(sw & 0xff); m0 = 16.0f * (8.0f * d0 - r0.y * (float)((sw >> 8) & 0xff));
                            d1 = r1.x * (float)((sw >> 16) & 0xff); m1 = 16.0f * (8.0f * d1 - r1.y * (float)(sw >> 24));
                        }
                        #pragma unroll
                        for (int p = 0; p < NP; p++) {
                            int cc[4] = {0, 0, 0, 0};
                            mma_s8(cc, a0, a1, a2, a3, b[s][p].x, b[s][p].y);
                            float v0 = (float)((cc[0] << 8) + cc[1]) * xs[s][p].x;      // row g,   token 4p+t
                            float v1 = (float)((cc[2] << 8) + cc[3]) * xs[s][p].x;      // row g+8
                            acc[r][p][0] = fmaf(v0, d0, acc[r][p][0]);
                            acc[r][p][1] = fmaf(v1, d1, acc[r][p][1]);
                            if (FMT == LG_FMT_Q4_K) {     // nibbles are stored as (q-8): add back (8 d sc - dmin m) * sum(x)
                                acc[r][p][0] = fmaf(m0, xs[s][p].y, acc[r][p][0]);
                                acc[r][p][1] = fmaf(m1, xs[s][p].y, acc[r][p][1]);
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + stage);
            if (++stage == NS) { stage = 0; phase ^= 1; }
        }

        LG_STAMP(a.tag, 3);
        // the consumer warps' partial sums, added in warp order; output idx = ((r NP + p) 4 + token) 16 + row
        #pragma unroll
        for (int r = 0; r < R; r++)
            #pragma unroll
            for (int p = 0; p < NP; p++) {
                red[(warp * R * NP + r * NP + p) * 64 + t * 16 + g] = acc[r][p][0];
                red[(warp * R * NP + r * NP + p) * 64 + t * 16 + g + 8] = acc[r][p][1];
            }
        consumer_sync();
        float fs[SLOTS];
        #pragma unroll
        for (int j = 0; j < SLOTS; j++) {
            const int idx = threadIdx.x + j * CT;
            float sum = 0.0f;
            if (idx < RN) {
                #pragma unroll
                for (int w2 = 0; w2 < LG_GEMV_CW; w2++) sum += red[w2 * RN + idx];
            }
            fs[j] = sum;
        }
        if (cl) {
            // k slices of one cluster: ranks 1.. send their sums to rank 0 and are done with the item; rank 0 adds them in
            // rank order once every byte has arrived (bounded wait)
            asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
            if (ks != 0) {
                #pragma unroll
                for (int j = 0; j < SLOTS; j++) {
                    const int idx = threadIdx.x + j * CT;
                    if (idx < RN) dsmem_st_async_f32(cred + (size_t)(ks - 1) * RN + idx, cbar, 0, fs[j]);
                }
                consumer_sync();
                continue;
            }
            // (waited for even after an earlier timeout: this CTA must not leave while peers still send into it)
            if (!mbar_wait_cluster(cbar, 0)) { ok = false; if (lane == 0) atomicOr(a.err, LG_ERR_MBAR_TIMEOUT); }
            LG_STAMP(a.tag, 4);
            #pragma unroll
            for (int j = 0; j < SLOTS; j++) {
                const int idx = threadIdx.x + j * CT;
                if (idx < RN)
                    for (int r2 = 1; r2 < a.kslices; r2++) fs[j] += cred[(size_t)(r2 - 1) * RN + idx];
            }
        }
        if (EB == LG_EPI_GEGLU) {
            #pragma unroll
            for (int j = 0; j < SLOTS; j++) {
                const int idx = threadIdx.x + j * CT;
                if (idx < RN) fin[idx] = fs[j];
            }
            consumer_sync();
            // one warp per token: lane o = output (r, row8) of this item's 32 outputs
            for (int tok = warp; tok < NP * 4 && tok < a.M; tok += LG_GEMV_CW) {
                const int p = tok >> 2, tl = tok & 3, row8 = lane & 7;
                #pragma unroll
                for (int rh = 0; rh < R / 4; rh++) {
                    const int r = rh * 4 + (lane >> 3);
                    const int ig = ((r * NP + p) * 4 + tl) * 16 + row8;
                    const float gate = fin[ig], up = fin[ig + 8];
                    float y = __fmul_rn(gelu_tanh(gate * 0.0625f), up * 0.0625f);
                    quant_group_store(y, lane, tok, rt0 / 4 + rh, a.outp);
                }
            }
        } else if (EB == LG_EPI_GATE) {
            #pragma unroll
            for (int j = 0; j < SLOTS; j++) {
                const int idx = threadIdx.x + j * CT;
                if (idx < RN) fin[idx] = fs[j];
            }
            consumer_sync();
            // one warp per token: lane = row of the item's 32 rows (R = 2)
            for (int tok = warp; tok < NP * 4 && tok < a.M; tok += LG_GEMV_CW) {
                const int p = tok >> 2, tl = tok & 3, r = lane >> 4, row = (rt0 + r) * 16 + (lane & 15);
                const float gv = fin[((r * NP + p) * 4 + tl) * 16 + (lane & 15)] * 0.0625f;
                const float mv = row < a.n_valid_rows ? a.mul[(size_t)tok * a.ld_mul + row] : 0.0f;
                quant_group_store(__fmul_rn(gelu_tanh(gv), mv), lane, tok, rt0 / 2, a.outp);
            }
        } else {
            float4 part[SLOTS];
            #pragma unroll
            for (int j = 0; j < SLOTS; j++) {
                int idx = threadIdx.x + j * CT;
                part[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (idx < RN) {
                    int rp = idx >> 6, r = rp / NP, p = rp % NP, tok = p * 4 + ((idx >> 4) & 3);
                    float sum = fs[j] * 0.0625f;
                    int row = (rt0 + r) * 16 + (idx & 15);
                    if (rt0 + r < a.n_row_tiles && tok < a.M) {
                        if (EB == LG_EPI_STORE || EB == LG_EPI_SUMS) {
                            a.out[((size_t)ks * LG_MAXM + tok) * a.ldo + row] = sum;
                            if (EB == LG_EPI_SUMS && row < a.n_cols) {
                                const float wo = __fmul_rn(w_v[j], sum);
                                part[j] = make_float4(__fmul_rn(sum, sum), __fmul_rn(x_v[j], wo), __fmul_rn(wo, wo), __fmul_rn(x_v[j], x_v[j]));
                            }
                        } else if (row < a.n_valid_rows) {
                            if (a.softcap > 0.0f) sum = a.softcap * tanhf(sum / a.softcap);
                            if (a.logits) a.logits[(size_t)tok * a.ldo + row] = sum;
                            if (sum > best_v[j]) { sec_v[j] = best_v[j]; best_v[j] = sum; best_i[j] = row; }   // rows ascend per slot: first max wins
                            else if (sum > sec_v[j]) sec_v[j] = sum;
                        }
                    }
                }
            }
            if (EB == LG_EPI_SUMS) {
                // the item's four sums per token: 16 rows of one (row tile, token) lie in one half warp (xor tree), then
                // the row tiles in ascending order
                float4 *hs = (float4 *)fin;                     // [R NP 4] one entry per (row tile, panel, token)
                #pragma unroll
                for (int j = 0; j < SLOTS; j++) {
                    float4 v = part[j];
                    #pragma unroll
                    for (int o = 8; o > 0; o >>= 1) {
                        v.x += __shfl_xor_sync(0xffffffffu, v.x, o); v.y += __shfl_xor_sync(0xffffffffu, v.y, o);
                        v.z += __shfl_xor_sync(0xffffffffu, v.z, o); v.w += __shfl_xor_sync(0xffffffffu, v.w, o);
                    }
                    const int idx = threadIdx.x + j * CT;
                    if (idx < RN && (idx & 15) == 0) hs[idx >> 4] = v;
                }
                consumer_sync();
                if (threadIdx.x < a.M) {
                    const int tok = threadIdx.x, p = tok >> 2, tl = tok & 3;
                    float4 tot = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    #pragma unroll
                    for (int r = 0; r < R; r++) {
                        const float4 v = hs[(r * NP + p) * 4 + tl];
                        tot.x += v.x; tot.y += v.y; tot.z += v.z; tot.w += v.w;
                    }
                    a.sums[(size_t)tok * LG_SUMS_ITEMS + grp] = tot;
                }
            }
        }
        consumer_sync();
        LG_STAMP(a.tag, 6);
    }

    if (EB == LG_EPI_HEAD) {
        // candidates of this CTA: one per (slot, thread); merge per token (larger value, lower index on ties)
        float *cv = red; int *ci = (int *)(red + RN); float *c2 = red + 2 * RN;
        #pragma unroll
        for (int j = 0; j < SLOTS; j++) {
            int idx = threadIdx.x + j * CT;
            if (idx < RN) { cv[idx] = best_v[j]; ci[idx] = best_i[j]; c2[idx] = sec_v[j]; }
        }
        consumer_sync();
        if (threadIdx.x < a.M) {
            int tok = threadIdx.x, p = tok >> 2, tl = tok & 3;
            float bv = -INFINITY, s2 = -INFINITY; int bi = 0x7fffffff;
            for (int r = 0; r < R; r++)
                for (int row = 0; row < 16; row++) {
                    int idx = ((r * NP + p) * 4 + tl) * 16 + row;
                    float v = cv[idx]; int i2 = ci[idx];
                    if (v > bv || (v == bv && i2 < bi)) { s2 = fmaxf(s2, bv); bv = v; bi = i2; }
                    else s2 = fmaxf(s2, v);
                    s2 = fmaxf(s2, c2[idx]);
                }
            a.amax_val[(size_t)blockIdx.x * LG_MAXM + tok] = bv;
            a.amax_idx[(size_t)blockIdx.x * LG_MAXM + tok] = bi;
            if (a.amax_val2) a.amax_val2[(size_t)blockIdx.x * LG_MAXM + tok] = s2;
        }
    }
}

// Merge the per-CTA argmax candidates: out[tok] = index of the largest logit, lowest index on ties.
// With val2 / margin: also the runner-up's value, margin[tok] = best - second best logit (the draft head's confidence).
__device__ __forceinline__ void top2_merge(float &bv, int &bi, float &s2, float ov, int oi, float o2) {
    if (ov > bv || (ov == bv && oi < bi)) { s2 = fmaxf(s2, bv); bv = ov; bi = oi; }
    else s2 = fmaxf(s2, ov);
    s2 = fmaxf(s2, o2);
}
// Block-wide merge of the per-CTA candidates of token `tok`; the result is valid in thread 0.
__device__ __forceinline__ void argmax_block(const float *__restrict__ val, const int *__restrict__ idx, int n_parts, int tok,
                                             const float *__restrict__ val2, float &bv, int &bi, float &s2) {
    bv = -INFINITY; s2 = -INFINITY; bi = 0x7fffffff;
    for (int i = threadIdx.x; i < n_parts; i += blockDim.x)
        top2_merge(bv, bi, s2, val[(size_t)i * LG_MAXM + tok], idx[(size_t)i * LG_MAXM + tok], val2 ? val2[(size_t)i * LG_MAXM + tok] : -INFINITY);
    __shared__ float sv[32], sv2[32]; __shared__ int si[32];
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o), o2 = __shfl_xor_sync(0xffffffffu, s2, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        top2_merge(bv, bi, s2, ov, oi, o2);
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; sv2[threadIdx.x >> 5] = s2; }
    __syncthreads();
    if (threadIdx.x < 32) {
        int nw = blockDim.x >> 5;
        bv = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY; bi = threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
        s2 = threadIdx.x < nw ? sv2[threadIdx.x] : -INFINITY;
        #pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, o), o2 = __shfl_xor_sync(0xffffffffu, s2, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            top2_merge(bv, bi, s2, ov, oi, o2);
        }
    }
}
__global__ void lg_argmax_final(const float *__restrict__ val, const int *__restrict__ idx, int n_parts, int *out,
                                const float *__restrict__ val2, float *__restrict__ margin) {
    pdl_launch(); pdl_wait();
    int tok = blockIdx.x;
    float bv, s2; int bi;
    argmax_block(val, idx, n_parts, tok, val2, bv, bi, s2);
    if (threadIdx.x == 0) {
        out[tok] = bi == 0x7fffffff ? 0 : bi;
        if (margin) margin[tok] = bv - s2;
    }
}

// ---------------------------------------------------------------------------------------------
// embedding gather
// ---------------------------------------------------------------------------------------------
// x[tok][0..ne) = decode(token_embd row toks[tok]) * sqrt(ne) from the TILE-MAJOR copy (the same
// matrix is the output head).  Bit-identical to decoding the file row: value = d * (nibble-8).
// Element e of matrix row `row` from the tile-major copy: the file's decode, bit for bit.
__device__ __forceinline__ float lg_tile_value(const uint4 *__restrict__ wq, const uint2 *__restrict__ ws, const uint2 *__restrict__ wd,
                                               const uint4 *__restrict__ wm, int fmt, int nkp, int row, int e) {
    const int rt = row >> 4, r = row & 15, g = r & 7, hi8 = r >> 3;
    const int kp = e >> 6, s = (e >> 5) & 1, kk = e & 31;
    const size_t tile = (size_t)rt * nkp + kp;
    if (fmt >= LG_FMT_I8) {
        // i8 tiles: value = (d * s) * q - m
        const int half = kk >> 4, t = (kk & 15) >> 2, i = kk & 3;
        const int q = ((const int8_t *)wq)[tile * 1024 + (size_t)s * 512 + (g * 4 + t) * 16 + (half * 2 + hi8) * 4 + i];
        const uint16_t db = ((const uint16_t *)(ws + tile * 8 + g))[s * 2 + hi8];
        const int sc = ((const int8_t *)(wd + tile * 8 + g))[hi8 * 4 + s * 2 + half];
        float v = __fmul_rn(__fmul_rn(__half2float(__ushort_as_half(db)), (float)sc), (float)q);
        if (fmt == LG_FMT_I8M) v = __fsub_rn(v, ((const float *)(wm + tile * 8 + g))[s * 2 + hi8]);
        return v;
    }
    const int t = (kk & 15) >> 2, i = kk & 3;
    const uint32_t word = ((const uint32_t *)wq)[(tile * 32 + g * 4 + t) * 4 + s * 2 + hi8];
    const int nib = (word >> (8 * i + (kk >> 4) * 4)) & 15;
    const int qv = (nib ^ 8) - 8;                               // stored two's complement of (q-8)
    const uint2 sc = ws[tile * 8 + g];
    const uint32_t sw = s ? sc.y : sc.x;
    if (fmt == LG_FMT_Q4_0) {
        const float d = __half2float(__ushort_as_half((unsigned short)(hi8 ? (sw >> 16) : (sw & 0xffff))));
        return __fmul_rn(d, (float)qv);
    }
    const uint2 dd = wd[tile * 8 + g];
    const uint32_t dw = hi8 ? dd.y : dd.x;
    const float d = __half2float(__ushort_as_half((unsigned short)(dw & 0xffff)));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(dw >> 16)));
    const uint32_t sm = hi8 ? (sw >> 16) : (sw & 0xffff);
    return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)(sm & 0xff)), (float)(qv + 8)), __fmul_rn(dmin, (float)(sm >> 8)));
}
__global__ void lg_embed_rows(const uint4 *__restrict__ wq, const uint2 *__restrict__ ws, const uint2 *__restrict__ wd,
                              const uint4 *__restrict__ wm, int fmt, int nkp, int n_rows, const int *__restrict__ toks, float scale,
                              float *__restrict__ out, int ldo) {
    pdl_launch(); pdl_wait();
    const int tok = blockIdx.x;
    const int row = min(max(toks[tok], 0), n_rows - 1);         // an out-of-range id must not read outside the table
    for (int e = threadIdx.x; e < nkp * 64; e += blockDim.x)
        out[(size_t)tok * ldo + e] = __fmul_rn(lg_tile_value(wq, ws, wd, wm, fmt, nkp, row, e), scale);
}

// ---------------------------------------------------------------------------------------------
// norms
// ---------------------------------------------------------------------------------------------
__global__ void lg_norm_kernel(LgNormArgs a) {
    pdl_launch(); pdl_wait();
    if (a.skip && *a.skip) return;
    extern __shared__ float row[];       // 2n floats + 32
    float *rowx = row + a.n, *red = rowx + a.n;
    const int tok = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float *x = a.x + (size_t)tok * a.ldx;
    float ss2 = 0.0f;
    if (a.add_src) {
        // the partial sums and the residual row are fetched together (one memory latency)
        float ss = 0.0f;
        for (int i = threadIdx.x; i < a.n; i += blockDim.x) {
            float v = 0.0f;
            for (int p = 0; p < a.n_parts; p++) v += a.add_src[(size_t)p * a.part_stride + (size_t)tok * a.ld_add + i];
            rowx[i] = x[i];
            row[i] = v;
            ss += v * v;
        }
        ss = block_sum(ss, red);
        float s = 1.0f / sqrtf(ss / (float)a.n + a.eps);
        for (int i = threadIdx.x; i < a.n; i += blockDim.x) {
            float v = __fadd_rn(rowx[i], __fmul_rn(__fmul_rn(row[i], s), a.add_w[i]));
            v = __fmul_rn(v, a.out_scale);
            x[i] = v;
            row[i] = v;
            ss2 += v * v;
        }
    } else {
        for (int i = threadIdx.x; i < a.n; i += blockDim.x) { float v = x[i]; row[i] = v; ss2 += v * v; }
    }
    if (!a.norm_w && !a.want_panel && !a.y && !a.yh) return;
    float s = 1.0f;
    if (a.norm_w) {
        ss2 = block_sum(ss2, red);
        s = 1.0f / sqrtf(ss2 / (float)a.n + a.eps);
    } else {
        __syncthreads();
    }
    for (int sb = warp; sb * 32 < a.n; sb += nw) {
        int i = sb * 32 + lane;
        float yv = a.norm_w ? __fmul_rn(__fmul_rn(row[i], s), a.norm_w[i]) : row[i];   // no norm_w: the row itself
        if (a.y) a.y[(size_t)tok * a.ldy + i] = yv;
        if (a.yh) a.yh[(size_t)tok * a.ldyh + i] = __float2half_rn(yv);
        if (a.want_panel) quant_group_store(yv, lane, tok, sb, a.panel);
    }
}

// ---- the same norm spread over a thread-block cluster ------------------------------------------
// One cluster of LG_NORM_CL CTAs per token row; CTA r owns a contiguous run of 32-element groups.
// The two sums of squares are exchanged through distributed shared memory (every CTA writes its
// partial into slot r of every peer, then the slots are added in rank order), so a row's result is
// fixed by (n, LG_NORM_CL) alone.  Shortens the latency chain of the single-CTA kernel: each CTA
// touches 1/8 of the row and the whole row is in flight at once.
#define LG_NORM_CL 8
#define LG_NORM_CL_THREADS 128
#define LG_NORM_CL_EPT 4               // row elements per thread the batched-load path holds in registers (rows up to 4096)


__global__ void __launch_bounds__(LG_NORM_CL_THREADS) lg_norm_cluster_kernel(LgNormArgs a) {
    extern __shared__ float row[];                       // this CTA's run of the row, then the two weight runs (3 * gpc*32 floats)
    __shared__ float slots[2][LG_NORM_CL];               // partial sums of squares of every rank, two rounds
    __shared__ float red[32];
    const uint32_t rank = cluster_rank();
    const int tok = blockIdx.x / LG_NORM_CL, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = LG_NORM_CL_THREADS / 32;
    const int ng = a.n >> 5, gpc = (ng + LG_NORM_CL - 1) / LG_NORM_CL;
    const int g0 = rank * gpc, g1 = min(ng, g0 + gpc), i0 = g0 * 32, cnt = max(0, (g1 - g0) * 32);
    float *wa = row + gpc * 32, *wn = wa + gpc * 32;
    // the norm weights do not depend on the previous kernel (and are cold in HBM): fetch them first
    pdl_launch();
    for (int j = threadIdx.x; j < cnt; j += LG_NORM_CL_THREADS) {
        if (a.add_src) wa[j] = a.add_w[i0 + j];
        if (a.norm_w) wn[j] = a.norm_w[i0 + j];
    }
    LG_STAMP(a.tag, 0);
    LG_STAMP_KIND(a.tag, 7);
    pdl_wait();
    LG_STAMP(a.tag, 1);
    if (a.skip && *a.skip) return;                       // the whole cluster leaves on the same word: nobody waits at a cluster barrier
    float *x = a.x + (size_t)tok * a.ldx;
    float ss2 = 0.0f;
    if (a.add_src && cnt <= LG_NORM_CL_EPT * LG_NORM_CL_THREADS && a.n_parts <= 4) {
        // every load of this thread -- the k-slice partials and the residual elements -- is issued before the first use,
        // so the chain after the dependency wait holds ONE memory latency instead of one per partial and one for x
        float pv[LG_NORM_CL_EPT][4], xv[LG_NORM_CL_EPT];
        #pragma unroll
        for (int u = 0; u < LG_NORM_CL_EPT; u++) {
            const int j = threadIdx.x + u * LG_NORM_CL_THREADS;
            #pragma unroll
            for (int p = 0; p < 4; p++)
                pv[u][p] = (j < cnt && p < a.n_parts) ? __ldcg(a.add_src + (size_t)p * a.part_stride + (size_t)tok * a.ld_add + i0 + j) : 0.0f;
            xv[u] = j < cnt ? __ldcg(x + i0 + j) : 0.0f;
        }
        float ss = 0.0f, sv[LG_NORM_CL_EPT];
        #pragma unroll
        for (int u = 0; u < LG_NORM_CL_EPT; u++) {
            float v = 0.0f;
            #pragma unroll
            for (int p = 0; p < 4; p++) v += pv[u][p];           // p >= n_parts adds an exact zero: the order of the sum is that of the loop form
            sv[u] = v;
            ss += v * v;
        }
        ss = block_sum(ss, red);
        if (threadIdx.x < LG_NORM_CL) dsmem_store(&slots[0][rank], threadIdx.x, ss);
        cluster_sync_all();
        float tot = 0.0f;
        #pragma unroll
        for (int r = 0; r < LG_NORM_CL; r++) tot += slots[0][r];
        const float s = 1.0f / sqrtf(tot / (float)a.n + a.eps);
        #pragma unroll
        for (int u = 0; u < LG_NORM_CL_EPT; u++) {
            const int j = threadIdx.x + u * LG_NORM_CL_THREADS;
            if (j < cnt) {
                float v = __fadd_rn(xv[u], __fmul_rn(__fmul_rn(sv[u], s), wa[j]));
                v = __fmul_rn(v, a.out_scale);
                x[i0 + j] = v;
                row[j] = v;
                ss2 += v * v;
            }
        }
    } else if (a.add_src) {
        float ss = 0.0f;
        for (int j = threadIdx.x; j < cnt; j += LG_NORM_CL_THREADS) {
            const int i = i0 + j;
            float v = 0.0f;
            for (int p = 0; p < a.n_parts; p++) v += a.add_src[(size_t)p * a.part_stride + (size_t)tok * a.ld_add + i];
            row[j] = v;
            ss += v * v;
        }
        ss = block_sum(ss, red);
        if (threadIdx.x < LG_NORM_CL) dsmem_store(&slots[0][rank], threadIdx.x, ss);
        cluster_sync_all();
        float tot = 0.0f;
        #pragma unroll
        for (int r = 0; r < LG_NORM_CL; r++) tot += slots[0][r];
        const float s = 1.0f / sqrtf(tot / (float)a.n + a.eps);
        for (int j = threadIdx.x; j < cnt; j += LG_NORM_CL_THREADS) {
            const int i = i0 + j;
            float v = __fadd_rn(x[i], __fmul_rn(__fmul_rn(row[j], s), wa[j]));
            v = __fmul_rn(v, a.out_scale);
            x[i] = v;
            row[j] = v;
            ss2 += v * v;
        }
    } else {
        for (int j = threadIdx.x; j < cnt; j += LG_NORM_CL_THREADS) { float v = x[i0 + j]; row[j] = v; ss2 += v * v; }
    }
    if (!a.norm_w && !a.want_panel && !a.y) return;
    float s = 1.0f;
    if (a.norm_w) {
        ss2 = block_sum(ss2, red);
        if (threadIdx.x < LG_NORM_CL) dsmem_store(&slots[1][rank], threadIdx.x, ss2);
        cluster_sync_all();
        float tot = 0.0f;
        #pragma unroll
        for (int r = 0; r < LG_NORM_CL; r++) tot += slots[1][r];
        s = 1.0f / sqrtf(tot / (float)a.n + a.eps);
    } else {
        __syncthreads();
    }
    for (int gq = g0 + warp; gq < g1; gq += nw) {
        const int i = gq * 32 + lane;
        float yv = a.norm_w ? __fmul_rn(__fmul_rn(row[i - i0], s), wn[i - i0]) : row[i - i0];
        if (a.y) a.y[(size_t)tok * a.ldy + i] = yv;
        if (a.want_panel) quant_group_store(yv, lane, tok, gq, a.panel);
    }
    LG_STAMP(a.tag, 6);
    // every remote write into this CTA's slots precedes a cluster barrier this CTA has passed: safe to exit
}

// ---- residual update + next norm from the producer's partial sums ---------------------------------
// The matmul before this kernel (SUMS epilogue) left the complete rows o and, per work item and token, the partial sums
//   A = sum o^2,  B = sum x (w o),  C = sum (w o)^2,  D = sum x^2.
// With s1 = 1/rms(o) the new residual row is x' = (x + (o s1) w) scale, and its own mean square follows from the same
// sums without touching the row again:  sum x'^2 = scale^2 (D + 2 s1 B + s1^2 C).  So one warp per (token, 32 columns)
// does the whole update with a single round of loads after the dependency wait -- no reduction across CTAs, no second
// pass: x' goes back to the residual stream, y = (x' s2) norm_w (or x' itself without norm_w) to the next panel.
// Every token's sums are added in a fixed order (lane-strided, then the shuffle tree), whatever the block's width.
struct LgEltArgs {
    float *x; int ldx;
    const float *o; int ldo;                 // complete rows [M][ldo]
    const float4 *sums; int n_sums;          // [LG_MAXM][LG_SUMS_ITEMS], n_sums entries per token
    const float *add_w, *norm_w; float out_scale, eps; int n;
    LgPanel panel; int want_panel;
    float *y; int ldy;                       // optional f32 copy of y
    const int *skip; int tag;
};
#define LG_ELT_WARPS 4
__global__ void __launch_bounds__(LG_ELT_WARPS * 32) lg_elt_kernel(LgEltArgs a) {
    const int lane = threadIdx.x & 31, tok = blockIdx.y, gq = blockIdx.x * LG_ELT_WARPS + (threadIdx.x >> 5);
    const int i = gq * 32 + lane;
    const bool live = i < a.n;
    pdl_launch();
    // the norm weights do not depend on the previous kernel
    const float wa = live ? a.add_w[i] : 0.0f, wn = (live && a.norm_w) ? a.norm_w[i] : 1.0f;
    LG_STAMP(a.tag, 0);
    LG_STAMP_KIND(a.tag, 7);
    pdl_wait();
    LG_STAMP(a.tag, 1);
    if (a.skip && *a.skip) return;
    if (gq * 32 >= a.n) return;
    float4 pv[LG_SS_PER_LANE];
    #pragma unroll
    for (int j = 0; j < LG_SS_PER_LANE; j++) {
        const int k = lane + 32 * j;
        pv[j] = k < a.n_sums ? __ldcg(a.sums + (size_t)tok * LG_SUMS_ITEMS + k) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    const float xv = live ? __ldcg(a.x + (size_t)tok * a.ldx + i) : 0.0f;
    const float ov = live ? __ldcg(a.o + (size_t)tok * a.ldo + i) : 0.0f;
    float4 tot = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    #pragma unroll
    for (int j = 0; j < LG_SS_PER_LANE; j++) { tot.x += pv[j].x; tot.y += pv[j].y; tot.z += pv[j].z; tot.w += pv[j].w; }
    tot.x = warp_sum(tot.x); tot.y = warp_sum(tot.y); tot.z = warp_sum(tot.z); tot.w = warp_sum(tot.w);
    const float nf = (float)a.n;
    const float s1 = 1.0f / sqrtf(tot.x / nf + a.eps);
    float v = __fadd_rn(xv, __fmul_rn(__fmul_rn(ov, s1), wa));
    v = __fmul_rn(v, a.out_scale);
    if (live) a.x[(size_t)tok * a.ldx + i] = v;
    float yv = v;
    if (a.norm_w) {
        const float ssq = __fmul_rn(__fmul_rn(a.out_scale, a.out_scale),
                                    __fadd_rn(tot.w, __fadd_rn(__fmul_rn(__fmul_rn(2.0f, s1), tot.y), __fmul_rn(__fmul_rn(s1, s1), tot.z))));
        const float s2 = 1.0f / sqrtf(fmaxf(ssq, 0.0f) / nf + a.eps);
        yv = __fmul_rn(__fmul_rn(v, s2), wn);
    }
    if (!live) yv = 0.0f;
    if (a.y && live) a.y[(size_t)tok * a.ldy + i] = yv;
    if (a.want_panel) quant_group_store(yv, lane, tok, gq, a.panel);
    LG_STAMP(a.tag, 6);
}

// Quantise f32 rows into a panel (used where the producer is not one of the fused kernels).
__global__ void lg_quant_rows(const float *__restrict__ x, int ldx, int n, LgPanel P) {
    pdl_launch(); pdl_wait();
    int tok = blockIdx.y, lane = threadIdx.x & 31;
    int sb = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (sb * 32 >= n) return;
    quant_group_store(x[(size_t)tok * ldx + sb * 32 + lane], lane, tok, sb, P);
}

// ---------------------------------------------------------------------------------------------
// attention: q/k/v post-processing + split-KV flash-decode on tensor cores + combine, one launch
// ---------------------------------------------------------------------------------------------
// Keys are partitioned on ABSOLUTE position boundaries: tile T covers positions [T*S, (T+1)*S), S = lg_attn_tile(hd).
// Query j (token j of the block, position p_j = pos + j + qpos_off) attends positions
// [max(0, p_j + win_shrink - window + 1), p_j]  (window <= 0: from 0).
// A CTA handles one KV head and one tile for all of that head's queries (gqa heads x M tokens):
//   1. per-head RMSNorm + NeoX RoPE of its queries from the raw projection (f32), split into an
//      f16 hi + f16 lo pair so the tensor-core dot keeps ~22 bits of q; the CTA whose tile holds a
//      new position also normalises / rotates that position's K row and normalises its V row and
//      writes both to the f16 cache (round to nearest even) before loading the tile;
//   2. S = Q K^T and O = P V with mma.sync.m16n8k16 (f16 operands, f32 accumulate), K/V tile brought
//      in with cp.async, P also as hi + lo; scale 1.0, masks per query;
//   3. the partial (max, sum, acc[hd]) of each (query, tile) goes to scratch; the LAST CTA of a KV
//      head to finish (ticket counter) merges that head's queries over their tiles in ascending
//      order, normalises and writes the o-projection's panel.
// A partial depends only on (query position, tile) and the merge order is fixed, so a row's result
// does not depend on M or on which other queries share the launch.
struct LgAttnArgs {
    // raw projection rows [M][ld] = [q (H*hd) | k (Hkv*hd) | v (Hkv*hd)]; q_ready: q is [M][H][hd], final
    const float *qkv; int ld; int q_ready;
    int has_v, owns_kv;                  // v projection present; this layer writes K/V rows
    int early_kv;                        // the tile's cached rows may be fetched before the dependency wait (see the kernel)
    int G;                               // lg_attn_deep_kernel only: tiles of 64 keys per CTA span
    const float *q_norm, *k_norm; float eps;
    const float2 *rope;                  // [M][hd/2] (cos, sin) of this layer kind at the block's positions
    __half *kc, *vc; int seq, kv_dim;
    int H, Hkv, hd, M;
    int n_slots;               // tile slots in the scratch (>= tiles a block can touch)
    int window;                // <=0: full causal
    int qpos_off;              // 0 for the target; -1 for the draft head (query at pos sees keys < pos)
    int win_shrink;            // draft head: the window start stays pos-W+1 (one key fewer)
    const int *pos;
    float *part;               // [n_slots][M][H][hd] un-normalised tile accumulators
    float2 *part_ml;           // [n_slots][M][H] (max, sum) of each (query, tile)
    int *tickets;              // [Hkv], zero between launches
    LgPanel out; float *out_f32;   // merged output: panel of [M][H*hd] and/or f32 [M][H][hd]
    __half *out_h; int ld_h;       // and/or f16 rows [M][ld_h] (input of the wide prompt matmul)
    int tag;                       // launch index for LG_STAMP (profiling builds)
    int *err;                      // status word for bounded waits that gave up (may be null)
    const int *skip;               // optional: non-zero -> the launch does nothing (a draft that was called off)
};

#define LG_ATTN_THREADS 256
// keys per tile: 128, or 64 for head sizes whose K/V tiles would not fit in shared memory otherwise
__host__ __device__ constexpr int lg_attn_tile(int hd) { return hd > 256 ? 64 : 128; }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void *p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void *p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void *dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// cos / sin of the NeoX rotation angles of the block's M positions, computed once per forward and
// shared by every CTA of every layer of that kind: tab[tok][i] = (cos, sin)(pos_tok * base^(-2i/hd) / div[i]).
__global__ void lg_rope_table_kernel(const int *pos, int M, int hd, float base, const float *div, float2 *tab) {
    pdl_launch(); pdl_wait();
    const int half = hd >> 1;
    for (int u = blockIdx.x * blockDim.x + threadIdx.x; u < M * half; u += gridDim.x * blockDim.x) {
        const int tok = u / half, i = u % half;
        float freq = powf(base, -2.0f * (float)i / (float)hd);
        float ang = (float)(*pos + tok) * freq / (div ? div[i] : 1.0f);
        tab[u] = make_float2(cosf(ang), sinf(ang));
    }
}
// The tables of both layer kinds (sliding-window: blockIdx.y 0, full attention: 1) in one launch.
__global__ void lg_rope_tables_kernel(const int *pos, int M, int hd_a, float base_a, const float *div_a, float2 *tab_a,
                                      int hd_b, float base_b, const float *div_b, float2 *tab_b) {
    pdl_launch(); pdl_wait();
    const bool second = blockIdx.y != 0;
    const int hd = second ? hd_b : hd_a, half = hd >> 1;
    const float base = second ? base_b : base_a;
    const float *div = second ? div_b : div_a;
    float2 *tab = second ? tab_b : tab_a;
    for (int u = blockIdx.x * blockDim.x + threadIdx.x; u < M * half; u += gridDim.x * blockDim.x) {
        const int tok = u / half, i = u % half;
        float freq = powf(base, -2.0f * (float)i / (float)hd);
        float ang = (float)(*pos + tok) * freq / (div ? div[i] : 1.0f);
        tab[u] = make_float2(cosf(ang), sinf(ang));
    }
}

// RMSNorm (optional weight) + optional NeoX RoPE of one head vector by one warp.
// lane owns pairs i = lane*PER + e (e < PER) and their partners i + hd/2;  out_lo[i], out_hi[i] returned in v0/v1.
// In two halves (the loads; the arithmetic), for callers that put the loads of several rows in flight before the first use.
template <int HD>
__device__ __forceinline__ void head_load(const float *src, const float2 *rope, int lane,
                                          float (&v0)[HD / 64], float (&v1)[HD / 64], float2 (&cs)[HD / 64]) {
    constexpr int PER = HD / 64, HALF = HD / 2;
    #pragma unroll
    for (int e = 0; e < PER; e++) {
        const int i = lane * PER + e;
        v0[e] = src[i]; v1[e] = src[i + HALF];               // plain loads: a caller may pass rows staged in shared memory
        cs[e] = rope ? rope[i] : make_float2(1.0f, 0.0f);
    }
}
template <int HD>
__device__ __forceinline__ void head_finish(const float *w, bool rot, float eps, int lane,
                                            float (&v0)[HD / 64], float (&v1)[HD / 64], const float2 (&cs)[HD / 64]) {
    constexpr int PER = HD / 64, HALF = HD / 2;
    float ss = 0.0f;
    #pragma unroll
    for (int e = 0; e < PER; e++) ss += v0[e] * v0[e] + v1[e] * v1[e];
    ss = warp_sum(ss);
    float s = 1.0f / sqrtf(ss / (float)HD + eps);
    #pragma unroll
    for (int e = 0; e < PER; e++) {
        int i = lane * PER + e;
        float a = __fmul_rn(v0[e], s), b = __fmul_rn(v1[e], s);
        if (w) { a = __fmul_rn(a, w[i]); b = __fmul_rn(b, w[i + HALF]); }
        if (rot) {
            const float c = cs[e].x, sn = cs[e].y;
            float r0 = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, sn));
            float r1 = __fadd_rn(__fmul_rn(a, sn), __fmul_rn(b, c));
            a = r0; b = r1;
        }
        v0[e] = a; v1[e] = b;
    }
}
template <int HD>
__device__ __forceinline__ void head_norm_rope(const float *src, const float *w, const float2 *rope, float eps, int lane,
                                               float (&v0)[HD / 64], float (&v1)[HD / 64]) {
    float2 cs[HD / 64];
    head_load<HD>(src, rope, lane, v0, v1, cs);
    head_finish<HD>(w, rope != nullptr, eps, lane, v0, v1, cs);
}

// dynamic smem: Qhi | Qlo [NQ16][HD+8] f16 | K [S][HD+8] | V [S][HD+8] | scores [NQ16][S] f32 | Phi | Plo [NQ16][S+8] f16 | ml [NQ16][2]
template <int HD>
__global__ void __launch_bounds__(LG_ATTN_THREADS) lg_attn_kernel(LgAttnArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    // the per-head norm weights are cold in HBM and do not depend on the previous kernel: fetch them first
    __shared__ float s_qn[HD], s_kn[HD];
    pdl_launch();
    LG_STAMP(a.tag, 0);
    LG_STAMP_KIND(a.tag, 5);
    if (!a.q_ready)
        for (int i = threadIdx.x; i < HD; i += LG_ATTN_THREADS) { s_qn[i] = a.q_norm[i]; s_kn[i] = a.k_norm ? a.k_norm[i] : 1.0f; }
    // early_kv: the position and the cached rows below the block were written by earlier graph launches (this layer
    // writes its own rows, and only here), so the tile may start streaming before the previous kernel has finished
    if (!a.early_kv) { pdl_wait(); if (a.skip && *a.skip) return; }
    constexpr int S = lg_attn_tile(HD), LDH = HD + 8, LDP = S + 8, PER = HD / 64, HALF = HD / 2, NW = LG_ATTN_THREADS / 32;
    const int kvh = blockIdx.x, gqa = a.H / a.Hkv, nq = gqa * a.M, nq16 = (nq + 15) & ~15;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos0 = *a.pos;
    const int p_first = pos0 + a.qpos_off, p_last = pos0 + a.M - 1 + a.qpos_off;
    if (p_last < 0) return;
    const int lo_first = a.window > 0 ? max(0, p_first + a.win_shrink - a.window + 1) : 0;
    const int t_lo = lo_first / S, t_hi = p_last / S;
    const int T = t_lo + blockIdx.y;
    if (T > t_hi) return;
    const int slot = T % a.n_slots;
    const bool writes_kv = a.owns_kv && !a.q_ready;

    __half *qhi = (__half *)smem, *qlo = qhi + (size_t)nq16 * LDH;
    __half *sk = qlo + (size_t)nq16 * LDH, *sv = sk + (size_t)S * LDH;
    float *sc = (float *)(sv + (size_t)S * LDH);
    __half *phi = (__half *)(sc + (size_t)nq16 * S), *plo = phi + (size_t)nq16 * LDP;
    float *ml = (float *)(plo + (size_t)nq16 * LDP);

    // ---- 1. cached K and V rows of the tile start streaming into shared memory at once; rows of the
    //         block's own new positions are produced below and written to the cache and the tile ----
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
    if (a.early_kv) pdl_wait();
    LG_STAMP(a.tag, 1);

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
    LG_STAMP(a.tag, 2);
    cp_async_wait_all();
    __syncthreads();
    LG_STAMP(a.tag, 3);

    // ---- 3. scores: warp w takes keys [w*S/8, (w+1)*S/8) ----
    const int g = lane >> 2, t = lane & 3;
    constexpr int KPW = S / NW, NKT = KPW / 8;                  // keys and 8-key tiles per warp
    for (int mt = 0; mt < nq16 / 16; mt++) {
        float c0[NKT][4];
        #pragma unroll
        for (int n = 0; n < NKT; n++) c0[n][0] = c0[n][1] = c0[n][2] = c0[n][3] = 0.0f;
        const __half *qa_hi = qhi + (size_t)(mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDH + (lane >> 4) * 8;
        const __half *qa_lo = qlo + (size_t)(mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDH + (lane >> 4) * 8;
        const __half *kb = sk + (size_t)(warp * KPW + (lane & 7)) * LDH + (lane >> 3) * 8;      // 4 matrices: d = k0, +8, +16, +24
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
        if (lane == 0) { ml[qi * 2] = mx; ml[qi * 2 + 1] = sum; }
    }
    __syncthreads();

    // ---- 5. O = P V: PVW warps split the head dims ----
    constexpr int PVW = HD / 16 < NW ? HD / 16 : NW;          // warps that take part
    constexpr int DW = HD / PVW;                               // dims per warp (a multiple of 16)
    constexpr int NT = DW / 8;
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
                if (qi < nq) {
                    const int tok = qi / gqa, hq = kvh * gqa + qi % gqa;
                    float *pp = a.part + (((size_t)slot * a.M + tok) * a.H + hq) * HD;
                    #pragma unroll
                    for (int n = 0; n < NT; n++)
                        *(float2 *)(pp + warp * DW + n * 8 + t * 2) = make_float2(o[n][h2 * 2], o[n][h2 * 2 + 1]);
                    if (warp == 0 && t == 0)
                        a.part_ml[((size_t)slot * a.M + tok) * a.H + hq] = make_float2(ml[qi * 2], ml[qi * 2 + 1]);
                }
            }
        }
    }

    // ---- 6. the last CTA of this KV head merges ----
    __shared__ int s_last;
    __syncthreads();
    LG_STAMP(a.tag, 4);
    if (threadIdx.x == 0) {
        __threadfence();
        s_last = atomicAdd(a.tickets + kvh, 1) == t_hi - t_lo;
    }
    __syncthreads();
    LG_STAMP(a.tag, 5);
    if (!s_last) return;
    __threadfence();
    // (a) every (query, tile) max and sum -> shared memory (the K/V tile area is free now)
    const int nt_all = t_hi - t_lo + 1;
    float2 *mls = (float2 *)sk;                               // [nq][nt_all]: (max, sum) then (weight, -)
    float *invl = ml;                                         // [nq]
    for (int i = threadIdx.x; i < nq * nt_all; i += LG_ATTN_THREADS) {
        const int qi = i / nt_all, T2 = t_lo + i % nt_all;
        const int tok = qi / gqa, hq = kvh * gqa + qi % gqa;
        mls[i] = __ldcg(a.part_ml + ((size_t)(T2 % a.n_slots) * a.M + tok) * a.H + hq);
    }
    __syncthreads();
    // (b) per query: global max over its tiles, weights exp(m_t - max), 1 / sum of weighted sums (fixed order)
    for (int qi = warp; qi < nq; qi += NW) {
        const int pj = pos0 + qi / gqa + a.qpos_off;
        const int lo = a.window > 0 ? max(0, pj + a.win_shrink - a.window + 1) : 0;
        const int i0 = pj >= 0 ? lo / S - t_lo : 0, i1 = pj >= 0 ? pj / S - t_lo : -1;
        float mx = -INFINITY;
        for (int i = i0 + lane; i <= i1; i += 32) { float2 v = mls[qi * nt_all + i]; if (v.y > 0.0f) mx = fmaxf(mx, v.x); }
        mx = warp_max(mx);
        // a tile always lands in lane (absolute tile index % 32), so the order of this sum does not depend on where the
        // block's first tile lies (tiles outside the query's window add exact zeros)
        float lsum = 0.0f;
        for (int T2 = (t_lo & ~31) + lane; T2 <= t_hi; T2 += 32) {
            if (T2 < t_lo) continue;
            const int i = T2 - t_lo;
            float2 v = mls[qi * nt_all + i];
            float w = (i >= i0 && i <= i1 && v.y > 0.0f) ? expf(v.x - mx) : 0.0f;
            mls[qi * nt_all + i].x = w;
            lsum += w * v.y;
        }
        lsum = warp_sum(lsum);
        if (lane == 0) invl[qi] = lsum > 0.0f ? 1.0f / lsum : 0.0f;
    }
    __syncthreads();
    // (c) weighted sum of the tiles' accumulators in ascending tile order: a thread owns 4 consecutive
    //     dims of a query, 16-byte loads, 8 tiles in flight; results staged in shared memory
    float *ybuf = (float *)qhi;                                // [nq][HD] f32 (the query area is free now)
    const size_t slot_stride = (size_t)a.M * a.H * HD;
    for (int u = threadIdx.x; u < nq * (HD / 4); u += LG_ATTN_THREADS) {
        const int qi = u / (HD / 4), d4 = (u % (HD / 4)) * 4;
        const float *base = a.part + ((size_t)(qi / gqa) * a.H + kvh * gqa + qi % gqa) * HD + d4;
        const float2 *wq = mls + (size_t)qi * nt_all;
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        int i = 0;
        for (; i + 8 <= nt_all; i += 8) {
            float4 v[8];
            #pragma unroll
            for (int j = 0; j < 8; j++) v[j] = __ldcg((const float4 *)(base + (size_t)((t_lo + i + j) % a.n_slots) * slot_stride));
            #pragma unroll
            for (int j = 0; j < 8; j++) {
                const float w = wq[i + j].x;
                acc.x = fmaf(w, v[j].x, acc.x); acc.y = fmaf(w, v[j].y, acc.y);
                acc.z = fmaf(w, v[j].z, acc.z); acc.w = fmaf(w, v[j].w, acc.w);
            }
        }
        {
            float4 v[8];
            #pragma unroll
            for (int j = 0; j < 8; j++)
                if (i + j < nt_all) v[j] = __ldcg((const float4 *)(base + (size_t)((t_lo + i + j) % a.n_slots) * slot_stride));
            #pragma unroll
            for (int j = 0; j < 8; j++)
                if (i + j < nt_all) {
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
    LG_STAMP(a.tag, 6);
}

// ---------------------------------------------------------------------------------------------
// GeGLU and the per-layer-embedding elementwise pieces
// ---------------------------------------------------------------------------------------------
// y = gelu_tanh(gate) * up -> panel.  gate/up are f32 rows; `up` may be a per-token vector (PLE).
__global__ void lg_geglu_kernel(const float *__restrict__ gate, const float *__restrict__ up, int ld_g, int ld_u,
                                int n, LgPanel P) {
    pdl_launch(); pdl_wait();
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
    pdl_launch(); pdl_wait();
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
    int stop;                  // this round's remaining drafts are called off (a draft's confidence margin fell below the threshold)
    int n_skipped;             // drafts called off so far
};
// After a verify of M rows: adv = 1 + run of out[j-1] == toks[j]; append toks[1..adv-1] and
// out[adv-1] to the token log; next round starts at pos+adv with toks[0] = out[adv-1];
// h_prev <- normed hidden of row adv-1.  (The cache needs no rollback: rows past pos+adv are
// overwritten by the next round before any query can read them.)
__global__ void lg_accept_kernel(LgRoundState *st, int M, const float *__restrict__ hidden, int ld, int ne,
                                 float *__restrict__ h_prev, int *__restrict__ log, int log_cap,
                                 int advance_state) {
    pdl_launch(); pdl_wait();
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
__global__ void lg_replay_drafts_kernel(LgRoundState *st, int M, const int *__restrict__ replay, const int *__restrict__ n_replay) {
    pdl_launch(); pdl_wait();
    int j = threadIdx.x + 1;
    const int n = (replay && n_replay) ? *n_replay : 0;      // no table set: every draft is token 0
    if (j < M) { int i = st->n_emitted + j - 1; st->toks[j] = (i >= 0 && i < n) ? replay[i] : 0; }
}

// draft-head input: cat = [ embed(tok)*sqrt(nb) , h_prev ] is assembled by lg_embed_rows + this copy
__global__ void lg_copy_f32(float *__restrict__ dst, const float *__restrict__ src, int n) {
    pdl_launch(); pdl_wait();
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = src[i];
}
// The start of a draft-head forward in one launch: the position (set_pos_j >= 0: dpos = pos + set_pos_j, the round's stop
// flag cleared before its first draft), the concatenated input [ embed(toks[slot-1]) * scale , h ] quantised group by group
// into the pre-projection's panel (h = h_src, or -- h_src null -- what the previous kernel left in cat[nb ..]), and the
// rotation tables of both layer kinds at the draft's position.  One warp per 32-element group; the last block does the
// tables.  cat keeps the f32 rows (the chained draft's post-projection writes its half there).
struct LgDraftBeginArgs {
    LgRoundState *st; int slot, set_pos_j;
    const uint4 *wq; const uint2 *ws, *wd; const uint4 *wm; int fmt, nkp, n_rows; float scale;
    const float *h_src; float *cat; int nb; LgPanel p_cat;
    int hd_a; float base_a; float2 *tab_a; int hd_b; float base_b; float2 *tab_b;
};
__global__ void lg_draft_begin_kernel(LgDraftBeginArgs a) {
    pdl_launch(); pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int dpos = a.set_pos_j >= 0 ? a.st->pos + a.set_pos_j : a.st->dpos;
    if (blockIdx.x == gridDim.x - 1) {
        if (threadIdx.x == 0 && a.set_pos_j >= 0) { a.st->dpos = dpos; if (a.set_pos_j == 0) a.st->stop = 0; }
        for (int k = 0; k < 2; k++) {
            const int hd = k ? a.hd_b : a.hd_a, half = hd >> 1;
            const float base = k ? a.base_b : a.base_a;
            float2 *tab = k ? a.tab_b : a.tab_a;
            for (int i = threadIdx.x; i < half; i += blockDim.x) {
                const float ang = (float)dpos * powf(base, -2.0f * (float)i / (float)hd);
                tab[i] = make_float2(cosf(ang), sinf(ang));
            }
        }
        return;
    }
    const int row = min(max(a.st->toks[a.slot - 1], 0), a.n_rows - 1);
    for (int gq = blockIdx.x * nw + warp; gq < 2 * a.nb / 32; gq += (gridDim.x - 1) * nw) {
        const int i = gq * 32 + lane;
        float v;
        if (i < a.nb) v = __fmul_rn(lg_tile_value(a.wq, a.ws, a.wd, a.wm, a.fmt, a.nkp, row, i), a.scale);
        else v = a.h_src ? a.h_src[i - a.nb] : a.cat[i];
        if (i < a.nb || a.h_src) a.cat[i] = v;
        quant_group_store(v, lane, 0, gq, a.p_cat);
    }
}
__global__ void lg_set_draft_pos(LgRoundState *st, int j) { pdl_launch(); pdl_wait(); st->dpos = st->pos + j; if (j == 0) st->stop = 0; }
// slots a head cannot draft repeat the previous token, so the verify simply rejects them
__global__ void lg_pad_drafts(LgRoundState *st, int from, int M) { pdl_launch(); pdl_wait(); for (int j = from; j < M; j++) st->toks[j] = st->toks[j - 1]; }
// Draft j is in (lg_draft_pick_kernel): keep it -- or, when the round's drafting was called off before it ran, repeat the previous token (the
// verify then rejects the slot, as for a head that cannot chain).  A draft whose confidence margin (best - second best
// logit) is below *thr calls off the drafts after it: they would most likely be rejected, and their forwards are skipped.
// (Runs as the tail of the draft head's argmax merge: the winner of the per-CTA candidates becomes draft j.)
__global__ void lg_draft_pick_kernel(const float *__restrict__ val, const int *__restrict__ idx, int n_parts,
                                     const float *__restrict__ val2, LgRoundState *st, int j, const float *thr) {
    pdl_launch(); pdl_wait();
    float bv, s2; int bi;
    argmax_block(val, idx, n_parts, 0, val2, bv, bi, s2);
    if (threadIdx.x == 0) {
        if (st->stop) { st->toks[j] = st->toks[j - 1]; st->n_skipped++; return; }
        st->toks[j] = bi == 0x7fffffff ? 0 : bi;
        if (thr && bv - s2 < *thr) st->stop = 1;
    }
}
