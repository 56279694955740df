/* lg_formats.h -- element-wise decode of the ggml block formats beyond q4_0 / q4_K, shared by the host C
 * (lg_quant.c) and the device code (lg_kernels.cuh).
 *
 * Every format here decodes as   y = (d * s) * q  [- m]   in f32, evaluated in that order, which is the order of the
 * reference's decoders (src/quant.c:184-274: q5_K `d1 * q - m1` with d1 = d*sc, m1 = min*m; q3_K `dl * q` with
 * dl = d_all * (scale - 32); q6_K `d * sc * q`; q8_0 `d * q`), so a device decode built from the four pieces below is
 * bit-identical to it:
 *      q   small integer weight        (fits int8)
 *      s   integer scale of the element's group of 16 (q6_K, q3_K) or 32 (q5_K; q8_0: 1)
 *      d   f16 scale of the element's block (q8_0) or super-block (the K formats), as raw f16 bits
 *      m   f32 offset of the element's group of 32 (q5_K: dmin * m; the others 0)
 * Block layouts (bytes): q8_0 34 = d, 32 x int8;  q6_K 210 = ql[128], qh[64], int8 scales[16], d;
 * q5_K 176 = d, dmin, scales[12], qh[32], qs[128];  q3_K 110 = hmask[32], qs[64], scales[12], d.
 */
#ifndef LG_FORMATS_H
#define LG_FORMATS_H
#include <stdint.h>

#ifdef __CUDACC__
#define LG_HD __host__ __device__ __forceinline__
#else
#define LG_HD static inline
#endif

#define LG_T_Q8_0 8
#define LG_T_Q3_K 11
#define LG_T_Q5_K 13
#define LG_T_Q6_K 14

LG_HD int lg_fmt_block(int type) { return type == LG_T_Q8_0 ? 32 : 256; }
LG_HD int lg_fmt_bytes(int type) { return type == LG_T_Q8_0 ? 34 : type == LG_T_Q6_K ? 210 : type == LG_T_Q5_K ? 176 : 110; }
LG_HD int lg_fmt_is_i8(int type) { return type == LG_T_Q8_0 || type == LG_T_Q6_K || type == LG_T_Q5_K || type == LG_T_Q3_K; }

/* 6-bit (scale, min) pair j (0..7) of the 12 packed bytes q4_K and q5_K share */
LG_HD void lg_k4_pair(const uint8_t *p, int j, int *sc, int *mn) {
    if (j < 4) { *sc = p[j] & 63; *mn = p[j + 4] & 63; }
    else { *sc = (p[j + 4] & 15) | ((p[j - 4] >> 6) << 4); *mn = (p[j + 4] >> 4) | ((p[j] >> 6) << 4); }
}

/* Element e (0 .. block-1) of block b: the integer pieces.  *dbits = raw f16 bits of d; *mbits = raw f16 bits of dmin
 * and *mi its integer multiplier (q5_K), both 0 otherwise. */
LG_HD void lg_fmt_elem(int type, const uint8_t *b, int e, int *q, int *s, uint16_t *dbits, uint16_t *mbits, int *mi) {
    *mbits = 0; *mi = 0;
    if (type == LG_T_Q8_0) {
        *dbits = (uint16_t)(b[0] | (b[1] << 8));
        *q = (int8_t)b[2 + e]; *s = 1;
    } else if (type == LG_T_Q6_K) {
        /* halves of 128; in a half, quarter c (32 elements) takes the low (c < 2) or high nibble of ql[l + 32 (c & 1)]
         * and bits 2c, 2c+1 of qh[l]; one int8 scale per 16 elements */
        const int n = e >> 7, c = (e & 127) >> 5, l = e & 31;
        const int lo = b[n * 64 + l + (c & 1) * 32], hi = b[128 + n * 32 + l];
        *q = (((c >> 1) ? (lo >> 4) : (lo & 15)) | (((hi >> (2 * c)) & 3) << 4)) - 32;
        *s = (int8_t)b[192 + (e >> 4)];
        *dbits = (uint16_t)(b[208] | (b[209] << 8));
    } else if (type == LG_T_Q5_K) {
        /* pairs of sub-blocks of 32 share 32 bytes of qs (low / high nibble); bit j of qh[l] is the fifth bit of sub-block j */
        const int j = e >> 5, l = e & 31;
        int sc, mn;
        lg_k4_pair(b + 4, j, &sc, &mn);
        *q = ((b[48 + (j >> 1) * 32 + l] >> (4 * (j & 1))) & 15) + (((b[16 + l] >> j) & 1) << 4);
        *s = sc; *mi = mn;
        *dbits = (uint16_t)(b[0] | (b[1] << 8));
        *mbits = (uint16_t)(b[2] | (b[3] << 8));
    } else {
        /* q3_K: halves of 128; in a half, quarter c takes bits 2c, 2c+1 of qs[n*32 + l]; bit (4n + c) of hmask[l] set
         * means "no -4"; sixteen 6-bit scales (low 4 bits in bytes 0..7 by nibble, high 2 bits in bytes 8..11), minus 32 */
        const int n = e >> 7, c = (e & 127) >> 5, l = e & 31, si = e >> 4, i = si & 3, grp = si >> 2;
        const uint8_t *sb = b + 96;
        const int nib = grp < 2 ? (sb[(grp & 1) * 4 + i] & 15) : (sb[(grp & 1) * 4 + i] >> 4);
        *s = (nib | (((sb[8 + i] >> (2 * grp)) & 3) << 4)) - 32;
        *q = ((b[32 + n * 32 + l] >> (2 * c)) & 3) - (((b[l] >> (4 * n + c)) & 1) ? 0 : 4);
        *dbits = (uint16_t)(b[108] | (b[109] << 8));
    }
}
#endif
