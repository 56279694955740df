/* lg_quant.c -- ggml block geometry and f32 decode for the formats on the decode path.
 * The decode must be bit-identical to the reference's (src/quant.c:14-36 half->float,
 * :155-182 q4_K, :276-285 q4_0): q4_0 value = d * (nibble - 8) with element j in the low
 * nibble of byte j and element j+16 in the high nibble; q4_K value = (d*sc)*q - (dmin*m) with
 * eight 6-bit (sc, m) pairs packed into 12 bytes.
 */
#include <stdlib.h>
#include <string.h>
#include "lg_host.h"
#include "lg_formats.h"

float lg_half_to_float(uint16_t h) {
    uint32_t s = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 31, f = h & 1023, bits;
    if (e == 31) bits = s | 0x7F800000u | (f << 13);
    else if (e) bits = s | ((e + 112) << 23) | (f << 13);
    else if (!f) bits = s;
    else {                                   /* subnormal half: renormalise */
        int sh = 0;
        while (!(f & 1024)) { f <<= 1; sh++; }
        bits = s | ((uint32_t)(113 - sh) << 23) | ((f & 1023) << 13);
    }
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

int ggml_blck_size(uint32_t t) {
    switch (t) {
    case GGML_TYPE_F32: case GGML_TYPE_F16: case GGML_TYPE_BF16: return 1;
    case GGML_TYPE_Q4_0: case GGML_TYPE_Q8_0: return 32;
    case GGML_TYPE_Q4_K: case GGML_TYPE_Q3_K: case GGML_TYPE_Q5_K: case GGML_TYPE_Q6_K: return 256;
    default: return 0;
    }
}
size_t ggml_type_size(uint32_t t) {
    switch (t) {
    case GGML_TYPE_F32: return 4;
    case GGML_TYPE_F16: case GGML_TYPE_BF16: return 2;
    case GGML_TYPE_Q4_0: return 18;
    case GGML_TYPE_Q8_0: return 34;
    case GGML_TYPE_Q4_K: return 144;
    case GGML_TYPE_Q3_K: return 110;
    case GGML_TYPE_Q5_K: return 176;
    case GGML_TYPE_Q6_K: return 210;
    default: return 0;
    }
}
size_t ggml_nbytes(uint32_t t, int64_t n) {
    int b = ggml_blck_size(t);
    if (!b || n < 0 || n % b) return 0;
    return (size_t)(n / b) * ggml_type_size(t);
}

static void q4k_pair(const uint8_t *p, int j, int *sc, int *mn) {
    if (j < 4) { *sc = p[j] & 63; *mn = p[j + 4] & 63; }
    else { *sc = (p[j + 4] & 15) | ((p[j - 4] >> 6) << 4); *mn = (p[j + 4] >> 4) | ((p[j] >> 6) << 4); }
}

bool dequantize_into(uint32_t type, const void *src, float *y, int64_t n) {
    int blk = ggml_blck_size(type);
    if (!blk || n % blk) return false;
    const uint8_t *p = src;
    int64_t nb = n / blk;
    switch (type) {
    case GGML_TYPE_F32: memcpy(y, src, (size_t)n * 4); return true;
    case GGML_TYPE_F16:
        for (int64_t i = 0; i < n; i++) { uint16_t h; memcpy(&h, p + 2 * i, 2); y[i] = lg_half_to_float(h); }
        return true;
    case GGML_TYPE_BF16:
        for (int64_t i = 0; i < n; i++) {
            uint16_t h; memcpy(&h, p + 2 * i, 2);
            uint32_t b = (uint32_t)h << 16; memcpy(&y[i], &b, 4);
        }
        return true;
    case GGML_TYPE_Q4_0:
        for (int64_t b = 0; b < nb; b++, p += 18, y += 32) {
            uint16_t h; memcpy(&h, p, 2);
            float d = lg_half_to_float(h);
            for (int j = 0; j < 16; j++) {
                y[j]      = d * (float)((int)(p[2 + j] & 15) - 8);
                y[j + 16] = d * (float)((int)(p[2 + j] >> 4) - 8);
            }
        }
        return true;
    case GGML_TYPE_Q8_0: case GGML_TYPE_Q6_K: case GGML_TYPE_Q5_K: case GGML_TYPE_Q3_K: {
        /* y = (d * s) * q - (dmin * m), element by element (src/quant.c:184-274 evaluates the same products in the same order) */
        const int bytes = lg_fmt_bytes((int)type);
        for (int64_t b = 0; b < nb; b++, p += bytes, y += blk)
            for (int e = 0; e < blk; e++) {
                int q, sc, mi; uint16_t db, mb;
                lg_fmt_elem((int)type, p, e, &q, &sc, &db, &mb, &mi);
                float ds = lg_half_to_float(db) * (float)sc;
                float v = ds * (float)q;
                if (type == GGML_TYPE_Q5_K) { float off = lg_half_to_float(mb) * (float)mi; v = v - off; }
                y[e] = v;
            }
        return true;
    }
    case GGML_TYPE_Q4_K:
        for (int64_t b = 0; b < nb; b++, p += 144) {
            uint16_t h0, h1; memcpy(&h0, p, 2); memcpy(&h1, p + 2, 2);
            float d = lg_half_to_float(h0), dmin = lg_half_to_float(h1);
            const uint8_t *q = p + 16;
            for (int pair = 0; pair < 4; pair++, q += 32) {
                int s0, m0, s1, m1;
                q4k_pair(p + 4, 2 * pair, &s0, &m0);
                q4k_pair(p + 4, 2 * pair + 1, &s1, &m1);
                float d0 = d * (float)s0, o0 = dmin * (float)m0, d1 = d * (float)s1, o1 = dmin * (float)m1;
                for (int j = 0; j < 32; j++) *y++ = d0 * (float)(q[j] & 15) - o0;
                for (int j = 0; j < 32; j++) *y++ = d1 * (float)(q[j] >> 4) - o1;
            }
        }
        return true;
    default: return false;
    }
}

float *dequantize_row(const struct gguf_tensor *t, int64_t row, int64_t row_len) {
    int blk = ggml_blck_size(t->type);
    if (!t->data || !blk || row_len % blk) return NULL;
    const uint8_t *src = (const uint8_t *)t->data + (size_t)(row * row_len / blk) * ggml_type_size(t->type);
    float *y = malloc((size_t)row_len * sizeof(float));
    if (y && !dequantize_into(t->type, src, y, row_len)) { free(y); y = NULL; }
    return y;
}
