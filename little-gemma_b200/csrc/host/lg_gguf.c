/* lg_gguf.c -- GGUF v2/v3 reader (little endian): header, metadata, tensor table, and the
 * data section mapped read-only.  Independent implementation of the container API the
 * little-gemma host exposes (include/gguf.h:97-136; on-disk format as parsed by
 * src/gguf.c:249-386): strings are u64 length + bytes, arrays are u32 element type + u64
 * count + payload, tensor offsets are relative to the data section, which starts at the next
 * multiple of general.alignment (default 32).
 */
#define _GNU_SOURCE
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <fcntl.h>
#include <unistd.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include "lg_host.h"

#define LG_GGUF_MAGIC 0x46554747u      /* "GGUF" */
#define LG_MAX_STR    (1ull << 30)

struct cursor { const unsigned char *p, *end; int bad; };

static void take(struct cursor *c, void *dst, size_t n) {
    if (c->bad || (size_t)(c->end - c->p) < n) { c->bad = 1; memset(dst, 0, n); return; }
    memcpy(dst, c->p, n);
    c->p += n;
}
static uint32_t take_u32(struct cursor *c) { uint32_t v; take(c, &v, 4); return v; }
static uint64_t take_u64(struct cursor *c) { uint64_t v; take(c, &v, 8); return v; }

static char *take_str(struct cursor *c) {
    uint64_t n = take_u64(c);
    if (c->bad || n > LG_MAX_STR || (uint64_t)(c->end - c->p) < n) { c->bad = 1; return NULL; }
    char *s = malloc(n + 1);
    if (!s) { c->bad = 1; return NULL; }
    memcpy(s, c->p, n);
    s[n] = 0;
    c->p += n;
    return s;
}

static size_t scalar_size(uint32_t t) {
    switch (t) {
    case GGUF_TYPE_UINT8: case GGUF_TYPE_INT8: case GGUF_TYPE_BOOL: return 1;
    case GGUF_TYPE_UINT16: case GGUF_TYPE_INT16: return 2;
    case GGUF_TYPE_UINT32: case GGUF_TYPE_INT32: case GGUF_TYPE_FLOAT32: return 4;
    case GGUF_TYPE_UINT64: case GGUF_TYPE_INT64: case GGUF_TYPE_FLOAT64: return 8;
    default: return 0;
    }
}

static void parse_value(struct cursor *c, struct gguf_meta *kv) {
    kv->type = take_u32(c);
    size_t sz = scalar_size(kv->type);
    if (sz) { take(c, &kv->value, sz); return; }
    if (kv->type == GGUF_TYPE_STRING) { kv->value.str = take_str(c); return; }
    if (kv->type != GGUF_TYPE_ARRAY) { c->bad = 1; return; }
    kv->value.arr.type = take_u32(c);
    kv->value.arr.n = take_u64(c);
    uint64_t n = kv->value.arr.n;
    size_t esz = scalar_size(kv->value.arr.type);
    if (c->bad || n > LG_MAX_STR) { c->bad = 1; return; }
    if (esz) {
        if ((uint64_t)(c->end - c->p) < n * esz) { c->bad = 1; return; }
        kv->value.arr.data = malloc(n * esz > 0 ? n * esz : 1);
        if (!kv->value.arr.data) { c->bad = 1; return; }
        take(c, kv->value.arr.data, n * esz);
    } else if (kv->value.arr.type == GGUF_TYPE_STRING) {
        /* every string costs at least its 8-byte length word: more entries than that cannot be in the file */
        if (n > (uint64_t)(c->end - c->p) / 8) { c->bad = 1; return; }
        char **v = calloc(n ? n : 1, sizeof(char *));
        kv->value.arr.data = v;
        if (!v) { c->bad = 1; return; }
        for (uint64_t i = 0; i < n && !c->bad; i++) v[i] = take_str(c);
    } else c->bad = 1;
}

void free_gguf(struct gguf_context *g) {
    if (!g) return;
    for (uint64_t i = 0; g->meta && i < g->header.num_meta; i++) {
        struct gguf_meta *kv = &g->meta[i];
        free(kv->key);
        if (kv->type == GGUF_TYPE_STRING) free(kv->value.str);
        else if (kv->type == GGUF_TYPE_ARRAY) {
            if (kv->value.arr.type == GGUF_TYPE_STRING && kv->value.arr.data)
                for (uint64_t j = 0; j < kv->value.arr.n; j++) free(((char **)kv->value.arr.data)[j]);
            free(kv->value.arr.data);
        }
    }
    for (uint64_t i = 0; g->tensors && i < g->header.num_tensors; i++) free(g->tensors[i].name);
    free(g->meta);
    free(g->tensors);
    if (g->map_base) munmap(g->map_base, g->map_len);
    if (g->map_fd >= 0) close(g->map_fd);
    free(g);
}

struct gguf_context *load_gguf(const char *path) {
    int fd = open(path, O_RDONLY);
    if (fd < 0) { fprintf(stderr, "gguf: cannot open %s\n", path); return NULL; }
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 24) { close(fd); return NULL; }
    void *base = mmap(NULL, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    if (base == MAP_FAILED) { close(fd); return NULL; }

    struct gguf_context *g = calloc(1, sizeof *g);
    if (!g) { munmap(base, (size_t)st.st_size); close(fd); return NULL; }
    g->map_base = base; g->map_len = (size_t)st.st_size; g->map_fd = fd;

    struct cursor c = { base, (const unsigned char *)base + st.st_size, 0 };
    g->header.magic = take_u32(&c);
    g->header.version = take_u32(&c);
    g->header.num_tensors = take_u64(&c);
    g->header.num_meta = take_u64(&c);
    if (g->header.magic != LG_GGUF_MAGIC || g->header.version < 2 || g->header.version > 3 ||
        g->header.num_tensors > (1u << 24) || g->header.num_meta > (1u << 24)) {
        fprintf(stderr, "gguf: %s is not a little-endian GGUF v2/v3 file\n", path);
        g->header.num_tensors = g->header.num_meta = 0;
        free_gguf(g);
        return NULL;
    }
    g->meta = calloc(g->header.num_meta ? g->header.num_meta : 1, sizeof *g->meta);
    g->tensors = calloc(g->header.num_tensors ? g->header.num_tensors : 1, sizeof *g->tensors);
    if (!g->meta || !g->tensors) { free_gguf(g); return NULL; }
    for (uint64_t i = 0; i < g->header.num_meta && !c.bad; i++) {
        g->meta[i].key = take_str(&c);
        parse_value(&c, &g->meta[i]);
    }
    for (uint64_t i = 0; i < g->header.num_tensors && !c.bad; i++) {
        struct gguf_tensor *t = &g->tensors[i];
        t->name = take_str(&c);
        t->n_dims = take_u32(&c);
        if (t->n_dims < 1 || t->n_dims > 4) { c.bad = 1; break; }
        for (uint32_t d = 0; d < 4; d++) t->dims[d] = d < t->n_dims ? take_u64(&c) : 1;
        t->type = take_u32(&c);
        t->offset = take_u64(&c);
    }
    if (c.bad) { fprintf(stderr, "gguf: %s is truncated or malformed\n", path); free_gguf(g); return NULL; }

    g->alignment = gguf_get_u32(g, "general.alignment", 32);
    if (g->alignment == 0) g->alignment = 32;
    size_t used = (size_t)(c.p - (const unsigned char *)base);
    g->data_offset = (used + g->alignment - 1) / g->alignment * g->alignment;
    if (g->data_offset > g->map_len) g->data_offset = g->map_len;
    g->data = (unsigned char *)base + g->data_offset;
    g->data_size = g->map_len - g->data_offset;
    for (uint64_t i = 0; i < g->header.num_tensors; i++) {
        struct gguf_tensor *t = &g->tensors[i];
        /* element count with overflow caught: no format packs more than 32 elements into a byte-sized unit
         * smaller than 1/32 byte per element, so a count beyond 32 x the data section cannot be real */
        int64_t n = 1;
        int wrapped = 0;
        for (uint32_t d = 0; d < t->n_dims; d++) {
            if (t->dims[d] > (uint64_t)INT64_MAX || __builtin_mul_overflow(n, (int64_t)t->dims[d], &n)) { wrapped = 1; break; }
            if ((uint64_t)n > (uint64_t)g->data_size * 32u + 32u) { wrapped = 1; break; }
        }
        size_t bytes = wrapped ? 0 : ggml_nbytes(t->type, n);
        if (wrapped || t->offset > g->data_size || bytes > g->data_size - t->offset) {
            fprintf(stderr, "gguf: tensor %s lies outside the file\n", t->name);
            free_gguf(g);
            return NULL;
        }
        t->data = (unsigned char *)g->data + t->offset;
    }
    return g;
}

void gguf_data_dontneed(const struct gguf_context *g, const void *p, size_t bytes) {
    if (!g || !g->map_base) return;
    const unsigned char *lo = p, *hi = lo + bytes;
    const unsigned char *d0 = g->data, *d1 = d0 + g->data_size;
    if (lo < d0 || hi > d1) return;
    long page = sysconf(_SC_PAGESIZE);
    uintptr_t a = ((uintptr_t)lo + (uintptr_t)page - 1) / (uintptr_t)page * (uintptr_t)page;
    uintptr_t b = (uintptr_t)hi / (uintptr_t)page * (uintptr_t)page;
    if (b > a) madvise((void *)a, b - a, MADV_DONTNEED);
}

const struct gguf_meta *gguf_find_meta(const struct gguf_context *g, const char *key) {
    for (uint64_t i = 0; i < g->header.num_meta; i++)
        if (g->meta[i].key && strcmp(g->meta[i].key, key) == 0) return &g->meta[i];
    return NULL;
}

const struct gguf_tensor *gguf_find_tensor(const struct gguf_context *g, const char *name) {
    for (uint64_t i = 0; i < g->header.num_tensors; i++)
        if (g->tensors[i].name && strcmp(g->tensors[i].name, name) == 0) return &g->tensors[i];
    return NULL;
}

uint32_t gguf_get_u32(const struct gguf_context *g, const char *key, uint32_t fb) {
    const struct gguf_meta *kv = gguf_find_meta(g, key);
    if (!kv) return fb;
    if (kv->type == GGUF_TYPE_UINT32) return kv->value.u32;
    if (kv->type == GGUF_TYPE_INT32) return (uint32_t)kv->value.i32;
    return fb;
}
int32_t gguf_get_i32(const struct gguf_context *g, const char *key, int32_t fb) {
    const struct gguf_meta *kv = gguf_find_meta(g, key);
    if (!kv) return fb;
    if (kv->type == GGUF_TYPE_INT32) return kv->value.i32;
    if (kv->type == GGUF_TYPE_UINT32) return (int32_t)kv->value.u32;
    return fb;
}
float gguf_get_f32(const struct gguf_context *g, const char *key, float fb) {
    const struct gguf_meta *kv = gguf_find_meta(g, key);
    return kv && kv->type == GGUF_TYPE_FLOAT32 ? kv->value.f32 : fb;
}
const char *gguf_get_str(const struct gguf_context *g, const char *key, const char *fb) {
    const struct gguf_meta *kv = gguf_find_meta(g, key);
    return kv && kv->type == GGUF_TYPE_STRING && kv->value.str ? kv->value.str : fb;
}
