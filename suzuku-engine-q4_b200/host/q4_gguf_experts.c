/* See q4_gguf_experts.h.  GGUF container layout (public ggml specification):
 *   u32 magic "GGUF" | u32 version | u64 n_tensors | u64 n_kv
 *   n_kv x { string key | u32 type | value }      string = u64 length + bytes
 *   n_tensors x { string name | u32 n_dims | u64 ne[n_dims] | u32 ggml type | u64 offset }
 *   padding to `general.alignment` (default 32) | tensor data
 */
#define _GNU_SOURCE
#include "q4_gguf_experts.h"

#include <fcntl.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

enum { KV_U8, KV_I8, KV_U16, KV_I16, KV_U32, KV_I32, KV_F32, KV_BOOL, KV_STR, KV_ARR, KV_U64, KV_I64, KV_F64 };

uint64_t q4b_gguf_row_bytes(uint32_t type, uint64_t ncols) {
    /* {values per block, bytes per block} by ggml type id */
    static const struct { uint32_t type, per, bytes; } T[] = {
        {0, 1, 4},    {1, 1, 2},     {2, 32, 18},   {3, 32, 20},   {6, 32, 22},   {7, 32, 24},   {8, 32, 34},
        {9, 32, 36},  {10, 256, 84}, {11, 256, 110}, {12, 256, 144}, {13, 256, 176}, {14, 256, 210},
        {15, 256, 292}, {16, 256, 66}, {17, 256, 74}, {18, 256, 98}, {19, 256, 50}, {20, 32, 18},
        {21, 256, 110}, {22, 256, 82}, {23, 256, 136}, {30, 1, 2}};
    for (size_t i = 0; i < sizeof T / sizeof T[0]; i++)
        if (T[i].type == type) return (ncols % T[i].per) ? 0 : ncols / T[i].per * T[i].bytes;
    return 0;
}

/* buffered sequential reader over the head of the file */
typedef struct {
    int fd;
    uint64_t pos;
    bool ok;
} rd_t;

static void rd_bytes(rd_t *r, void *dst, uint64_t n) {
    if (!r->ok) return;
    uint8_t *d = (uint8_t *)dst;
    while (n) {
        const ssize_t k = pread(r->fd, d, n > (1u << 20) ? (1u << 20) : (size_t)n, (off_t)r->pos);
        if (k <= 0) {
            r->ok = false;
            return;
        }
        d += k;
        r->pos += (uint64_t)k;
        n -= (uint64_t)k;
    }
}
static uint32_t rd_u32(rd_t *r) {
    uint32_t v = 0;
    rd_bytes(r, &v, 4);
    return v;
}
static uint64_t rd_u64(rd_t *r) {
    uint64_t v = 0;
    rd_bytes(r, &v, 8);
    return v;
}
/* string into buf (truncated to cap - 1, always terminated); the rest is skipped */
static void rd_str(rd_t *r, char *buf, size_t cap) {
    const uint64_t n = rd_u64(r);
    if (!r->ok || n > (1ull << 30)) {
        r->ok = false;
        return;
    }
    const uint64_t keep = n < cap - 1 ? n : cap - 1;
    if (buf) {
        rd_bytes(r, buf, keep);
        buf[keep] = 0;
        r->pos += n - keep;
    } else {
        r->pos += n;
    }
}
static uint64_t kv_scalar_size(uint32_t t) {
    switch (t) {
    case KV_U8: case KV_I8: case KV_BOOL: return 1;
    case KV_U16: case KV_I16: return 2;
    case KV_U32: case KV_I32: case KV_F32: return 4;
    case KV_U64: case KV_I64: case KV_F64: return 8;
    default: return 0;
    }
}
/* skips one value of type t; *u32_out receives it when it is a u32 */
static void kv_skip(rd_t *r, uint32_t t, uint32_t *u32_out) {
    if (t == KV_STR) {
        rd_str(r, NULL, 0);
    } else if (t == KV_ARR) {
        const uint32_t et = rd_u32(r);
        const uint64_t n = rd_u64(r);
        if (et == KV_STR) {
            for (uint64_t i = 0; i < n && r->ok; i++) rd_str(r, NULL, 0);
        } else if (et == KV_ARR || !kv_scalar_size(et)) {
            r->ok = false;
        } else {
            r->pos += n * kv_scalar_size(et);
        }
    } else if (kv_scalar_size(t)) {
        if (t == KV_U32 && u32_out) {
            *u32_out = rd_u32(r);
        } else {
            r->pos += kv_scalar_size(t);
        }
    } else {
        r->ok = false;
    }
}

bool q4b_gguf_open(q4b_gguf *g, const char *path) {
    if (!g || !path) return false;
    memset(g, 0, sizeof *g);
    g->fd = open(path, O_RDONLY);
    if (g->fd < 0) return false;
    rd_t r = {g->fd, 0, true};
    const uint32_t magic = rd_u32(&r);
    g->version = rd_u32(&r);
    if (!r.ok || magic != 0x46554747u || (g->version != 2 && g->version != 3)) goto fail;
    g->n_tensors = rd_u64(&r);
    const uint64_t n_kv = rd_u64(&r);
    if (!r.ok || g->n_tensors > (1u << 24) || n_kv > (1u << 24)) goto fail;
    g->alignment = 32;
    for (uint64_t i = 0; i < n_kv && r.ok; i++) {
        char key[128];
        rd_str(&r, key, sizeof key);
        const uint32_t t = rd_u32(&r);
        uint32_t v = 0;
        const bool is_align = strcmp(key, "general.alignment") == 0 && t == KV_U32;
        kv_skip(&r, t, is_align ? &v : NULL);
        if (is_align && v && (v & (v - 1)) == 0) g->alignment = v;
    }
    g->tensors = (q4b_gguf_tensor *)calloc(g->n_tensors ? g->n_tensors : 1, sizeof *g->tensors);
    if (!r.ok || !g->tensors) goto fail;
    for (uint64_t i = 0; i < g->n_tensors && r.ok; i++) {
        q4b_gguf_tensor *t = &g->tensors[i];
        rd_str(&r, t->name, sizeof t->name);
        t->n_dims = rd_u32(&r);
        if (t->n_dims == 0 || t->n_dims > 4) goto fail;
        for (uint32_t d = 0; d < 4; d++) t->ne[d] = d < t->n_dims ? rd_u64(&r) : 1;
        t->type = rd_u32(&r);
        t->offset = rd_u64(&r);
        const uint64_t rb = q4b_gguf_row_bytes(t->type, t->ne[0]);
        t->nbytes = rb * t->ne[1] * t->ne[2] * t->ne[3];     /* 0: a type this reader cannot size */
    }
    if (!r.ok) goto fail;
    g->data_off = (r.pos + g->alignment - 1) / g->alignment * g->alignment;
    return true;
fail:
    q4b_gguf_close(g);
    return false;
}

void q4b_gguf_close(q4b_gguf *g) {
    if (!g) return;
    if (g->fd >= 0) close(g->fd);
    free(g->tensors);
    memset(g, 0, sizeof *g);
    g->fd = -1;
}

const q4b_gguf_tensor *q4b_gguf_find(const q4b_gguf *g, const char *name) {
    if (!g || !name) return NULL;
    for (uint64_t i = 0; i < g->n_tensors; i++)
        if (strcmp(g->tensors[i].name, name) == 0) return &g->tensors[i];
    return NULL;
}

static const q4b_gguf_tensor *layer_tensor(const q4b_gguf *g, int32_t layer, const char *suffix) {
    char want[128];
    snprintf(want, sizeof want, "blk.%d.%s", layer, suffix);
    return q4b_gguf_find(g, want);
}

bool q4b_gguf_expert_parts(const q4b_gguf *g, int32_t layer, const q4b_gguf_tensor **gate,
                           const q4b_gguf_tensor **up, const q4b_gguf_tensor **down, uint64_t *off_gate,
                           uint64_t *off_up, uint64_t *off_down, uint64_t *total, uint32_t *n_expert) {
    if (!g || layer < 0) return false;
    const q4b_gguf_tensor *tg = layer_tensor(g, layer, "ffn_gate_exps.weight");
    const q4b_gguf_tensor *tu = layer_tensor(g, layer, "ffn_up_exps.weight");
    const q4b_gguf_tensor *td = layer_tensor(g, layer, "ffn_down_exps.weight");
    if (!tg || !tu || !td || tg->n_dims != 3 || tu->n_dims != 3 || td->n_dims != 3) return false;
    const uint64_t ne = tg->ne[2];
    if (ne == 0 || tu->ne[2] != ne || td->ne[2] != ne || !tg->nbytes || !tu->nbytes || !td->nbytes) return false;
    /* gate and up are [n_ff x n_embd], down is [n_embd x n_ff] */
    if (tu->ne[0] != tg->ne[0] || tu->ne[1] != tg->ne[1] || td->ne[0] != tg->ne[1] || td->ne[1] != tg->ne[0])
        return false;
    const uint64_t sg = tg->nbytes / ne, su = tu->nbytes / ne, sd = td->nbytes / ne;
    if (gate) *gate = tg;
    if (up) *up = tu;
    if (down) *down = td;
    if (off_gate) *off_gate = 0;
    if (off_up) *off_up = sg;
    if (off_down) *off_down = sg + su;
    if (total) *total = sg + su + sd;
    if (n_expert) *n_expert = (uint32_t)ne;
    return true;
}

static bool read_at(const q4b_gguf *g, uint8_t *dst, uint64_t n, uint64_t off) {
    while (n) {
        const ssize_t k = pread(g->fd, dst, n > (1u << 30) ? (1u << 30) : (size_t)n, (off_t)off);
        if (k <= 0) return false;
        dst += k;
        off += (uint64_t)k;
        n -= (uint64_t)k;
    }
    return true;
}

int64_t q4b_gguf_read_pack(const q4b_gguf *g, int32_t layer, int32_t eid, uint8_t *dst) {
    const q4b_gguf_tensor *t[3];
    uint64_t off[3], total;
    uint32_t ne;
    if (!dst || !q4b_gguf_expert_parts(g, layer, &t[0], &t[1], &t[2], &off[0], &off[1], &off[2], &total, &ne))
        return -1;
    if (eid < 0 || (uint32_t)eid >= ne) return -1;
    for (int i = 0; i < 3; i++) {
        const uint64_t slice = t[i]->nbytes / ne;
        if (!read_at(g, dst + off[i], slice, g->data_off + t[i]->offset + slice * (uint64_t)eid)) return -1;
    }
    return (int64_t)total;
}

int64_t q4b_gguf_read_shared_pack(const q4b_gguf *g, int32_t layer, uint8_t *dst, uint64_t cap) {
    static const char *const names[3] = {"ffn_gate_shexp.weight", "ffn_up_shexp.weight", "ffn_down_shexp.weight"};
    uint64_t off = 0;
    for (int i = 0; i < 3; i++) {
        const q4b_gguf_tensor *t = layer_tensor(g, layer, names[i]);
        if (!t || !t->nbytes || !dst || off + t->nbytes > cap) return -1;
        if (!read_at(g, dst + off, t->nbytes, g->data_off + t->offset)) return -1;
        off += t->nbytes;
    }
    return (int64_t)off;
}
