/* Build glue that compiles the reference engine's own CPU expert path
 * (src/q4_cpuexp.c + src/q4_quant.c, unmodified, from where the reference
 * checkout lies) into oracle/_ref/libq4ref.so and exposes it through a few
 * flat entry points for the tests and for the timed CPU baseline.
 *
 * TEST INFRASTRUCTURE ONLY.  None of the reference's source text is copied
 * here: q4_cpuexp.c is pulled in with #include so that its file-local kernels
 * (cpx_quant8, dq8_iq3_s, cpx_dot8) can be called directly, and the two engine
 * lookups it needs (q4_expert_parts, q4_expert_host_ptr; the engine versions
 * are src/q4_expert.c:962-982 and :1710-1723) are served from a caller-given
 * table of packed-expert pointers.
 *
 * Build: see oracle/build.py (needs -I <reference>/src).
 */
#include "q4_cpuexp.c"

/* q4.h only forward-declares this type (src/q4.h:166), so the harness owns
 * its layout: packed experts are looked up by id in a pointer table. */
struct q4_expert_cache {
    const uint8_t *const *packs;
    uint32_t n_packs;
    q4_tensor tg, tu, td;
    uint64_t sg, su, sd;
};

static struct q4_expert_cache g_shim;
static q4_gguf g_shim_gguf;

bool q4_expert_parts(const q4_gguf *g, int32_t layer, const q4_tensor **gate,
                     const q4_tensor **up, const q4_tensor **down,
                     uint64_t *off_gate, uint64_t *off_up, uint64_t *off_down,
                     uint64_t *total) {
    (void)g;
    (void)layer;
    *gate = &g_shim.tg;
    *up = &g_shim.tu;
    *down = &g_shim.td;
    *off_gate = 0;
    *off_up = g_shim.sg;
    *off_down = g_shim.sg + g_shim.su;
    *total = g_shim.sg + g_shim.su + g_shim.sd;
    return true;
}

const uint8_t *q4_expert_host_ptr(const q4_expert_cache *c, int32_t layer,
                                  int32_t eid) {
    (void)layer;
    if (eid < 0 || (uint32_t)eid >= c->n_packs) return NULL;
    return c->packs[eid];
}

static uint32_t g_shim_down_type = Q4_T_IQ3_S;   /* type of the down projection of the packs */
static uint32_t g_shim_gu_type = Q4_T_IQ3_S;     /* type of gate and up */
void q4ref_set_down_type(uint32_t type) { g_shim_down_type = type; }
void q4ref_set_gu_type(uint32_t type) { g_shim_gu_type = type; }

static void shim_tensor(q4_tensor *t, uint32_t type, uint64_t cols, uint64_t rows, uint32_t n_exp) {
    memset(t, 0, sizeof *t);
    t->n_dims = 3;
    t->ne[0] = cols;
    t->ne[1] = rows;
    t->ne[2] = n_exp;
    t->ggml_type = type;
    t->n_experts = (int32_t)n_exp;
    t->nbytes = q4_row_bytes(type, cols) * rows * n_exp;
    t->kind = Q4_KIND_ROUTED;
}

static void shim_setup(const uint8_t *const *packs, uint32_t n_packs,
                       uint32_t n_embd, uint32_t n_ff) {
    g_shim.packs = packs;
    g_shim.n_packs = n_packs;
    shim_tensor(&g_shim.tg, g_shim_gu_type, n_embd, n_ff, n_packs);
    shim_tensor(&g_shim.tu, g_shim_gu_type, n_embd, n_ff, n_packs);
    shim_tensor(&g_shim.td, g_shim_down_type, n_ff, n_embd, n_packs);
    g_shim.sg = g_shim.tg.nbytes / n_packs;
    g_shim.su = g_shim.tu.nbytes / n_packs;
    g_shim.sd = g_shim.td.nbytes / n_packs;
    memset(&g_shim_gguf, 0, sizeof g_shim_gguf);
    g_shim_gguf.n_embd = n_embd;
    g_shim_gguf.n_ff_exp = n_ff;
}

/* ---- flat entry points ---- */

int q4ref_q8_bytes(void) { return (int)sizeof(cpx_q8); }

void q4ref_quant8(const float *x, uint64_t n, void *out) {
    cpx_quant8(x, n, (cpx_q8 *)out);
}

/* The dispatching row dot the CPU pool uses (AVX-512 when the host has it). */
float q4ref_dot8(const uint8_t *row, const void *xq, uint64_t n) {
    float v = 0.f;
    cpx_fgrid_init();
    cpx_esigns_init();
    cpx_dot8(Q4_T_IQ3_S, row, (const cpx_q8 *)xq, n, &v);
    return v;
}

/* The AVX2 kernel, whatever the host supports. */
float q4ref_dot8_avx2(const uint8_t *row, const void *xq, uint64_t n) {
    return dq8_iq3_s(row, (const cpx_q8 *)xq, n);
}

/* The float-activation row dot (src/q4_cpuexp.c:182-221). */
float q4ref_dot_f32(const uint8_t *row, const float *x, uint64_t n) {
    return dot_iq3_s(row, x, n);
}

int q4ref_dequant_row(const uint8_t *src, uint64_t n, float *dst) {
    return q4_dequant_row(Q4_T_IQ3_S, src, n, dst) ? 1 : 0;
}
/* The same three for any type the CPU path takes. */
int q4ref_dequant_row_t(uint32_t type, const uint8_t *src, uint64_t n, float *dst) {
    return q4_dequant_row(type, src, n, dst) ? 1 : 0;
}
float q4ref_dot8_t(uint32_t type, const uint8_t *row, const void *xq, uint64_t n) {
    float v = 0.f;
    cpx_fgrid_init();
    cpx_esigns_init();
    cpx_dot8(type, row, (const cpx_q8 *)xq, n, &v);
    return v;
}
float q4ref_dot8_avx2_iq4nl(const uint8_t *row, const void *xq, uint64_t n) {
    return dq8_iq4_nl(row, (const cpx_q8 *)xq, n);
}
float q4ref_dot8_avx2_iq4xs(const uint8_t *row, const void *xq, uint64_t n) {
    return dq8_iq4_xs(row, (const cpx_q8 *)xq, n);
}

/* y (+)= W x through the scalar reference GEMV (src/q4_quant.c:595-626). */
int q4ref_gemv(uint32_t type, const uint8_t *w, uint64_t nrows, uint64_t ncols,
               const float *x, float *y) {
    memset(y, 0, nrows * sizeof(float));
    return q4_gemv(type, w, nrows, ncols, x, y, 1.0f) ? 1 : 0;
}

void q4ref_rms_norm(const float *x, const float *w, float *y, uint64_t n, float eps) {
    q4_rms_norm(x, w, y, n, eps);
}
void q4ref_softmax(float *x, uint64_t n) { q4_softmax(x, n); }
void q4ref_topk(const float *p, uint32_t n, uint32_t k, int32_t *ids, float *wts,
                int renorm) {
    q4_topk(p, n, k, ids, wts, renorm != 0);
}

int q4ref_threads(void) { return cpx_threads(); }
int q4ref_selftest(void) { return q4_cpx_selftest(); }

/* One token, k experts: ids index the caller's pointer table.
 * Returns 0 on success. */
int q4ref_expert_job(const uint8_t *const *packs, uint32_t n_packs,
                     const int32_t *ids, const float *wts, uint32_t k,
                     const float *x, uint32_t n_embd, uint32_t n_ff, float *y) {
    shim_setup(packs, n_packs, n_embd, n_ff);
    uint64_t tag = 0;
    int s;
    while ((s = q4_cpuex_dispatch2(&g_shim_gguf, &g_shim, 0, x, ids, wts, k, y,
                                   &tag)) == -1)
        q4_cpuex_retire();
    if (s < 0) return s;
    return q4_cpuex_join_tag(s, tag) ? 0 : -3;
}

/* 2..8 tokens, expert reuse across the window (src/q4_cpuexp.c:2618-2753).
 * x and y are token-major; ids/wts concatenated per token, tn[t] counts. */
int q4ref_expert_job_win(const uint8_t *const *packs, uint32_t n_packs,
                         const int32_t *ids, const float *wts,
                         const uint32_t *tn, uint32_t n_tok, const float *x,
                         uint32_t n_embd, uint32_t n_ff, float *y) {
    shim_setup(packs, n_packs, n_embd, n_ff);
    uint64_t tag = 0;
    int s;
    while ((s = q4_cpuex_dispatch_win(&g_shim_gguf, &g_shim, 0, x, n_tok, ids,
                                      wts, tn, y, &tag)) == -1)
        q4_cpuex_retire();
    if (s < 0) return s;
    return q4_cpuex_join_tag(s, tag) ? 0 : -3;
}

/* Timed loop for the CPU baseline: `jobs` single-token jobs, job j using
 * ids[j*k .. j*k+k) and x + (j % n_x) * n_embd.  Returns seconds, <0 on
 * error. */
double q4ref_time_jobs(const uint8_t *const *packs, uint32_t n_packs,
                       const int32_t *ids, const float *wts, uint32_t k,
                       uint32_t jobs, const float *x, uint32_t n_x,
                       uint32_t n_embd, uint32_t n_ff, float *y) {
    shim_setup(packs, n_packs, n_embd, n_ff);
    struct timespec t0, t1;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (uint32_t j = 0; j < jobs; j++) {
        uint64_t tag = 0;
        int s;
        while ((s = q4_cpuex_dispatch2(&g_shim_gguf, &g_shim, 0,
                                       x + (size_t)(j % n_x) * n_embd,
                                       ids + (size_t)j * k, wts + (size_t)j * k,
                                       k, y, &tag)) == -1)
            q4_cpuex_retire();
        if (s < 0) return -1.0;
        if (!q4_cpuex_join_tag(s, tag)) return -2.0;
    }
    clock_gettime(CLOCK_MONOTONIC, &t1);
    return (double)(t1.tv_sec - t0.tv_sec) + 1e-9 * (double)(t1.tv_nsec - t0.tv_nsec);
}

/* Timed loop for the CPU baseline of a whole MoE layer, one token per job:
 * RMSNorm -> fp32 router GEMV -> softmax -> top-k (src/q4_quant.c:595-755)
 * -> one expert job with the k picks plus the shared expert at weight 1
 * (src/q4_cpuexp.c:2503).  Layer l of job j is j % n_layers; its packs are
 * packs[l * (n_expert + 1) ..], the shared expert last.  Returns seconds. */
double q4ref_time_layers(const uint8_t *const *packs, uint32_t n_layers,
                         uint32_t n_expert, const float *const *routers,
                         const float *const *norm_w, float eps, uint32_t topk,
                         uint32_t jobs, const float *x, uint32_t n_x,
                         uint32_t n_embd, uint32_t n_ff, float *y,
                         int32_t *ids_out) {
    float *xn = malloc(sizeof(float) * n_embd);
    float *p = malloc(sizeof(float) * n_expert);
    int32_t ids[CPX_MAX_E];
    float wts[CPX_MAX_E];
    if (!xn || !p || topk + 1 > CPX_MAX_E) return -1.0;
    struct timespec t0, t1;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (uint32_t j = 0; j < jobs; j++) {
        const uint32_t l = j % n_layers;
        shim_setup(packs + (size_t)l * (n_expert + 1), n_expert + 1, n_embd, n_ff);
        q4_rms_norm(x + (size_t)(j % n_x) * n_embd, norm_w[l], xn, n_embd, eps);
        memset(p, 0, sizeof(float) * n_expert);
        q4_gemv(Q4_T_F32, (const uint8_t *)routers[l], n_expert, n_embd, xn, p, 1.0f);
        q4_softmax(p, n_expert);
        q4_topk(p, n_expert, topk, ids, wts, true);
        ids[topk] = (int32_t)n_expert;
        wts[topk] = 1.0f;
        uint64_t tag = 0;
        int s;
        while ((s = q4_cpuex_dispatch2(&g_shim_gguf, &g_shim, 0, xn, ids, wts,
                                       topk + 1, y, &tag)) == -1)
            q4_cpuex_retire();
        if (s < 0) return -1.0;
        if (!q4_cpuex_join_tag(s, tag)) return -2.0;
        if (ids_out) memcpy(ids_out + (size_t)j * topk, ids, sizeof(int32_t) * topk);
    }
    clock_gettime(CLOCK_MONOTONIC, &t1);
    free(xn);
    free(p);
    return (double)(t1.tv_sec - t0.tv_sec) + 1e-9 * (double)(t1.tv_nsec - t0.tv_nsec);
}

static double shim_now(void) {
    struct timespec t;
    clock_gettime(CLOCK_MONOTONIC, &t);
    return (double)t.tv_sec + 1e-9 * (double)t.tv_nsec;
}

/* Timed loop for the CPU baseline of the many-token workloads: `steps` layer jobs of
 * n_tok tokens each.  Per layer job every token is normed and routed on the host
 * (q4_rms_norm, q4_gemv F32, q4_softmax, q4_topk: src/q4_quant.c:595-755); the expert
 * work then goes to the worker pool in windows of as many tokens as one window job takes
 * (at most 8 tokens and 64 picks, src/q4_cpuexp.c:2618-2640), the shared expert as one
 * more pick of every token at weight 1; a last single token goes through the one-token
 * job.  Layer l of job j is j % n_layers (packs as in q4ref_time_layers).  chain != 0:
 * the output rows of a job are the input rows of the next (a stack of layers); else
 * every job reads x.  x, y, scratch: n_tok rows of n_embd floats.  Returns seconds
 * (< 0 on error); *router_s receives the part spent in norm + router + softmax + top-k. */
double q4ref_time_layers_win(const uint8_t *const *packs, uint32_t n_layers, uint32_t n_expert,
                             const float *const *routers, const float *const *norm_w, float eps,
                             uint32_t topk, uint32_t steps, const float *x, uint32_t n_tok,
                             uint32_t n_embd, uint32_t n_ff, int chain, float *y, double *router_s) {
    const uint32_t k1 = topk + 1;
    uint32_t win = 64u / k1;
    if (win > 8) win = 8;
    if (k1 > CPX_MAX_E || win < 1 || n_tok == 0) return -1.0;
    float *xn = malloc(sizeof(float) * (size_t)n_tok * n_embd);
    float *cur = malloc(sizeof(float) * (size_t)n_tok * n_embd);
    float *p = malloc(sizeof(float) * n_expert);
    int32_t *ids = malloc(sizeof(int32_t) * (size_t)n_tok * k1);
    float *wts = malloc(sizeof(float) * (size_t)n_tok * k1);
    uint32_t tn[8];
    if (!xn || !cur || !p || !ids || !wts) return -1.0;
    memcpy(cur, x, sizeof(float) * (size_t)n_tok * n_embd);
    for (uint32_t t = 0; t < 8; t++) tn[t] = k1;
    double t_router = 0.0;
    const double t0 = shim_now();
    for (uint32_t j = 0; j < steps; j++) {
        const uint32_t l = j % n_layers;
        shim_setup(packs + (size_t)l * (n_expert + 1), n_expert + 1, n_embd, n_ff);
        const double r0 = shim_now();
        for (uint32_t t = 0; t < n_tok; t++) {
            q4_rms_norm(cur + (size_t)t * n_embd, norm_w[l], xn + (size_t)t * n_embd, n_embd, eps);
            memset(p, 0, sizeof(float) * n_expert);
            q4_gemv(Q4_T_F32, (const uint8_t *)routers[l], n_expert, n_embd, xn + (size_t)t * n_embd, p, 1.0f);
            q4_softmax(p, n_expert);
            q4_topk(p, n_expert, topk, ids + (size_t)t * k1, wts + (size_t)t * k1, true);
            ids[(size_t)t * k1 + topk] = (int32_t)n_expert;
            wts[(size_t)t * k1 + topk] = 1.0f;
        }
        t_router += shim_now() - r0;
        for (uint32_t t = 0; t < n_tok;) {
            uint32_t n = n_tok - t < win ? n_tok - t : win;
            uint64_t tag = 0;
            int s;
            if (n >= 2) {
                while ((s = q4_cpuex_dispatch_win(&g_shim_gguf, &g_shim, 0, xn + (size_t)t * n_embd, n,
                                                  ids + (size_t)t * k1, wts + (size_t)t * k1, tn,
                                                  y + (size_t)t * n_embd, &tag)) == -1)
                    q4_cpuex_retire();
            } else {
                while ((s = q4_cpuex_dispatch2(&g_shim_gguf, &g_shim, 0, xn + (size_t)t * n_embd,
                                               ids + (size_t)t * k1, wts + (size_t)t * k1, k1,
                                               y + (size_t)t * n_embd, &tag)) == -1)
                    q4_cpuex_retire();
            }
            if (s < 0) return -1.0;
            if (!q4_cpuex_join_tag(s, tag)) return -2.0;
            t += n;
        }
        if (chain) memcpy(cur, y, sizeof(float) * (size_t)n_tok * n_embd);
    }
    const double t1 = shim_now();
    if (router_s) *router_s = t_router;
    free(xn);
    free(cur);
    free(p);
    free(ids);
    free(wts);
    return t1 - t0;
}
