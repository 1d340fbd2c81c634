/* q4cuda: B200 (sm_100a) device layer for the routed-expert MoE feed-forward path
 * with IQ3_S weights and 8-bit activations.
 *
 * This header is the drop-in boundary.  The functions named q4_hip_* / q4_mmq_*
 * keep the names, argument meaning and error behaviour of the reference engine's
 * device C ABI (src/q4.h:837-1512 of shoutliberte/Suzuku-Engine-q4; each block
 * below cites the declaration it replaces), so the engine's MoE orchestration
 * (src/q4_moe.c) links against libq4cuda.so unchanged.  The q4_cuda_* functions
 * are additions: fused forms of call sequences the engine issues today.
 *
 * Conventions (same as the reference, src/q4_rocm.cu:5433-5438):
 *  - every operation returns bool: true = enqueued; false = NOTHING was enqueued
 *    (bad shape, unsupported type, library not initialised: all checks come before
 *    the first launch), so a caller may take another path without double-counting
 *    work.  The one exception is a CUDA launch error in the middle of a call that
 *    issues several kernels: false then follows launches that already went out;
 *  - d_* pointers are device pointers owned by the caller; everything is enqueued
 *    on one library-owned stream (q4_hip_stream) and nothing synchronises unless
 *    its comment says so;
 *  - nothing allocates after q4_hip_init()/q4_hip_moe_scratch_warm(), so every
 *    compute entry point may be captured in a CUDA graph (q4_hip_graph_begin);
 *  - there is no CPU fallback: without a usable sm_100 GPU q4_hip_init() returns
 *    false and every other entry point refuses.
 *
 * Expert tensors are IQ3_S (type id 21).  The one-token exec calls also take IQ4_NL (20), IQ4_XS (23),
 * IQ3_XXS (18) and IQ2_S (22) for gate+up and IQ4_NL, IQ4_XS and Q2_0 (42) for down; the many-token
 * calls IQ4_NL and IQ4_XS; all for packs kept in an arena in the engine's byte order.
 * Router tensors are F32 (type id 0).  q4_hip_moe_tok_ok() and q4_mmq_supported() answer
 * for a given shape and type mix.
 */
#ifndef Q4CUDA_H
#define Q4CUDA_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ggml type ids used on this path (src/q4.h:20-39). */
#define Q4_T_F32 0u
#define Q4_T_IQ3_S 21u
#define Q4_T_IQ4_NL 20u   /* these two: accepted by the one-token exec calls as the type of gate+up */
#define Q4_T_IQ4_XS 23u   /* (gt == ut) and/or of down (dt) */

/* ---------------- lifecycle and memory (src/q4.h:1029-1031,1397-1400,1511-1512,
 * 1233-1235,1232,1359) ---------------- */
bool q4_hip_init(void);
void q4_hip_shutdown(void);
bool q4_hip_ok(void);
void *q4_hip_stream(void);          /* the compute stream, a cudaStream_t */
void q4_hip_sync(void);             /* drain the device */
bool q4_hip_stream_sync(void);      /* drain the compute stream */
void *q4_hip_malloc(size_t n);
void q4_hip_free(void *p);
bool q4_hip_h2d(void *d, const void *h, size_t n);        /* synchronous */
bool q4_hip_d2h(void *h, const void *d, size_t n);        /* synchronous, after the compute stream */
bool q4_hip_h2d_async(void *d, const void *h, uint64_t n);
bool q4_hip_d2h_async(void *h, const void *d, uint64_t n);
bool q4_hip_fill(float *d, float v, uint64_t n);
bool q4_hip_copy_async(float *d, const float *s, uint64_t n);
uint64_t q4_hip_vram_free(void);
/* Page-locked host memory for asynchronous copies (src/q4.h:1251-1252). */
void *q4_hip_host_alloc_coh(size_t n);
void q4_hip_host_free_coh(void *p);

/* ---------------- expert arenas (src/q4.h:842-851,1402-1413) ----------------
 * A fixed-stride device array of packed experts, pack = gate rows | up rows |
 * down rows (src/q4_expert.c:962-982).  Arena 0 is the main model; the unmarked
 * names address arena 0.  Up to 4 arenas. */
bool q4_hip_experts_alloc_a(int arena, uint32_t n_slots, uint64_t slot_bytes);
void q4_hip_experts_free_a(int arena);
uint32_t q4_hip_experts_n_a(int arena);
bool q4_hip_experts_put_a(int arena, uint32_t slot, const uint8_t *host, uint64_t n);
bool q4_hip_experts_put_async_a(int arena, uint32_t slot, const uint8_t *host, uint64_t n);
const uint8_t *q4_hip_experts_dev_a(int arena, uint32_t slot);
const uint8_t *q4_hip_experts_base_a(int arena);
uint64_t q4_hip_experts_stride_a(int arena);
bool q4_hip_experts_alloc(uint32_t n_slots, uint64_t slot_bytes);
void q4_hip_experts_free(void);
uint32_t q4_hip_experts_n(void);
bool q4_hip_experts_put(uint32_t slot, const uint8_t *host, uint64_t n);
bool q4_hip_experts_put_async(uint32_t slot, const uint8_t *host, uint64_t n);
const uint8_t *q4_hip_experts_dev(uint32_t slot);
void q4_hip_copy_wait(void);        /* host-waits for queued expert uploads */

/* ---------------- graphs (src/q4.h:1227-1231) ---------------- */
int q4_hip_graph_begin(void);       /* 1 = capturing, 0 = refused */
void *q4_hip_graph_end(void);       /* executable graph or NULL */
uint32_t q4_hip_graph_nodes(void *exec);
bool q4_hip_graph_launch(void *exec);
void q4_hip_graph_free(void *exec);

/* ---------------- routed experts, one token (src/q4.h:898-899,930-935,
 * 1296-1311,956-958) ----------------
 * y[r] += sum_e wts[e] * down_e . Q8(silu(gate_e . Q8(x)) * (up_e . Q8(x)))
 * for the n experts at base + slots[e]*stride (+og/ou/od for gate/up/down).
 * x is quantised per 32 values to int8 ("Q8-A": scale amax/127, round to
 * nearest even; reference CPU path src/q4_cpuexp.c:605-637); h likewise, per
 * expert.  d_h receives the n*n_ff fp32 hidden rows.  d_h2/d_down are unused
 * scratch of the reference's unfused fallback and may be NULL.  n <= 64.
 * exec: slots/wts are HOST arrays.  exec_dev: device arrays and a device
 * count.  stage + exec_staged: the host writes the list into mapped memory,
 * the launch reads it at run time (graph replay with new routing). */
bool q4_hip_moe_tok_ok(uint32_t gt, uint32_t ut, uint32_t dt, uint32_t in_dim, uint32_t n_ff);
bool q4_hip_moe_exec(const uint8_t *base, uint64_t stride, const int32_t *slots,
                     const float *wts, uint32_t n, uint32_t gt, uint64_t og, uint32_t ut,
                     uint64_t ou, uint32_t dt, uint64_t od, const float *d_x, float *d_h,
                     float *d_h2, float *d_down, float *d_y, uint32_t n_ff, uint32_t in_dim,
                     uint32_t n_embd);
bool q4_hip_moe_exec_dev(const uint8_t *base, uint64_t stride, const int32_t *d_es,
                         const float *d_ew, const int32_t *d_nhit, uint32_t gt, uint64_t og,
                         uint32_t ut, uint64_t ou, uint32_t dt, uint64_t od, const float *d_x,
                         float *d_h, float *d_h2, float *d_down, float *d_y, uint32_t n_ff,
                         uint32_t in_dim, uint32_t n_embd);
bool q4_hip_moe_stage(const int32_t *slots, const float *wts, uint32_t n);
bool q4_hip_moe_exec_staged(const uint8_t *base, uint64_t stride, uint32_t gt, uint64_t og,
                            uint32_t ut, uint64_t ou, uint32_t dt, uint64_t od,
                            const float *d_x, float *d_h, float *d_h2, float *d_down,
                            float *d_y, uint32_t n_ff, uint32_t in_dim, uint32_t n_embd);
void q4_hip_moe_scratch_warm(void);

/* ---------------- router and norm (src/q4.h:1414-1418,1360-1363,1075-1080) ------- */
/* softmax over n logits, top-k on strict '>' (equal values keep the lower
 * index), weights renormalised over the k picks (src/q4_quant.c:715-755).
 * n <= 1024, k <= 64.  The first form copies the result out and syncs. */
bool q4_hip_softmax_topk(const float *d_logits, uint32_t n, uint32_t k, int32_t *h_ids,
                         float *h_wts);
bool q4_hip_softmax_topk_launch(const float *d_logits, uint32_t n, uint32_t k, int32_t *d_ids,
                                float *d_wts);
/* y = x * rsqrt(mean(x^2) + eps) * w over hc groups of n_embd (w may be NULL). */
bool q4_hip_grouped_rms(const float *x, const float *w, float *y, uint32_t n_embd, uint32_t hc,
                        float eps);
bool q4_hip_grouped_rms_n(const float *x, const float *w, float *y, uint32_t n_embd,
                          uint32_t hc, float eps, uint32_t n_tok);
/* Hyper-connection streams (src/q4.h:1366-1377): a token carries hc residual streams of n_embd
 * floats.  combine: res[t][c] += block[t] * 2 sigmoid(inject[t][c] / hc).  comb_rms: the same
 * update (block + hy when hy is given) and y[t][c] = RMSNorm(res[t][c]) * wn[c] in one launch,
 * bit for bit what combine followed by q4_hip_grouped_rms gives (the reference tests exactly
 * that, src/q4_test.c:1400-1430); y == NULL in the _n form: the update only. */
bool q4_hip_hc_combine(float *res, const float *block, const float *inject, uint32_t n_embd, uint32_t hc);
bool q4_hip_hc_combine_n(float *res, const float *block, const float *inject, uint32_t n_embd, uint32_t hc,
                         uint32_t n_tok);
bool q4_hip_hc_comb_rms(float *res, const float *block, const float *inject, const float *wn, float *y,
                        uint32_t n_embd, uint32_t hc, float eps);
bool q4_hip_hc_comb_rms_n(float *res, const float *block, const float *hy, const float *inject,
                          const float *wn, float *y, uint32_t n_embd, uint32_t hc, float eps, uint32_t n_tok);
/* d_y = scale * W d_x, all device pointers, overwrites y.  F32 or IQ3_S rows. */
bool q4_hip_gemv_dd(uint32_t ggml_type, const uint8_t *d_w, uint64_t nrows, uint64_t ncols,
                    const float *d_x, float *d_y, float scale);
bool q4_hip_gemv_dd_n(uint32_t ggml_type, const uint8_t *d_w, uint64_t nrows, uint64_t ncols,
                      const float *d_x, float *d_y, float scale, uint32_t n_batch);

/* ---------------- many tokens: prefill chunks and verify windows ----------------
 * (src/q4.h:1126-1128, 1131-1175, 1278-1285, 887-897)
 * The engine's own sequence (src/q4_moe.c:3166-3251, 3697-3748, 3887):
 *   route_pf   per token: softmax, top-k (ties to the lower index), weights
 *              renormalised; ids/wts are [n_tok][topk]
 *   assign_pf  per group of gsz tokens: picks sorted by expert.  Row p of group g
 *              (p counts from the group's first row g*gsz*topk) belongs to token
 *              a_tok[g*gsz*topk + p]; rsrc[t*topk+k] = p of pick k of token t (-1 for
 *              an id outside [0, n_exp)); rw = its weight; ek[g*512+e] = rows of
 *              expert e; stg[g*512 + i] = i-th used expert; stgn[g] = how many.
 *              Rows of one expert are in (token, pick) order.  n_exp <= 512.
 *   quantize   xq rows = Q8-A of x[ids[r]] (ids NULL = identity); xq is an opaque
 *              buffer of q4_mmq_q8_bytes(rows, cols) bytes
 *   mul_id     expert e owns xq/dst rows [bounds[e], bounds[e+1]) (device int32,
 *              n_expert+1 entries), weights at w + e*expert_stride_bytes, w_rows x
 *              w_cols IQ3_S; dst rows keep the xq order, ld_dst floats apart.  Gate and
 *              up are one [2*n_ff x n_embd] matrix per expert (contiguous in the pack).
 *   swiglu     h[r][k] = silu(gu[r][k]) * gu[r][n_ff + k]
 *   expert_reduce  y[t] += sum_k rw[t][k] * pd[rsrc[t][k]], k ascending
 * w_cols a multiple of 256 with w_rows * w_cols / 256 a multiple of 8.  Rows of 256,
 * 512, 1024 or 2048 columns are summed in a fixed order (reproducible); other widths
 * use atomic adds. */
int q4_mmq_on(void);
uint32_t q4_mmq_group(void);
bool q4_mmq_supported(uint32_t type, uint64_t w_rows);
uint64_t q4_mmq_q8_bytes(uint64_t rows, uint64_t cols);
uint64_t q4_mmq_pad(uint64_t row_bytes);
bool q4_mmq_quantize(const float *x, const int32_t *ids, void *xq, uint32_t w_type, uint64_t cols,
                     uint64_t rows);
bool q4_mmq_mul_id(const void *w, uint32_t type, uint64_t w_rows, uint64_t w_cols,
                   uint64_t expert_stride_bytes, uint32_t n_expert, const void *xq,
                   const int32_t *bounds, uint32_t max_rows, uint64_t total_rows, float *dst,
                   uint64_t ld_dst);
bool q4_mmq_swiglu(const float *gu, float *h, uint64_t rows, uint64_t n_ff);
bool q4_hip_expert_reduce(float *d_y, const float *d_pd, const int32_t *d_rsrc, const float *d_rw,
                          uint32_t n_tok, uint32_t topk, uint32_t n_embd);
bool q4_hip_route_pf(const float *d_rlog, int32_t *d_ids, float *d_wts, uint32_t n_tok,
                     uint32_t n_exp, uint32_t topk);
bool q4_hip_assign_pf(const int32_t *d_ids, const float *d_wts, int32_t *d_atok, int32_t *d_rsrc,
                      float *d_rw, int32_t *d_stg, uint32_t *d_stgn, uint32_t *d_ek, uint32_t gsz,
                      uint32_t topk, uint32_t n_exp, uint32_t n_tok);
/* 2..8 token verify window over per-token slot lists (d_es/d_ew at t*64, count in
 * d_nh[t]): every distinct expert is decoded once and applied to all the tokens that
 * picked it; d_y[t] (n_embd floats per token) is ADDED to; each token's result is the
 * one q4_hip_moe_exec_dev gives for that token alone, up to the order of the final
 * sum.  d_x is n_tok rows of in_dim floats; d_h is unused. */
bool q4_hip_moe_win_ok(uint32_t gt, uint32_t ut, uint32_t dt, uint32_t in_dim, uint32_t n_ff,
                       uint32_t n_tok);
bool q4_hip_moe_exec_win(const uint8_t *base, uint64_t stride, const int32_t *d_es,
                         const float *d_ew, const int32_t *d_nh, uint32_t n_tok, uint32_t gt,
                         uint64_t og, uint32_t ut, uint64_t ou, uint32_t dt, uint64_t od,
                         const float *d_x, float *d_h, float *d_y, uint32_t n_ff, uint32_t in_dim,
                         uint32_t n_embd);

/* ---------------- the engine's small steps around the expert products ----------------
 * What src/q4_moe.c issues between the products above: elementwise updates, one-row
 * reductions, the shared expert's gate, the decode layer's pack/final pair
 * (src/q4.h:971-976, 1130-1133, 1219-1226, 1321-1326, 1384, 1396, 1512).  All enqueue on
 * the compute stream; n counts floats. */
void q4_hip_clear(void);                                     /* drop a pending CUDA error */
bool q4_hip_silu(float *d, uint64_t n);                      /* d = d / (1 + exp(-d)) */
bool q4_hip_sigmoid(float *d, uint64_t n);
bool q4_hip_scale(float *d, float s, uint64_t n);
bool q4_hip_scale_silu(float *x, float s, uint64_t n);       /* v = s x; x = silu(v) */
bool q4_hip_mul(float *y, const float *a, const float *b, uint64_t n);
bool q4_hip_add(float *y, const float *a, const float *b, uint64_t n);
bool q4_hip_mul_sig(float *y, const float *a, const float *g, uint64_t n);   /* y = a sigmoid(g) */
bool q4_hip_silu_mul(float *g, const float *u, uint64_t n);  /* g = silu(g) u */
bool q4_hip_axpy(float *y, const float *x, float a, uint64_t n);
bool q4_hip_axpy_dalpha(float *y, const float *x, const float *d_alpha, uint64_t n);
bool q4_hip_axpy_rows(float *d_y, const float *d_x, const float *d_sg, uint32_t n, uint32_t n_tok);
bool q4_hip_dot(const float *a, const float *b, float *out, uint32_t n);
bool q4_hip_dot_sigmoid(const float *a, const float *b, float *out, uint32_t n);
/* d_y[t] += sigmoid(d_w . d_x[t]) * d_sh[t] for t < n_tok, one launch. */
bool q4_hip_sgate_axpy(float *d_y, const float *d_sh, const float *d_w, const float *d_x, uint32_t n,
                       uint32_t n_tok);
/* Head of a decode layer: d_y = 0; *d_dot = sigmoid(d_x . d_sgate) when d_sgate is given;
 * sm = silu(sm) * sm2 over n_sm floats; *flag_d += 1 when given.  qx (quantise x for the exec
 * that follows) needs nothing here: the exec entry points quantise x themselves. */
bool q4_hip_moe_pack(float *d_y, const float *d_x, const float *d_sgate, float *d_dot, void *flag_d,
                     uint32_t n_embd, bool qx, float *sm, const float *sm2, uint32_t n_sm);
/* Tail: v = y + hy + sh * (dot ? *dot : 1); res[c] += v * 2 sigmoid(inj[c] / hc), c < hc. */
bool q4_hip_moe_final(float *res, const float *y, const float *hy, const float *sh, const float *dot,
                      const float *inj, uint32_t n_embd, uint32_t hc);
/* Up to 8 matrices against one vector in one launch (src/q4.h:960-970); act != 0 gives
 * that segment out = silu(act * out).  Types here: F32 and IQ3_S. */
typedef struct {
    const uint8_t *w;
    float *out;
    uint32_t rows;
    uint32_t ty;
    float act;
} q4_seg_t;
bool q4_hip_gemv_m(const q4_seg_t *segs, uint32_t nseg, const float *d_x, uint32_t in_dim);
/* Routed experts of n_tok tokens over packed DEVICE lists: token t owns entries
 * [h_off[t], h_off[t+1]) (host offsets, at most 64 per token) of d_slots / d_wts, row t of
 * d_x and d_y, rows h_off[t].. of d_h (src/q4.h:895-902).  d_y is ADDED to. */
bool q4_hip_moe_exec_tok(const uint8_t *base, uint64_t stride, const int32_t *d_slots,
                         const float *d_wts, const uint32_t *h_off, uint32_t n_tok, uint32_t gt,
                         uint64_t og, uint32_t ut, uint64_t ou, uint32_t dt, uint64_t od,
                         const float *d_x, float *d_h, float *d_h2, float *d_y, uint32_t n_ff,
                         uint32_t in_dim, uint32_t n_embd);
/* Dense product of up to 8 activation rows in 8-bit form (src/q4.h:913-927, src/q4_mmvq.cu):
 * d_y[t][r] = scale * W[r] . q8(d_x[t]).  Weight types Q6_K (14), Q4_K (12), Q5_K (13), IQ4_XS (23),
 * IQ4_NL (20) with the reference's arithmetic (activations per 32 values, d = amax / 127,
 * q = rint(v / d); runs of 16 weights; fused multiply-adds in a fixed order, so a row's bits do
 * not depend on n), and IQ3_S (21) through the grouped expert product.  ncols <= 16384, whole
 * blocks; Q4_K / Q5_K rows 16-byte aligned, IQ4_XS 8, the others 2.
 * q4_mmvq_set(mode): 0 off, 1 (default) calls of 2..8 rows, 2 calls of 1..8 rows but only between
 * q4_mmvq_verify(1) and q4_mmvq_verify(0).  q4_mmvq_warm() allocates the row scratch (q4_hip_init
 * already does).  Between hold(x) and release() calls on the same x (same width, no more rows)
 * reuse its quantisation.  false: nothing was queued, the caller keeps its float path. */
bool q4_mmvq_n(uint32_t ty, const uint8_t *d_w, uint64_t nrows, uint64_t ncols, const float *d_x,
               float *d_y, float scale, uint32_t n);
void q4_mmvq_warm(void);
void q4_mmvq_hold(const float *d_x);
void q4_mmvq_release(void);
int q4_mmvq_on(void);
void q4_mmvq_verify(int on);
void q4_mmvq_set(int v);
/* Expert-indexed weight buffers and the gather into them (src/q4.h:1144-1174).  With every
 * expert resident in slot = id the engine can pass the arena itself to q4_mmq_mul_id and skip
 * both.  A copy gathered from a tiled arena keeps the tiled byte order (whole 880-byte tiles). */
bool q4_mmq_wbuf(uint64_t gu_bytes, uint64_t d_bytes, uint32_t n_exp, uint8_t **gu, uint8_t **d);
/* Point the two buffers at the caller's memory, or drop them (NULL); from the first call on
 * q4_mmq_wbuf never allocates and fails while they are dropped or too small.  The sizes come
 * from q4_mmq_wbuf_size / _need, which read the engine's model struct and therefore live in
 * suzuku-engine-q4_b200/host/q4_engine_glue.c, compiled with the engine. */
bool q4_mmq_wbuf_lend(void *gu, uint64_t gu_bytes, void *d, uint64_t d_bytes);
bool q4_mmq_gather(const uint8_t *abase, uint64_t astride, uint64_t goff, uint64_t gu_bytes,
                   uint64_t doff, uint64_t d_bytes, uint64_t gu_dst, uint64_t d_dst,
                   const int32_t *d_eid, const int32_t *d_slot, uint32_t n, uint8_t *d_gu,
                   uint8_t *d_d);
int q4_xg_on(void);   /* 0: the reference's fp16 prefill product is not offered */

/* ---------------- the rest of what src/q4_moe.c references ----------------
 * So that the engine's MoE layer code links unchanged.  Real: host-memory helpers
 * (src/q4.h:1058-1060), a memset ordered with the expert uploads (:1319), GEMV with host
 * operands or a row gather (:1061-1077; F32 and IQ3_S), the SwiGLU alias (:1108). */
bool q4_hip_host_register(void *p, size_t n);
void *q4_hip_host_devptr(void *p);
void q4_hip_host_unregister(void *p);
bool q4_hip_copy_memset(void *dst, int v, size_t n);
bool q4_hip_gemv(uint32_t ggml_type, const uint8_t *w, uint64_t nrows, uint64_t ncols, const float *x,
                 float *y, float scale);                       /* host W, x, y; synchronous */
bool q4_hip_gemv_dev(uint32_t ggml_type, const uint8_t *d_w, uint64_t nrows, uint64_t ncols,
                     const float *x, float *y, float scale);   /* device W; host x, y */
bool q4_hip_gemv_dd_n_which(uint32_t ggml_type, const uint8_t *d_w, uint64_t nrows, uint64_t ncols,
                            const float *d_x, float *d_y, float scale, uint32_t n_batch,
                            const int32_t *which);             /* token i reads x[which[i]] */
bool q4_hip_moe_act(float *d_g, const float *d_u, uint64_t n);  /* = q4_hip_silu_mul */
void q4_hip_mark_pt(int slot);                                  /* no-op */
/* Declined: always false (nothing enqueued), the reference's answer for an uncovered type.
 * The float-activation prefill products (src/q4.h:1090-1122) come after q4_mmq_mul_id in the
 * engine's order of preference; Q4_K / Q8_0 dense forms and the fp16 prefill product are
 * outside this path. */
bool q4_hip_moe_pf(uint32_t type, const uint8_t *wbase, uint64_t stride, uint64_t woff,
                   const int32_t *d_slots, const uint32_t *d_eb, const uint32_t *d_ec,
                   const int32_t *d_atok, const float *d_x, float *d_out, uint32_t nrows,
                   uint32_t ncols, uint32_t ne);
bool q4_hip_moe_pf2(uint32_t type, const uint8_t *wbase, uint64_t stride, uint64_t woff0,
                    uint64_t woff1, const int32_t *d_slots, const uint32_t *d_eb,
                    const uint32_t *d_ec, const int32_t *d_atok, const float *d_x, float *d_out0,
                    float *d_out1, uint32_t nrows, uint32_t ncols, uint32_t ne);
bool q4_hip_moe_wmma(uint32_t type, const uint8_t *wbase, uint64_t stride, uint64_t woff,
                     const int32_t *d_slots, const uint32_t *d_eb, const uint32_t *d_ec,
                     const int32_t *d_atok, const float *d_x, float *d_out, uint32_t nrows,
                     uint32_t ncols, uint32_t ne);
bool q4_hip_moe_wmma2(uint32_t type, const uint8_t *wbase, uint64_t stride, uint64_t woff0,
                      uint64_t woff1, const int32_t *d_slots, const uint32_t *d_eb,
                      const uint32_t *d_ec, const int32_t *d_atok, const float *d_x, float *d_out,
                      uint32_t nrows, uint32_t ncols, uint32_t ne);
bool q4_hip_gateup_q4k(const uint8_t *d_gate, const uint8_t *d_up, const float *d_x, float *d_h,
                       uint32_t n_ff, uint32_t n_embd);
bool q4_hip_gateup_q4k_n_which(const uint8_t *d_gate, const uint8_t *d_up, const float *d_x,
                               float *d_h, uint32_t n_ff, uint32_t n_embd, uint32_t n_tok,
                               const int32_t *which);
bool q4_hip_q8_reuse(const uint8_t *d_w, uint64_t nrows, uint64_t ncols, const float *d_x,
                     const int32_t *which, float *d_y, float scale, uint32_t n_batch);
bool q4_xg_gu_type(uint32_t type);
bool q4_xg_dn_type(uint32_t type);
bool q4_xg_shape_ok(uint32_t n_embd, uint32_t n_ff);
uint32_t q4_xg_tile_cap(uint32_t rows, uint32_t n_exp);
uint32_t q4_xg_tiles(const uint32_t *ek, const uint32_t *ebase, const int32_t *slot, uint32_t n_exp,
                     int32_t *out, uint32_t cap);
bool q4_xg_cvt(const float *x, void *x16, uint64_t n);
bool q4_xg_gu(uint32_t type, const uint8_t *abase, uint64_t astride, uint64_t og, uint64_t ou,
              uint32_t n_embd, uint32_t n_ff, const int32_t *d_tiles, uint32_t n_tiles,
              const void *x16, const int32_t *d_atok, void *h16);
bool q4_xg_dn(uint32_t type, const uint8_t *abase, uint64_t astride, uint64_t od, uint32_t n_ff,
              uint32_t n_embd, const int32_t *d_tiles, uint32_t n_tiles, const void *h16, float *out);
/* Expert offload machinery (router-miss mailbox, CPU-pool waits, prefetch prediction,
 * verify-timeline stamps; src/q4.h:1236-1259, 1266-1295, 293-300): not present where every
 * expert is resident.  The calls answer false / 0 and enqueue nothing; the engine then routes
 * with q4_hip_softmax_topk[_launch] and runs q4_hip_moe_exec[_dev]. */
bool q4_hip_route_dev(const float *d_rlog, const int32_t *devtab, int32_t *d_es, float *d_ew,
                      int32_t *d_nhit, const int32_t *restab, int32_t *d_res_s, float *d_res_w,
                      int32_t *d_res_n, uint32_t res_cap, void *mail, unsigned long long *d_seq,
                      unsigned long long *d_rseq, unsigned long long *d_prof, uint32_t n_exp,
                      uint32_t topk);
bool q4_hip_route_dev_n(const float *d_rlog, const int32_t *devtab, int32_t *d_es, float *d_ew,
                        int32_t *d_nh, void *mail, unsigned long long *d_seq,
                        unsigned long long *d_rseq, unsigned long long *d_prof, uint32_t n_exp,
                        uint32_t topk, uint32_t n_tok);
bool q4_hip_cpx_wait(void *done_d, void *expect_d, void *progress_d);
bool q4_hip_cpx_spin_init(void);
bool q4_hip_cpx_spin(const unsigned long long *want_d, const unsigned long long *done_d);
unsigned long long q4_hip_cpx_wait_timeouts(void);
void q4_hip_cpx_wait_reset(void);
unsigned long long q4_hip_cpx_wait_lastseen(void);
size_t q4_hip_pred_size(void);
bool q4_hip_pred_sel(const float *d_plog, const int32_t *devtab, const unsigned long long *d_tseq,
                     unsigned long long *d_cnt, void *stg, uint32_t n_exp, uint32_t n_tok,
                     uint32_t kmax, float pmin);
bool q4_hip_vtl_init(void);
bool q4_hip_vtl_stamp(uint32_t slot);
bool q4_hip_vtl_read(double *out, uint32_t n, double off_ns);
double q4_hip_vtl_calib(void);

/* ---------------- additions (no single counterpart in the reference) ------------ */

/* Stage tests: the building blocks of the expert kernels, exposed so that the
 * integer stages can be compared bit for bit with the CPU path.
 * q4_cuda_quant8: per 32 floats -> int8 q[n], scale d[n/32], sum bs[n/32]
 *   (src/q4_cpuexp.c:605-637 computes the same three).
 * q4_cuda_iq3s_dequant: rows*ncols weights -> fp32 (src/q4_quant.c:384-422).
 * q4_cuda_iq3s_idot: I[r][g] = integer dot of row r's 32-group g with q
 *   (src/q4_cpuexp.c:694-699,855-892 before the sub-scale multiply). */
bool q4_cuda_quant8(const float *d_x, uint64_t n, int8_t *d_q, float *d_d, int32_t *d_bs);
/* The same two stages for IQ4_NL rows (18-byte blocks of 32; src/q4_quant.c:270-290,
 * src/q4_cpuexp.c:977-996): fp32 dequantisation, and I[r][g] = table value x q per block. */
/* Stage tests of IQ3_XXS (18), IQ2_S (22) and Q2_0 (42): dequantised rows, and the exact integer
 * part of every 32-group's dot with int8 activations (before the sub-scales; Q2_0: codes 0..3 x q). */
bool q4_cuda_fmt_dequant(uint32_t type, const uint8_t *d_w, uint64_t nrows, uint64_t ncols, float *d_out);
bool q4_cuda_fmt_idot(uint32_t type, const uint8_t *d_w, uint64_t nrows, uint64_t ncols, const int8_t *d_q,
                      int32_t *d_I);
bool q4_cuda_iq4nl_dequant(const uint8_t *d_w, uint64_t nrows, uint64_t ncols, float *d_out);
bool q4_cuda_iq4nl_idot(const uint8_t *d_w, uint64_t nrows, uint64_t ncols, const int8_t *d_q,
                        int32_t *d_I);
/* ... and by type id, 20 (IQ4_NL) or 23 (IQ4_XS, 136-byte super-blocks; src/q4_quant.c:455-480,
 * src/q4_cpuexp.c:945-975). */
bool q4_cuda_iq4_dequant(uint32_t type, const uint8_t *d_w, uint64_t nrows, uint64_t ncols, float *d_out);
bool q4_cuda_iq4_idot(uint32_t type, const uint8_t *d_w, uint64_t nrows, uint64_t ncols,
                      const int8_t *d_q, int32_t *d_I);
bool q4_cuda_iq3s_dequant(const uint8_t *d_w, uint64_t nrows, uint64_t ncols, float *d_out);
bool q4_cuda_iq3s_idot(const uint8_t *d_w, uint64_t nrows, uint64_t ncols, const int8_t *d_q,
                       int32_t *d_I);

/* One MoE layer for one token, every stage on the device with no host round
 * trip: RMSNorm -> router GEMV -> softmax/top-k -> k routed experts + the shared
 * expert -> y.  Replaces the sequence the engine issues in q4_moe_layer_dev
 * (src/q4_moe.c:2077-2133: gemv_dd, fill, softmax_topk, moe_exec, shared
 * gate/up/silu_mul/down, axpy).
 *   base/stride/og/ou/od: expert arena addressing as in q4_hip_moe_exec;
 *   routed expert id e lives in slot e, the shared expert in slot shared_slot
 *   (negative = no shared expert);
 *   d_x: n_embd fp32 hidden state; d_norm_w may be NULL (no norm weight);
 *   d_router: [n_expert][n_embd] fp32;
 *   d_y: n_embd fp32, OVERWRITTEN;
 *   d_ids/d_wts (topk entries, may be NULL) receive the routing.
 * n_embd % 256 == 0, n_ff % 256 == 0, n_expert <= 1024, topk <= 63. */
bool q4_cuda_moe_decode(const uint8_t *base, uint64_t stride, uint64_t og, uint64_t ou,
                        uint64_t od, int32_t shared_slot, const float *d_x,
                        const float *d_norm_w, float eps, const float *d_router,
                        uint32_t n_expert, uint32_t topk, uint32_t n_embd, uint32_t n_ff,
                        float *d_y, int32_t *d_ids, float *d_wts);

/* One MoE layer for n_tok tokens (any number: a verify window, an expert-parallel
 * shard's batch, a prefill chunk): the sequence above in one call, every stage on
 * the device.  Arguments as q4_cuda_moe_decode, with d_x / d_y holding n_tok rows,
 * d_ids / d_wts [n_tok][topk], the shared expert (if any) in slot n_expert and gate
 * and up contiguous in the pack (ou == og + gate bytes).  d_ws is caller-owned
 * scratch of at least q4_cuda_moe_layer_n_ws_bytes(...) bytes. */
uint64_t q4_cuda_moe_layer_n_ws_bytes(uint32_t n_tok, uint32_t topk, uint32_t n_expert,
                                      uint32_t n_embd, uint32_t n_ff);
bool q4_cuda_moe_layer_n(const uint8_t *base, uint64_t stride, uint64_t og, uint64_t ou,
                         uint64_t od, int32_t shared_slot, const float *d_x,
                         const float *d_norm_w, float eps, const float *d_router,
                         uint32_t n_expert, uint32_t topk, uint32_t n_embd, uint32_t n_ff,
                         uint32_t n_tok, float *d_y, int32_t *d_ids, float *d_wts, void *d_ws,
                         uint64_t ws_bytes);
/* RMSNorm, router product and softmax / top-k of up to 256 tokens in ONE launch (n_embd == 2048): d_xn
 * [n_tok][n_embd], d_logits [n_tok][n_expert], d_ids / d_wts [n_tok][topk], the values of
 * q4_hip_grouped_rms_n + q4_hip_gemv_dd_n + q4_hip_route_pf bit for bit.  false: another shape. */
bool q4_cuda_route_small(const float *d_x, const float *d_norm_w, float eps, const float *d_router,
                         uint32_t n_expert, uint32_t topk, uint32_t n_embd, uint32_t n_tok, float *d_xn,
                         float *d_logits, int32_t *d_ids, float *d_wts);
/* The same with the experts' formats named: gate and up of type gt, down of type dt, each IQ3_S (21),
 * IQ4_NL (20) or IQ4_XS (23); a pack with a part that is not IQ3_S sits in an arena in the engine's byte
 * order.  Workspace size as for q4_cuda_moe_layer_n. */
bool q4_cuda_moe_layer_nt(const uint8_t *base, uint64_t stride, uint32_t gt, uint64_t og, uint64_t ou,
                          uint32_t dt, uint64_t od, int32_t shared_slot, const float *d_x,
                          const float *d_norm_w, float eps, const float *d_router, uint32_t n_expert,
                          uint32_t topk, uint32_t n_embd, uint32_t n_ff, uint32_t n_tok, float *d_y,
                          int32_t *d_ids, float *d_wts, void *d_ws, uint64_t ws_bytes);

/* Routed experts for one token without any allocation on the call path.  It has no
 * counterpart in the reference: it exists for hosts that cannot call cudaMalloc by the
 * time experts run -- the engine's planner gives all free device memory to expert slots
 * and KV pages at start-up, so a later allocation fails; a stream that is being captured
 * may not allocate; a latency-bound loop cannot take an allocation's device-wide sync.
 * Same arithmetic and accumulate semantics as q4_hip_moe_exec_dev (y += sum_e w_e *
 * FFN_e(x), d_h receives the n hidden rows), with d_slots / d_wts device arrays of n
 * entries and the work enqueued on the caller's `stream` (a cudaStream_t).  The
 * quantised activations live in a fixed array inside the library image (about 40 KB per
 * GPU, held until the process exits) instead of allocated buffers, hence the limits:
 * n <= 16 experts, in_dim <= 4096, n_ff <= 2048 (larger sizes are refused with a message
 * on stderr; every argument check comes before the first launch, so false from a check means
 * nothing was enqueued -- false can also report a launch error of the runtime itself after
 * part of the sequence went out).  q4_hip_init() is not required.  The first call on each
 * device looks up the array's device address, fills the codebook constant and waits for
 * that copy; make that first call before any stream capture begins.  All calls share the one array, which keeps the
 * previous call's contents (nothing in it needs clearing: a call overwrites all it
 * reads); calls that overlap on the GPU race, so serialise them. */
bool q4_cuda_moe_exec_noalloc(const uint8_t *base, uint64_t stride, const int32_t *d_slots,
                              const float *d_wts, uint32_t n, uint64_t og, uint64_t ou,
                              uint64_t od, const float *d_x, float *d_h, float *d_y,
                              uint32_t n_ff, uint32_t in_dim, uint32_t n_embd, void *stream);

/* Resident storage format of an arena.  By default q4_hip_experts_put*_a rewrites
 * each pack, in place and at the same size, into the library's tiled form of
 * IQ3_S (every run of eight 110-byte super-blocks regrouped by field so that all
 * device loads are aligned); base/stride/offset addressing is unchanged and every
 * entry point recognises pointers into a tiled arena.  Only arenas whose slot size is
 * that of an all-IQ3_S pack (a multiple of 84480 bytes = 330 * 256) are tiled; any other
 * slot size stays in the engine's byte order.  No reference counterpart.
 *   set_tiled_default(0/1/2): format of arenas allocated afterwards (also: env
 *     Q4B_TILED=0); 2 = the caller vouches that the slots hold IQ3_S bytes only, and
 *     any slot size that is a multiple of the 880-byte tile is tiled (single matrices);
 *   tiled_a: 1 if the arena is tiled;
 *   retile_a: convert slots that were filled on the device in engine byte order
 *     (e.g. by q4_cuda_synth_iq3s);
 *   get_a: copy a slot back to the host in the engine's byte order (synchronous). */
void q4_cuda_set_tiled_default(int on);
int q4_cuda_experts_tiled_a(int arena);
bool q4_cuda_experts_retile_a(int arena, uint32_t first_slot, uint32_t n_slots);
bool q4_cuda_experts_get_a(int arena, uint32_t slot, uint8_t *host, uint64_t n);

/* The same layer for a caller that holds HOST buffers (h_x in, h_y out, n_embd
 * floats each, page-locked for speed): copy in, run, copy out, wait. */
bool q4_cuda_moe_decode_host(const uint8_t *base, uint64_t stride, uint64_t og, uint64_t ou,
                             uint64_t od, int32_t shared_slot, const float *h_x,
                             const float *d_norm_w, float eps, const float *d_router,
                             uint32_t n_expert, uint32_t topk, uint32_t n_embd, uint32_t n_ff,
                             float *h_y);
/* A layer's arguments bound once: the per-token calls then take only the token's buffers
 * (an engine decodes thousands of tokens through the same layer).  plan() returns NULL for a
 * shape the path does not take; plan_dev = q4_cuda_moe_decode, plan_host =
 * q4_cuda_moe_decode_host with the bound arguments. */
void *q4_cuda_decode_plan(const uint8_t *base, uint64_t stride, uint64_t og, uint64_t ou, uint64_t od,
                          int32_t shared_slot, const float *d_norm_w, float eps, const float *d_router,
                          uint32_t n_expert, uint32_t topk, uint32_t n_embd, uint32_t n_ff);
bool q4_cuda_decode_plan_dev(void *plan, const float *d_x, float *d_y, int32_t *d_ids, float *d_wts);
bool q4_cuda_decode_plan_host(void *plan, const float *h_x, float *h_y);
void q4_cuda_decode_plan_free(void *plan);

/* A stack of MoE layers for one token in ONE launch: y of layer l is x of layer l + 1 (no
 * counterpart in the reference, whose graph issues the per-layer chain once per layer,
 * src/q4_moe.c:2077-2133).  All layers share the shape, the arena stride and the pack offsets;
 * each has its own expert base (slot 0 of that layer), norm weights (may be NULL) and router.
 * plan() copies the descriptors to the device (it allocates: call it outside graph capture)
 * and returns NULL for a shape the persistent kernel does not take (n_embd 2048, n_ff 512,
 * n_expert <= 768, topk <= 32, tiled arena, at most 64 layers); the caller then loops over
 * q4_cuda_moe_decode.  _dev: d_x in, d_y out (both n_embd floats, d_y OVERWRITTEN), d_ids /
 * d_wts [n_layers][topk] or NULL.  _host: the same with page-locked host buffers, waits for
 * the result; false if the kernel reported an error (q4_cuda_device_error says which).
 * Launches on the library's stream must not overlap (they share the exchange scratch). */
typedef struct {
    const uint8_t *base;
    const float *d_norm_w;
    const float *d_router;
} q4_cuda_stack_layer_t;
void *q4_cuda_decode_stack_plan(const q4_cuda_stack_layer_t *layers, uint32_t n_layers, uint64_t stride,
                                uint64_t og, uint64_t ou, uint64_t od, int32_t shared_slot, float eps,
                                uint32_t n_expert, uint32_t topk, uint32_t n_embd, uint32_t n_ff);
uint32_t q4_cuda_decode_stack_layers(void *plan);
bool q4_cuda_decode_stack_dev(void *plan, const float *d_x, float *d_y, int32_t *d_ids, float *d_wts);
bool q4_cuda_decode_stack_host(void *plan, const float *h_x, float *h_y);
void q4_cuda_decode_stack_free(void *plan);
/* Optional per-plan extras.  set_sgate: the shared expert of `layer` is weighted by
 * sigmoid(d_sgate . xn) (xn = the layer's normalised input row; src/q4_moe.c:1404-1435) instead of 1;
 * d_sgate = n_embd floats on the device, 16-byte aligned, NULL = weight 1 again.  set_final: the
 * plan's last layer also adds its output to the hc residual streams, d_res[c][i] += y[i] *
 * 2 sigmoid(d_inject[c] / hc), c < hc <= 64 -- bit for bit what q4_hip_moe_final(d_res, y, 0, 0, NULL,
 * d_inject, n_embd, hc) gives after the layer (src/q4_rocm.cu:15990-16003); d_res = NULL turns it off.
 * Both apply to q4_cuda_decode_stack_dev / _host calls on the plan, not to sessions. */
bool q4_cuda_decode_stack_set_sgate(void *plan, uint32_t layer, const float *d_sgate);
bool q4_cuda_decode_stack_set_final(void *plan, float *d_res, const float *d_inject, uint32_t hc);
/* Sessions: the stack kernel stays resident and a step costs no launch.  begin launches it on
 * the library's stream over `plan`; it then waits on a doorbell in pinned host memory.  step
 * copies the token's row (n_embd floats, any host memory) into the session's pinned buffer and
 * rings; the kernel runs the next layers_per_step layers of the plan (cyclically: with 1, step s
 * is layer s mod n_layers; 0 = all of them) and writes the result row and the step number into
 * pinned host memory, where step is spinning; step copies the row to h_y and returns.  While a
 * session is live its kernel holds every SM: other work on the device waits and the other decode
 * calls of this library answer false, so end the session before anything else has to run.  The
 * kernel leaves by itself after max_steps steps (0: 2^20) or idle_ms without a ring (0: 2000,
 * at most 10000); the next step starts it again.  One session at a time.  step returns false if
 * the kernel reported an error (q4_cuda_device_error) or never answered. */
void *q4_cuda_decode_session_begin(void *plan, uint32_t layers_per_step, uint32_t max_steps, uint32_t idle_ms);
bool q4_cuda_decode_session_step(void *session, const float *h_x, float *h_y);
bool q4_cuda_decode_session_end(void *session);

/* Diagnostics of the single-kernel layer path: when enabled, the kernel records
 * the GPU's nanosecond timer at the phase boundaries of one layer of the launch
 * (profile_layer, default 0); read copies the last launch's stamps, out[cta * 16 + slot],
 * and returns the number of CTAs.  enable allocates or frees (call it outside graph
 * capture).  wait_limit sets how many polls a CTA spends waiting for another CTA's
 * values before it gives up and sets bit 2 (value 4) of the device error word
 * (0 = the default, about a tenth of a second); it exists so that a test can make the
 * wait run out. */
bool q4_cuda_fused_profile_enable(int on);
void q4_cuda_fused_profile_layer(uint32_t layer);
uint32_t q4_cuda_fused_profile_read(unsigned long long *out, uint32_t max_ctas);
void q4_cuda_decode_wait_limit(uint32_t polls);

/* Fused forms of two steps of the prefill sequence (no reference counterpart):
 * swiglu_quantize = q4_mmq_swiglu followed by q4_mmq_quantize of the result, without the fp32
 * h rows in between (hq of q4_mmq_q8_bytes(rows, n_ff) bytes); expert_reduce_set =
 * q4_hip_expert_reduce onto a zeroed y, without the zeroing. */
bool q4_cuda_mmq_swiglu_quantize(const float *gu, void *hq, uint64_t rows, uint64_t n_ff);
bool q4_cuda_expert_reduce_set(float *d_y, const float *d_pd, const int32_t *d_rsrc, const float *d_rw,
                               uint32_t n_tok, uint32_t topk, uint32_t n_embd);

/* Row assignment for one rank of an expert-parallel layer (no reference counterpart): the picks
 * of all n_tok tokens (global expert ids) -> rows of the experts [own_first, own_first + own_count)
 * this rank holds, renumbered from 0; with has_shared one more pick (local expert own_count,
 * weight 1) for tokens [tok_first, tok_first + tok_count).  d_atok/d_rsrc/d_rw as
 * q4_hip_assign_pf with topk + has_shared columns and one group of n_tok tokens (unused rows of
 * d_atok get -1); d_bounds receives own_count + has_shared + 1 row bounds for q4_mmq_mul_id. */
bool q4_cuda_assign_local(const int32_t *d_ids, const float *d_wts, int32_t *d_atok, int32_t *d_rsrc,
                          float *d_rw, int32_t *d_bounds, uint32_t n_tok, uint32_t topk,
                          uint32_t own_first, uint32_t own_count, int has_shared, uint32_t tok_first,
                          uint32_t tok_count);

/* Which grouped product q4_mmq_mul_id and q4_cuda_moe_layer_n run (no reference
 * counterpart; the reference picks its tile kernel by row count inside q4_mmq_mul_id,
 * src/q4_mmq.cu:387-470): -1 = by size (experts with 12 rows or more go to the tensor-core
 * kernel when the weight rows are a multiple of 128; the others to the streaming CUDA-core
 * kernel on tiled arenas, else to the general CUDA-core kernel),
 * 0 = CUDA-core kernels only, 1 = the tensor-core kernel whenever the shape allows,
 * 2 = the general CUDA-core kernel only.  Returns false for an unknown mode, or for 1
 * when the tensor-core path could not be set up. */
bool q4_cuda_mmq_tc_mode(int mode);
/* Activation quantiser of the many-token sequence (q4_mmq_quantize, q4_cuda_mmq_swiglu_quantize,
 * q4_cuda_moe_layer_n): 0 (default) = Q8-A, the product's own (d = amax / 127, round to nearest
 * even: the reference's CPU path); 1 = Q8-C, ggml's q8_1 (d_inv = 127 / amax, round half away from
 * zero, d = 1 / d_inv: what the reference's grouped device product quantises with,
 * third_party/llama.cpp/ggml/src/ggml-cuda/quantize.cu:491-553).  q8_sections gives the device
 * pointers of a row buffer's parts for stage tests. */
void q4_cuda_mmq_q8_compat(int on);
bool q4_cuda_mmq_q8_sections(const void *xq, uint64_t rows, uint64_t cols, const int8_t **q, const float **d,
                             const int32_t **sums);

/* Seeded synthetic tensors generated on the device (benchmark and smoke
 * support, no reference counterpart): n_blocks IQ3_S super-blocks with
 * fp16 d = |N(0,1)| * 2^-6 and uniform random payload bytes; n fp32 values
 * N(mean, std).  Content depends only on (seed, index). */
bool q4_cuda_synth_iq3s(uint8_t *d_out, uint64_t n_blocks, uint64_t seed);
/* The same, for blocks [first_block, first_block + n_blocks) of the seeded tensor:
 * a rank that holds a shard generates exactly the bytes the full tensor has there. */
bool q4_cuda_synth_iq3s_at(uint8_t *d_out, uint64_t n_blocks, uint64_t seed, uint64_t first_block);
bool q4_cuda_synth_normal(float *d_out, uint64_t n, uint64_t seed, float mean, float std);

/* Device-side timing on the compute stream, for benchmarks: records an event
 * pair around whatever is enqueued between begin and end; ms() waits for the
 * end event. */
bool q4_cuda_timer_begin(void);
bool q4_cuda_timer_end(void);
float q4_cuda_timer_ms(void);
/* The same with many marks: mark(i) records mark i (i < 2048) on the compute stream;
 * between_ms(i, j) waits for mark j and returns the device time from mark i to mark j. */
bool q4_cuda_timer_mark(uint32_t i);
float q4_cuda_timer_between_ms(uint32_t i, uint32_t j);
/* Number of kernels this library has launched since init (its own count). */
uint64_t q4_cuda_launch_count(void);
/* Last error word written by a kernel's self-check (0 = none); clears it. */
uint32_t q4_cuda_device_error(void);

#ifdef __cplusplus
}
#endif
#endif
