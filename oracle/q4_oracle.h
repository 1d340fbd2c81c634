/* CPU oracle for the IQ3_S x 8-bit-activation MoE feed-forward path.
 *
 * TEST INFRASTRUCTURE ONLY.  This is a plain-C restatement of the arithmetic of
 * the reference engine's CPU expert path; it exists so that the CUDA kernels
 * can be checked against it.  Nothing in the shipped library links or calls it.
 *
 * Parity status: PINNED.  Every function below is checked (tests/test_oracle.py)
 * against the reference's own closed-form known answers (src/q4_test.c:34-73)
 * and, where the compiled reference CPU path is available (oracle/_ref), bit for
 * bit against the reference functions named beside each declaration.
 *
 * Citations are file:line in the reference project (shoutliberte/Suzuku-Engine-q4).
 */
#ifndef Q4_ORACLE_H
#define Q4_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define Q4O_QK_K 256u          /* weights per IQ3_S super-block            */
#define Q4O_IQ3S_BYTES 110u    /* bytes per IQ3_S super-block              */

/* 32 activations quantised to int8: the reference's cpx_q8
 * (src/q4_cpuexp.c:588-592).  40 bytes. */
typedef struct {
    int8_t  q[32];
    float   d;   /* amax / 127 */
    int32_t bs;  /* sum of q   */
} q4o_q8;

/* Codebook entry i as the reference stores it: four magnitude bytes in one
 * 32-bit word (src/q4_iq_grids.inc:224). */
uint32_t q4o_iq3s_grid(uint32_t idx);

/* fp16 bits -> fp32, exact (the reference uses F16C, src/q4_cpuexp.c:29). */
float q4o_f16_to_f32(uint16_t h);

/* One super-block -> 256 signed magnitudes (+-1..+-15) and the eight odd
 * sub-scale multipliers 1+2s.  Layout: src/q4_quant.c:384-422. */
void q4o_iq3s_unpack(const uint8_t *blk, int8_t w[256], uint8_t ls[8], float *d);

/* Row of n weights (n % 256 == 0) -> fp32.  src/q4_quant.c:384-422
 * (dequant_iq3_s): value = (d * (1 + 2 s)) * magnitude * sign. */
void q4o_iq3s_dequant_row(const uint8_t *src, uint64_t n, float *dst);

/* Activation quantiser "Q8-A": src/q4_cpuexp.c:605-637 (cpx_quant8).
 * n % 32 == 0.  Round-to-nearest-even; amax == 0 gives d = 0, q = 0. */
void q4o_quant8(const float *x, uint64_t n, q4o_q8 *out);

/* Integer dot of every 32-group of one weight row with the quantised
 * activations: I[g] = sum_i sign_i * mag_i * q_i (no sub-scale applied).
 * n % 256 == 0; I has n / 32 entries.  src/q4_cpuexp.c:694-699,855-892. */
void q4o_iq3s_group_idot(const uint8_t *row, const q4o_q8 *x, uint64_t n, int32_t *I);

/* fp32 row dot in the reference's exact operation order (eight fp32 lanes,
 * one fused multiply-add per lane and group, fixed final tree):
 * src/q4_cpuexp.c:855-892 (dq8_iq3_s) and :39-46 (cpx_hsum). */
float q4o_iq3s_dot8(const uint8_t *row, const q4o_q8 *x, uint64_t n);

/* SwiGLU element: src/q4_cpuexp.c:2130,2282. */
float q4o_silu(float v);

/* One expert, one token (src/q4_cpuexp.c:2239-2321):
 *   h[r] = silu(gate_r . xq) * (up_r . xq)   r < n_ff
 *   hq   = Q8-A(h)
 *   y[r] += wt * (down_r . hq)               r < n_embd
 * pack = gate rows | up rows | down rows (src/q4_expert.c:962-982).
 * h_out (n_ff floats) and hq_out (n_ff/32) may be NULL. */
void q4o_expert_ffn(const uint8_t *pack, const q4o_q8 *xq, uint32_t n_embd,
                    uint32_t n_ff, float wt, float *y, float *h_out,
                    q4o_q8 *hq_out);

/* k experts, one token: quantise x once, zero y, run the experts in list
 * order (src/q4_cpuexp.c:2503-2612; the reference's cross-expert add order is
 * a race, this one is fixed). */
void q4o_expert_job(const uint8_t *const *packs, const float *wts, uint32_t k,
                    const float *x, uint32_t n_embd, uint32_t n_ff, float *y);

/* src/q4_quant.c:697-706 (q4_rms_norm): fp64 sum of squares. */
void q4o_rms_norm(const float *x, const float *w, float *y, uint64_t n, float eps);

/* fp32 GEMV y[r] = W[r] . x in the reference's order (src/q4_quant.c:582-593,
 * dot_f32: eight products summed left to right, then added to the total). */
void q4o_gemv_f32(const float *W, uint64_t nrows, uint64_t ncols, const float *x,
                  float *y);

/* src/q4_quant.c:715-726 (q4_softmax), in place. */
void q4o_softmax(float *x, uint64_t n);

/* src/q4_quant.c:728-755 (q4_topk): insertion sort on strict '>', so equal
 * values keep the lower index; optional renormalisation in rank order. */
void q4o_topk(const float *p, uint32_t n, uint32_t k, int32_t *ids, float *wts,
              int renormalize);

/* One MoE layer, one token: RMSNorm -> router -> softmax -> top-k ->
 * k routed experts + the shared expert (weight 1).
 * expert_base + id * expert_stride addresses a routed pack.
 * ids_out/wts_out (topk entries), xn_out (n_embd) may be NULL. */
void q4o_moe_layer(const float *x, const float *norm_w, float eps,
                   const float *router_w, uint32_t n_expert, uint32_t topk,
                   const uint8_t *expert_base, uint64_t expert_stride,
                   const uint8_t *shared_pack, uint32_t n_embd, uint32_t n_ff,
                   float *y, int32_t *ids_out, float *wts_out, float *xn_out);

/* ---- IQ4_NL (ggml type 20): 18-byte blocks of 32 weights, fp16 d + 16 bytes of 4-bit codes;
 * weight j = d * table[qs[j] & 15], weight j + 16 = d * table[qs[j] >> 4]
 * (src/q4_quant.c:270-290).  A routed expert's down projection may use it
 * (src/q4_rocm.cu:4926-4944 lists the accepted types). ---- */
#define Q4O_T_IQ3_S 21u
#define Q4O_T_IQ4_NL 20u
#define Q4O_IQ4NL_BYTES 18
void q4o_iq4nl_dequant_row(const uint8_t *src, uint64_t n, float *dst);
/* I[g] = sum over the 32 weights of block g of table value * q (int32, exact). */
void q4o_iq4nl_group_idot(const uint8_t *row, const q4o_q8 *x, uint64_t n, int32_t *I);
/* Row dot against Q8-A activations in the CPU path's order (src/q4_cpuexp.c:977-996): eight
 * running sums over 4-element slices, one fused multiply-add per block, fixed final tree. */
float q4o_iq4nl_dot8(const uint8_t *row, const q4o_q8 *x, uint64_t n);
/* ---- IQ4_XS (ggml type 23): 136-byte super-blocks of 256 weights: fp16 d, u16 scales_h,
 * scales_l[4], qs[128]; group ib has the 6-bit scale ls = low nibble | two high bits, weight =
 * d * (ls - 32) * table[code] with the IQ4_NL table and nibble order
 * (src/q4_quant.c:455-480; row dot src/q4_cpuexp.c:945-975). ---- */
#define Q4O_T_IQ4_XS 23u
#define Q4O_IQ4XS_BYTES 136
void q4o_iq4xs_dequant_row(const uint8_t *src, uint64_t n, float *dst);
void q4o_iq4xs_group_idot(const uint8_t *row, const q4o_q8 *x, uint64_t n, int32_t *I);
float q4o_iq4xs_dot8(const uint8_t *row, const q4o_q8 *x, uint64_t n);
/* By type id (IQ3_S, IQ4_NL, IQ4_XS). */
uint64_t q4o_row_bytes(uint32_t type, uint64_t ncols);
float q4o_dot8_t(uint32_t type, const uint8_t *row, const q4o_q8 *x, uint64_t n);
/* q4o_expert_ffn / q4o_expert_job with the types of gate+up and of down given. */
void q4o_expert_ffn_t(const uint8_t *pack, const q4o_q8 *xq, uint32_t n_embd, uint32_t n_ff,
                      uint32_t gu_type, uint32_t down_type, float wt, float *y, float *h_out,
                      q4o_q8 *hq_out);
void q4o_expert_job_t(const uint8_t *const *packs, const float *wts, uint32_t k, const float *x,
                      uint32_t n_embd, uint32_t n_ff, uint32_t gu_type, uint32_t down_type, float *y);

/* ---- "Q8-C": the q8_1 block quantiser the reference's grouped prefill GEMM
 * uses (third_party/llama.cpp/ggml/src/ggml-cuda/quantize.cu:491-553):
 * d_inv = 127/amax, q = roundf(x * d_inv) (half away from zero), d = 1/d_inv.
 * Output here is planar: q[n] int8 and d[n/32] float. amax == 0 gives q = 0,
 * d = 0 (the reference leaves that case undefined). */
void q4o_quant8_mmq(const float *x, uint64_t n, int8_t *q, float *d);

/* Row dot in the grouped-GEMM order (mmq-load-tiles.cuh:1387-1424,
 * mmq-vec-dot.cuh:189-197,266-273): for groups g ascending
 *   sum = sum + ((float)C_g * dA_g) * dB_g,  dA_g = (float)(1+2 s_g) * d. */
float q4o_iq3s_dot_mmq(const uint8_t *row, const int8_t *q, const float *dq,
                       uint64_t n);

/* ---- dense product of up to 8 activation rows in 8-bit form (src/q4_mmvq.cu) ---- */
#define Q4O_T_Q4_K 12u
#define Q4O_T_Q5_K 13u
#define Q4O_T_Q6_K 14u
/* src/q4_mmvq.cu:36-57: q = rint(v / d), d = amax / 127 per 32 values; s16 = sums per 16 */
void q4o_quant8_d(const float *x, uint64_t n, int8_t *q, float *d, int32_t *s16);
/* bytes and values per block of a type this product takes; 0 = not one of them */
int q4o_mv_geometry(uint32_t type, uint32_t *block_bytes, uint32_t *block_vals);
/* a * w + c of every run: pins the run decoders against the reference's q4_dequant_row */
void q4o_mv_dequant_row(uint32_t type, const uint8_t *row, uint64_t n, float *dst);
/* src/q4_mmvq.cu:195-243: one weight row x one quantised activation row, unscaled */
float q4o_mv_row(uint32_t type, const uint8_t *row, uint64_t n, const int8_t *q, const float *d,
                 const int32_t *s16);

/* ---- other routed-expert formats: IQ3_XXS (18), IQ2_S (22) for gate/up, Q2_0 (42) for down ---- */
#define Q4O_T_IQ3_XXS 18u
#define Q4O_T_IQ2_S 22u
#define Q4O_T_Q2_0 42u
/* src/q4_quant.c:424-452, :290-322, :177-188 */
void q4o_dequant_row_x(uint32_t type, const uint8_t *src, uint64_t n, float *dst);
/* exact integer part of every 32-group's dot (before sub-scales; Q2_0: codes 0..3 x q) */
void q4o_group_idot_x(uint32_t type, const uint8_t *row, const q4o_q8 *x, uint64_t n, int32_t *I);
/* src/q4_cpuexp.c:895-931, :814-852, :1113-1145; q4o_dot8_t and q4o_expert_job_t take these types too */
float q4o_dot8_x(uint32_t type, const uint8_t *row, const q4o_q8 *x, uint64_t n);

#ifdef __cplusplus
}
#endif
#endif
