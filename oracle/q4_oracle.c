/* CPU oracle for the IQ3_S x 8-bit-activation MoE feed-forward path.
 *
 * TEST INFRASTRUCTURE ONLY: a checker for the CUDA library, never part of it.
 * Parity status: PINNED (see q4_oracle.h).  Scalar C on purpose: every
 * operation and its rounding is visible.  Build with -ffp-contract=off so the
 * compiler fuses nothing that is not written as fmaf().
 *
 * Citations are file:line in the reference project.
 */
#include "q4_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "iq3s_codes.h"
#include "iq4nl_codes.h"

uint32_t q4o_iq3s_grid(uint32_t idx) {
    const uint32_t c = q4b_iq3s_codes[idx & 511u];
    uint32_t w = 0;
    for (int j = 0; j < 4; j++) w |= (2u * ((c >> (3 * j)) & 7u) + 1u) << (8 * j);
    return w;
}

float q4o_f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h >> 15) << 31;
    const uint32_t ex = (h >> 10) & 31u;
    uint32_t man = h & 1023u;
    uint32_t bits;
    if (ex == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal half: renormalise */
            int e = -1;
            do {
                e++;
                man <<= 1;
            } while (!(man & 1024u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 1023u) << 13);
        }
    } else if (ex == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((ex + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* Field offsets inside one 110-byte super-block (src/q4_quant.c:391-394). */
enum { OFF_QS = 2, OFF_QH = 66, OFF_SIGNS = 74, OFF_SCALES = 106 };

void q4o_iq3s_unpack(const uint8_t *blk, int8_t w[256], uint8_t ls[8], float *d) {
    uint16_t dh;
    memcpy(&dh, blk, 2);
    if (d) *d = q4o_f16_to_f32(dh);
    for (int ib = 0; ib < 8; ib++) {
        const uint8_t sb = blk[OFF_SCALES + ib / 2];
        ls[ib] = (uint8_t)(1 + 2 * ((ib & 1) ? (sb >> 4) : (sb & 15)));
        const uint8_t qh = blk[OFF_QH + ib];
        for (int k = 0; k < 8; k++) { /* k-th codebook index of this sub-block */
            const uint32_t idx = blk[OFF_QS + 8 * ib + k] | (((uint32_t)(qh >> k) & 1u) << 8);
            const uint32_t g = q4o_iq3s_grid(idx);
            const uint8_t sg = blk[OFF_SIGNS + 4 * ib + k / 2];
            for (int j = 0; j < 4; j++) {
                const int mag = (int)((g >> (8 * j)) & 0xff);
                const int neg = (sg >> (4 * (k & 1) + j)) & 1;
                w[32 * ib + 4 * k + j] = (int8_t)(neg ? -mag : mag);
            }
        }
    }
}

void q4o_iq3s_dequant_row(const uint8_t *src, uint64_t n, float *dst) {
    int8_t w[256];
    uint8_t ls[8];
    float d;
    for (uint64_t b = 0; b < n / Q4O_QK_K; b++) {
        q4o_iq3s_unpack(src + b * Q4O_IQ3S_BYTES, w, ls, &d);
        for (int ib = 0; ib < 8; ib++) {
            /* src/q4_quant.c:397-398: db = d * (1.f + 2.f * s) */
            const float db = d * (1.f + 2.f * (float)((ls[ib] - 1) / 2));
            for (int i = 0; i < 32; i++) {
                const int v = w[32 * ib + i];
                /* src/q4_quant.c:409: db * magnitude * (+-1) */
                dst[b * 256 + 32 * ib + i] = db * (float)abs(v) * (v < 0 ? -1.f : 1.f);
            }
        }
    }
}

void q4o_quant8(const float *x, uint64_t n, q4o_q8 *out) {
    for (uint64_t g = 0; g < n / 32; g++) {
        const float *xb = x + 32 * g;
        float a = 0.f;
        for (int i = 0; i < 32; i++) {
            const float v = fabsf(xb[i]);
            if (v > a) a = v;
        }
        out[g].d = a / 127.f;
        const float sc = a > 0.f ? 127.f / a : 0.f;
        int32_t bs = 0;
        for (int i = 0; i < 32; i++) {
            /* cvtps2dq under the default rounding mode = nearest even */
            long q = lrintf(xb[i] * sc);
            if (q > 127) q = 127;
            if (q < -128) q = -128;
            out[g].q[i] = (int8_t)q;
            bs += (int32_t)q;
        }
        out[g].bs = bs;
    }
}

void q4o_iq3s_group_idot(const uint8_t *row, const q4o_q8 *x, uint64_t n, int32_t *I) {
    int8_t w[256];
    uint8_t ls[8];
    for (uint64_t b = 0; b < n / Q4O_QK_K; b++) {
        q4o_iq3s_unpack(row + b * Q4O_IQ3S_BYTES, w, ls, NULL);
        for (int ib = 0; ib < 8; ib++) {
            int32_t s = 0;
            for (int i = 0; i < 32; i++) s += (int32_t)w[32 * ib + i] * x[8 * b + ib].q[i];
            I[8 * b + ib] = s;
        }
    }
}

float q4o_iq3s_dot8(const uint8_t *row, const q4o_q8 *x, uint64_t n) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int8_t w[256];
    uint8_t ls[8];
    float d;
    for (uint64_t b = 0; b < n / Q4O_QK_K; b++) {
        q4o_iq3s_unpack(row + b * Q4O_IQ3S_BYTES, w, ls, &d);
        for (int ib = 0; ib < 8; ib++) {
            const q4o_q8 *xg = x + 8 * b + ib;
            const float dd = d * xg->d; /* src/q4_cpuexp.c:884 */
            for (int lane = 0; lane < 8; lane++) {
                int32_t s = 0;
                for (int t = 0; t < 4; t++) s += (int32_t)w[32 * ib + 4 * lane + t] * xg->q[4 * lane + t];
                /* maddubs + madd by the 16-bit sub-scale, then cvt + fmadd
                 * (src/q4_cpuexp.c:694-699,881-887) */
                acc[lane] = fmaf(dd, (float)(s * (int32_t)ls[ib]), acc[lane]);
            }
        }
    }
    /* src/q4_cpuexp.c:39-46 */
    return ((acc[0] + acc[4]) + (acc[2] + acc[6])) + ((acc[1] + acc[5]) + (acc[3] + acc[7]));
}

float q4o_silu(float v) { return v / (1.f + expf(-v)); }

void q4o_expert_ffn(const uint8_t *pack, const q4o_q8 *xq, uint32_t n_embd,
                    uint32_t n_ff, float wt, float *y, float *h_out,
                    q4o_q8 *hq_out) {
    const uint64_t rb_gu = (uint64_t)(n_embd / Q4O_QK_K) * Q4O_IQ3S_BYTES;
    const uint64_t rb_d = (uint64_t)(n_ff / Q4O_QK_K) * Q4O_IQ3S_BYTES;
    const uint8_t *gate = pack;
    const uint8_t *up = pack + (uint64_t)n_ff * rb_gu;
    const uint8_t *down = up + (uint64_t)n_ff * rb_gu;
    float *h = (float *)malloc(sizeof(float) * n_ff);
    q4o_q8 *hq = (q4o_q8 *)malloc(sizeof(q4o_q8) * (n_ff / 32));
    for (uint32_t r = 0; r < n_ff; r++) {
        const float gv = q4o_iq3s_dot8(gate + r * rb_gu, xq, n_embd);
        const float uv = q4o_iq3s_dot8(up + r * rb_gu, xq, n_embd);
        h[r] = q4o_silu(gv) * uv;
    }
    q4o_quant8(h, n_ff, hq);
    for (uint32_t r = 0; r < n_embd; r++) {
        const float dv = q4o_iq3s_dot8(down + r * rb_d, hq, n_ff);
        const float t = wt * dv;
        y[r] = y[r] + t;
    }
    if (h_out) memcpy(h_out, h, sizeof(float) * n_ff);
    if (hq_out) memcpy(hq_out, hq, sizeof(q4o_q8) * (n_ff / 32));
    free(h);
    free(hq);
}

/* ---- IQ4_NL ---- */
static const int8_t q4o_iq4nl_values[16] = Q4B_IQ4NL_VALUES;

void q4o_iq4nl_dequant_row(const uint8_t *src, uint64_t n, float *dst) {
    for (uint64_t b = 0; b < n / 32; b++) {
        const uint8_t *blk = src + b * Q4O_IQ4NL_BYTES;
        const float d = q4o_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        for (int j = 0; j < 16; j++) {
            dst[32 * b + j] = d * (float)q4o_iq4nl_values[blk[2 + j] & 0xf];
            dst[32 * b + j + 16] = d * (float)q4o_iq4nl_values[blk[2 + j] >> 4];
        }
    }
}

static void iq4nl_unpack(const uint8_t *blk, int8_t w[32]) {
    for (int j = 0; j < 16; j++) {
        w[j] = q4o_iq4nl_values[blk[2 + j] & 0xf];
        w[j + 16] = q4o_iq4nl_values[blk[2 + j] >> 4];
    }
}

void q4o_iq4nl_group_idot(const uint8_t *row, const q4o_q8 *x, uint64_t n, int32_t *I) {
    int8_t w[32];
    for (uint64_t b = 0; b < n / 32; b++) {
        iq4nl_unpack(row + b * Q4O_IQ4NL_BYTES, w);
        int32_t s = 0;
        for (int i = 0; i < 32; i++) s += (int32_t)w[i] * x[b].q[i];
        I[b] = s;
    }
}

float q4o_iq4nl_dot8(const uint8_t *row, const q4o_q8 *x, uint64_t n) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int8_t w[32];
    for (uint64_t b = 0; b < n / 32; b++) {
        const uint8_t *blk = row + b * Q4O_IQ4NL_BYTES;
        iq4nl_unpack(blk, w);
        const float dd = q4o_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8))) * x[b].d; /* :989 */
        for (int lane = 0; lane < 8; lane++) {
            int32_t s = 0;
            for (int t = 0; t < 4; t++) s += (int32_t)w[4 * lane + t] * x[b].q[4 * lane + t];
            acc[lane] = fmaf(dd, (float)s, acc[lane]); /* src/q4_cpuexp.c:988-993 */
        }
    }
    return ((acc[0] + acc[4]) + (acc[2] + acc[6])) + ((acc[1] + acc[5]) + (acc[3] + acc[7]));
}

/* ---- IQ4_XS ---- */
static int iq4xs_ls(const uint8_t *blk, int ib) {
    const uint16_t sh = (uint16_t)(blk[2] | (blk[3] << 8));
    return ((blk[4 + ib / 2] >> (4 * (ib % 2))) & 0xf) | ((int)((sh >> (2 * ib)) & 3) << 4);
}
static void iq4xs_unpack_group(const uint8_t *blk, int ib, int8_t w[32]) {
    const uint8_t *qs = blk + 8 + 16 * ib;
    for (int j = 0; j < 16; j++) {
        w[j] = q4o_iq4nl_values[qs[j] & 0xf];
        w[j + 16] = q4o_iq4nl_values[qs[j] >> 4];
    }
}

void q4o_iq4xs_dequant_row(const uint8_t *src, uint64_t n, float *dst) {
    int8_t w[32];
    for (uint64_t b = 0; b < n / Q4O_QK_K; b++) {
        const uint8_t *blk = src + b * Q4O_IQ4XS_BYTES;
        const float d = q4o_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        for (int ib = 0; ib < 8; ib++) {
            const float dl = d * (float)(iq4xs_ls(blk, ib) - 32);
            iq4xs_unpack_group(blk, ib, w);
            for (int j = 0; j < 32; j++) dst[256 * b + 32 * ib + j] = dl * (float)w[j];
        }
    }
}

void q4o_iq4xs_group_idot(const uint8_t *row, const q4o_q8 *x, uint64_t n, int32_t *I) {
    int8_t w[32];
    for (uint64_t b = 0; b < n / Q4O_QK_K; b++)
        for (int ib = 0; ib < 8; ib++) {
            iq4xs_unpack_group(row + b * Q4O_IQ4XS_BYTES, ib, w);
            int32_t s = 0;
            for (int i = 0; i < 32; i++) s += (int32_t)w[i] * x[8 * b + ib].q[i];
            I[8 * b + ib] = s;
        }
}

float q4o_iq4xs_dot8(const uint8_t *row, const q4o_q8 *x, uint64_t n) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int8_t w[32];
    for (uint64_t b = 0; b < n / Q4O_QK_K; b++) {
        const uint8_t *blk = row + b * Q4O_IQ4XS_BYTES;
        const float d = q4o_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        for (int ib = 0; ib < 8; ib++) {
            const q4o_q8 *xg = x + 8 * b + ib;
            const int ls = iq4xs_ls(blk, ib) - 32;
            iq4xs_unpack_group(blk, ib, w);
            const float dd = d * xg->d; /* src/q4_cpuexp.c:968 */
            for (int lane = 0; lane < 8; lane++) {
                int32_t s = 0;
                for (int t = 0; t < 4; t++) s += (int32_t)w[4 * lane + t] * xg->q[4 * lane + t];
                acc[lane] = fmaf(dd, (float)(s * ls), acc[lane]); /* :966-972 */
            }
        }
    }
    return ((acc[0] + acc[4]) + (acc[2] + acc[6])) + ((acc[1] + acc[5]) + (acc[3] + acc[7]));
}

float q4o_dot8_x(uint32_t type, const uint8_t *row, const q4o_q8 *x, uint64_t n);
uint64_t q4o_row_bytes(uint32_t type, uint64_t ncols) {
    if (type == Q4O_T_IQ3_XXS) return (ncols / Q4O_QK_K) * 98;
    if (type == Q4O_T_IQ2_S) return (ncols / Q4O_QK_K) * 82;
    if (type == Q4O_T_Q2_0) return (ncols / 64) * 18;
    if (type == Q4O_T_IQ4_NL) return (ncols / 32) * Q4O_IQ4NL_BYTES;
    if (type == Q4O_T_IQ4_XS) return (ncols / Q4O_QK_K) * Q4O_IQ4XS_BYTES;
    return (ncols / Q4O_QK_K) * Q4O_IQ3S_BYTES;
}

float q4o_dot8_t(uint32_t type, const uint8_t *row, const q4o_q8 *x, uint64_t n) {
    if (type == Q4O_T_IQ3_XXS || type == Q4O_T_IQ2_S || type == Q4O_T_Q2_0) return q4o_dot8_x(type, row, x, n);
    if (type == Q4O_T_IQ4_NL) return q4o_iq4nl_dot8(row, x, n);
    if (type == Q4O_T_IQ4_XS) return q4o_iq4xs_dot8(row, x, n);
    return q4o_iq3s_dot8(row, x, n);
}

void q4o_expert_ffn_t(const uint8_t *pack, const q4o_q8 *xq, uint32_t n_embd, uint32_t n_ff,
                      uint32_t gu_type, uint32_t down_type, float wt, float *y, float *h_out,
                      q4o_q8 *hq_out) {
    const uint64_t rb_gu = q4o_row_bytes(gu_type, n_embd), rb_d = q4o_row_bytes(down_type, n_ff);
    const uint8_t *gate = pack, *up = pack + (uint64_t)n_ff * rb_gu, *down = up + (uint64_t)n_ff * rb_gu;
    float *h = (float *)malloc(sizeof(float) * n_ff);
    q4o_q8 *hq = (q4o_q8 *)malloc(sizeof(q4o_q8) * (n_ff / 32));
    for (uint32_t r = 0; r < n_ff; r++)
        h[r] = q4o_silu(q4o_dot8_t(gu_type, gate + r * rb_gu, xq, n_embd)) *
               q4o_dot8_t(gu_type, up + r * rb_gu, xq, n_embd);
    q4o_quant8(h, n_ff, hq);
    for (uint32_t r = 0; r < n_embd; r++) {
        const float t = wt * q4o_dot8_t(down_type, down + r * rb_d, hq, n_ff);
        y[r] = y[r] + t;
    }
    if (h_out) memcpy(h_out, h, sizeof(float) * n_ff);
    if (hq_out) memcpy(hq_out, hq, sizeof(q4o_q8) * (n_ff / 32));
    free(h);
    free(hq);
}

void q4o_expert_job_t(const uint8_t *const *packs, const float *wts, uint32_t k, const float *x,
                      uint32_t n_embd, uint32_t n_ff, uint32_t gu_type, uint32_t down_type, float *y) {
    q4o_q8 *xq = (q4o_q8 *)malloc(sizeof(q4o_q8) * (n_embd / 32));
    q4o_quant8(x, n_embd, xq);
    memset(y, 0, sizeof(float) * n_embd);
    for (uint32_t e = 0; e < k; e++)
        q4o_expert_ffn_t(packs[e], xq, n_embd, n_ff, gu_type, down_type, wts[e], y, NULL, NULL);
    free(xq);
}

void q4o_expert_job(const uint8_t *const *packs, const float *wts, uint32_t k,
                    const float *x, uint32_t n_embd, uint32_t n_ff, float *y) {
    q4o_q8 *xq = (q4o_q8 *)malloc(sizeof(q4o_q8) * (n_embd / 32));
    q4o_quant8(x, n_embd, xq);
    memset(y, 0, sizeof(float) * n_embd);
    for (uint32_t e = 0; e < k; e++)
        q4o_expert_ffn(packs[e], xq, n_embd, n_ff, wts[e], y, NULL, NULL);
    free(xq);
}

void q4o_rms_norm(const float *x, const float *w, float *y, uint64_t n, float eps) {
    double ss = 0;
    for (uint64_t i = 0; i < n; i++) ss += (double)x[i] * (double)x[i];
    const float scale = 1.0f / sqrtf((float)(ss / (double)n) + eps);
    for (uint64_t i = 0; i < n; i++) {
        const float t = x[i] * scale;
        y[i] = w ? t * w[i] : t;
    }
}

void q4o_gemv_f32(const float *W, uint64_t nrows, uint64_t ncols, const float *x,
                  float *y) {
    for (uint64_t r = 0; r < nrows; r++) {
        const float *a = W + r * ncols;
        float s = 0;
        uint64_t i = 0;
        for (; i + 8 <= ncols; i += 8) {
            float t = a[i] * x[i];
            for (int j = 1; j < 8; j++) t = t + a[i + j] * x[i + j];
            s = s + t;
        }
        for (; i < ncols; i++) s = s + a[i] * x[i];
        y[r] = s;
    }
}

void q4o_softmax(float *x, uint64_t n) {
    float m = x[0];
    for (uint64_t i = 1; i < n; i++)
        if (x[i] > m) m = x[i];
    float s = 0;
    for (uint64_t i = 0; i < n; i++) {
        x[i] = expf(x[i] - m);
        s = s + x[i];
    }
    const float inv = s > 0 ? 1.0f / s : 0;
    for (uint64_t i = 0; i < n; i++) x[i] = x[i] * inv;
}

void q4o_topk(const float *p, uint32_t n, uint32_t k, int32_t *ids, float *wts,
              int renormalize) {
    if (k > n) k = n;
    uint32_t have = 0;
    for (uint32_t i = 0; i < n; i++) {
        /* position of p[i] among the kept entries: after every entry that is
         * greater or equal (equal values keep the earlier index in front) */
        uint32_t pos = have;
        while (pos > 0 && p[i] > wts[pos - 1]) pos--;
        if (pos >= k) continue;
        const uint32_t last = have < k ? have : k - 1;
        for (uint32_t j = last; j > pos; j--) {
            ids[j] = ids[j - 1];
            wts[j] = wts[j - 1];
        }
        ids[pos] = (int32_t)i;
        wts[pos] = p[i];
        if (have < k) have++;
    }
    if (renormalize) {
        float s = 0;
        for (uint32_t i = 0; i < k; i++) s = s + wts[i];
        if (s > 0) {
            const float inv = 1.0f / s;
            for (uint32_t i = 0; i < k; i++) wts[i] = wts[i] * inv;
        }
    }
}

void q4o_moe_layer(const float *x, const float *norm_w, float eps,
                   const float *router_w, uint32_t n_expert, uint32_t topk,
                   const uint8_t *expert_base, uint64_t expert_stride,
                   const uint8_t *shared_pack, uint32_t n_embd, uint32_t n_ff,
                   float *y, int32_t *ids_out, float *wts_out, float *xn_out) {
    float *xn = (float *)malloc(sizeof(float) * n_embd);
    float *p = (float *)malloc(sizeof(float) * n_expert);
    int32_t *ids = (int32_t *)malloc(sizeof(int32_t) * (topk + 1));
    float *wts = (float *)malloc(sizeof(float) * (topk + 1));
    const uint8_t **packs = (const uint8_t **)malloc(sizeof(void *) * (topk + 1));
    q4o_rms_norm(x, norm_w, xn, n_embd, eps);
    q4o_gemv_f32(router_w, n_expert, n_embd, xn, p);
    q4o_softmax(p, n_expert);
    q4o_topk(p, n_expert, topk, ids, wts, 1);
    uint32_t k = topk;
    for (uint32_t i = 0; i < topk; i++) packs[i] = expert_base + (uint64_t)ids[i] * expert_stride;
    if (shared_pack) {
        packs[k] = shared_pack;
        wts[k] = 1.0f;
        k++;
    }
    q4o_expert_job(packs, wts, k, xn, n_embd, n_ff, y);
    if (ids_out) memcpy(ids_out, ids, sizeof(int32_t) * topk);
    if (wts_out) memcpy(wts_out, wts, sizeof(float) * topk);
    if (xn_out) memcpy(xn_out, xn, sizeof(float) * n_embd);
    free(xn);
    free(p);
    free(ids);
    free(wts);
    free(packs);
}

void q4o_quant8_mmq(const float *x, uint64_t n, int8_t *q, float *d) {
    for (uint64_t g = 0; g < n / 32; g++) {
        const float *xb = x + 32 * g;
        float amax = 0.f;
        for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(xb[i]));
        if (!(amax > 0.f)) {
            memset(q + 32 * g, 0, 32);
            d[g] = 0.f;
            continue;
        }
        const float d_inv = 127.0f / amax;
        for (int i = 0; i < 32; i++) q[32 * g + i] = (int8_t)roundf(xb[i] * d_inv);
        d[g] = 1.0f / d_inv;
    }
}

float q4o_iq3s_dot_mmq(const uint8_t *row, const int8_t *q, const float *dq,
                       uint64_t n) {
    int8_t w[256];
    uint8_t ls[8];
    float d;
    float sum = 0.f;
    for (uint64_t b = 0; b < n / Q4O_QK_K; b++) {
        q4o_iq3s_unpack(row + b * Q4O_IQ3S_BYTES, w, ls, &d);
        for (int ib = 0; ib < 8; ib++) {
            int32_t c = 0;
            for (int i = 0; i < 32; i++) c += (int32_t)w[32 * ib + i] * q[256 * b + 32 * ib + i];
            const float dA = (float)ls[ib] * d;
            const float t = (float)c * dA;
            sum = sum + t * dq[8 * b + ib];
        }
    }
    return sum;
}

/* ---- dense product of up to 8 activation rows in 8-bit form (src/q4_mmvq.cu) ----
 * Weight types: Q6_K, Q4_K, Q5_K (public ggml K-quant block formats), IQ4_XS, IQ4_NL.
 * The unit of work is a run of 16 consecutive weights that share one scale: every value in
 * it is a * w_i + c with integer w_i, so its dot with 16 quantised activations of scale dx is
 * dx * (a * sum(w_i q_i) + c * sum(q_i)). */

/* src/q4_mmvq.cu:36-57: per 32 values d = amax / 127, q = rint(v / d) (a division, not a
 * product with the reciprocal), and the integer sum of each half of the group. */
void q4o_quant8_d(const float *x, uint64_t n, int8_t *q, float *d, int32_t *s16) {
    for (uint64_t g = 0; g < n / 32; g++) {
        const float *xb = x + 32 * g;
        float a = 0.f;
        for (int i = 0; i < 32; i++) a = fmaxf(a, fabsf(xb[i]));
        const float dg = a / 127.f;
        int32_t s[2] = {0, 0};
        for (int i = 0; i < 32; i++) {
            const int v = dg > 0.f ? (int)rintf(xb[i] / dg) : 0;
            q[32 * g + i] = (int8_t)v;
            s[i >> 4] += v;
        }
        d[g] = dg;
        s16[2 * g] = s[0];
        s16[2 * g + 1] = s[1];
    }
}

static float mv_f16(const uint8_t *p) { return q4o_f16_to_f32((uint16_t)(p[0] | (p[1] << 8))); }

/* 6-bit scale and minimum of 32-value sub-block j out of the 12 packed bytes of a Q4_K /
 * Q5_K block: j < 4 sits in the low 6 bits of bytes j and j + 4; j >= 4 takes its low
 * nibbles from byte j + 4 and its two high bits from the top of bytes j - 4 and j. */
static void mv_k_scale_min(const uint8_t *p, int j, int *sc, int *mn) {
    if (j < 4) {
        *sc = p[j] & 63;
        *mn = p[j + 4] & 63;
    } else {
        *sc = (p[j + 4] & 15) | ((p[j - 4] >> 6) << 4);
        *mn = (p[j + 4] >> 4) | ((p[j] >> 6) << 4);
    }
}

int q4o_mv_geometry(uint32_t type, uint32_t *block_bytes, uint32_t *block_vals) {
    uint32_t bb = 0, bv = 256;
    switch (type) {
    case Q4O_T_Q6_K: bb = 210; break;
    case Q4O_T_Q4_K: bb = 144; break;
    case Q4O_T_Q5_K: bb = 176; break;
    case Q4O_T_IQ4_XS: bb = 136; break;
    case Q4O_T_IQ4_NL: bb = 18; bv = 32; break;
    default: return 0;
    }
    if (block_bytes) *block_bytes = bb;
    if (block_vals) *block_vals = bv;
    return 1;
}

/* Run r (16 values) of a block: the integer weights, the scale a, the offset c and the
 * position of its first value inside the block (src/q4_mmvq.cu:101-190). */
static void mv_run(uint32_t type, const uint8_t *blk, int r, int32_t w[16], float *a, float *c, int *first) {
    *c = 0.f;
    if (type == Q4O_T_Q6_K) {
        /* ql[128] | qh[64] | int8 scales[16] | f16 d.  Each half of the block (128 values) is
         * four strips of 32: strip s takes its low nibbles from ql bytes 32*(s&1)..+31 of the
         * half (upper nibble for s >= 2) and its two high bits from bits 2s..2s+1 of the
         * half's 32 qh bytes.  Stored values are offset by 32. */
        const int half = r >> 3, strip = (r >> 1) & 3, lo = (r & 1) * 16;
        const uint8_t *ql = blk + 64 * half + 32 * (strip & 1) + lo;
        const uint8_t *qh = blk + 128 + 32 * half + lo;
        for (int i = 0; i < 16; i++)
            w[i] = ((ql[i] >> (4 * (strip >> 1))) & 15) | (((qh[i] >> (2 * strip)) & 3) << 4);
        *a = mv_f16(blk + 208) * (float)(int8_t)blk[192 + 8 * half + 2 * strip + (r & 1)];
        *c = -32.f * *a;
        *first = 128 * half + 32 * strip + lo;
        return;
    }
    if (type == Q4O_T_Q4_K || type == Q4O_T_Q5_K) {
        /* f16 d | f16 dmin | scales[12] | (Q5_K: qh[32]) | qs[128].  Sub-block j = r / 2 (32
         * values): sub-blocks 2p and 2p + 1 are the low and high nibbles of qs bytes 32p..32p+31;
         * Q5_K adds bit j of qh byte l as bit 4 of value l. */
        const int j = r >> 1, lo = (r & 1) * 16;
        const uint8_t *qs = blk + (type == Q4O_T_Q5_K ? 48 : 16) + 32 * (j >> 1) + lo;
        for (int i = 0; i < 16; i++) {
            w[i] = (qs[i] >> (4 * (j & 1))) & 15;
            if (type == Q4O_T_Q5_K) w[i] |= ((blk[16 + lo + i] >> j) & 1) << 4;
        }
        int sc, mn;
        mv_k_scale_min(blk + 4, j, &sc, &mn);
        *a = mv_f16(blk) * (float)sc;
        *c = -mv_f16(blk + 2) * (float)mn;
        *first = 32 * j + lo;
        return;
    }
    /* IQ4_XS group r / 2 of the block, IQ4_NL the block itself: run r & 1 is the low (0) or high
     * (1) nibbles of the group's 16 bytes, looked up in the 16-value codebook */
    const int ib = r >> 1, hi = r & 1;
    const uint8_t *qs = type == Q4O_T_IQ4_XS ? blk + 8 + 16 * ib : blk + 2;
    for (int i = 0; i < 16; i++) w[i] = q4o_iq4nl_values[(qs[i] >> (4 * hi)) & 15];
    *a = type == Q4O_T_IQ4_XS ? mv_f16(blk) * (float)(iq4xs_ls(blk, ib) - 32) : mv_f16(blk);
    *first = 32 * ib + 16 * hi;
}

void q4o_mv_dequant_row(uint32_t type, const uint8_t *row, uint64_t n, float *dst) {
    uint32_t bb, bv;
    if (!q4o_mv_geometry(type, &bb, &bv)) return;
    for (uint64_t b = 0; b < n / bv; b++)
        for (int r = 0; r < (int)bv / 16; r++) {
            int32_t w[16];
            float a, c;
            int first;
            mv_run(type, row + b * bb, r, w, &a, &c, &first);
            for (int i = 0; i < 16; i++) dst[b * bv + (uint64_t)first + i] = a * (float)w[i] + c;
        }
}

/* One weight row against one quantised activation row, before the caller's scale
 * (src/q4_mmvq.cu:195-243): 32 lanes take the row's runs round robin, each lane adds
 * dx * (a * s + c * sum16) to its own accumulator with explicit fused multiply-adds, and the
 * lanes are summed by the butterfly (offsets 16, 8, 4, 2, 1).  Nothing here depends on how
 * many activation rows the call has. */
float q4o_mv_row(uint32_t type, const uint8_t *row, uint64_t n, const int8_t *q, const float *d,
                 const int32_t *s16) {
    uint32_t bb, bv;
    if (!q4o_mv_geometry(type, &bb, &bv)) return 0.f;
    const uint32_t rpb = bv / 16;
    const uint64_t n_runs = n / 16;
    const int has_c = type == Q4O_T_Q6_K || type == Q4O_T_Q4_K || type == Q4O_T_Q5_K;
    float acc[32];
    for (int lane = 0; lane < 32; lane++) {
        acc[lane] = 0.f;
        for (uint64_t t = (uint64_t)lane; t < n_runs; t += 32) {
            const uint64_t b = t / rpb;
            int32_t w[16];
            float a, c;
            int first;
            mv_run(type, row + b * bb, (int)(t % rpb), w, &a, &c, &first);
            const uint64_t e0 = b * bv + (uint64_t)first;
            int32_t s = 0;
            for (int i = 0; i < 16; i++) s += w[i] * (int32_t)q[e0 + i];
            float v = a * (float)s;
            if (has_c) v = fmaf(c, (float)s16[e0 >> 4], v);
            acc[lane] = fmaf(d[e0 >> 5], v, acc[lane]);
        }
    }
    for (int o = 16; o; o >>= 1) {
        float nx[32];
        for (int lane = 0; lane < 32; lane++) nx[lane] = acc[lane] + acc[lane ^ o];
        memcpy(acc, nx, sizeof acc);
    }
    return acc[0];
}

/* ---- the other formats a routed expert's projections may come in (src/q4_rocm.cu:4926-4944):
 * IQ3_XXS and IQ2_S (gate, up), Q2_0 (down).  Block layouts are the public ggml ones; the codebooks are
 * kept as packed level numbers (iq3xxs_codes.h, iq2s_codes.h). ---- */
#include "iq2s_codes.h"
#include "iq3xxs_codes.h"

static const uint8_t q4o_iq3xxs_levels[8] = {4, 12, 20, 28, 36, 44, 52, 62};
static const uint8_t q4o_iq2s_levels[3] = {8, 25, 43};
/* the 128-entry sign table of the IQ2/IQ3 "xxs" formats: seven stored bits, the eighth makes the
 * parity even (src/q4_iq_grids.inc: q4_ksigns_iq2xs) */
static uint8_t q4o_sign8(uint32_t i7) { return (uint8_t)(i7 | ((uint32_t)(__builtin_popcount(i7) & 1) << 7)); }

/* One 32-value group of a 256-value block: magnitudes (unsigned), sign bits (bit i: value i is
 * negative), the sub-scale of each of the eight 4-value lanes, and the block's fp16 d. */
typedef struct {
    uint8_t mag[32];
    uint32_t neg;
    int32_t ls[8];
} q4o_grp;

static float iq3xxs_group(const uint8_t *blk, int ib, q4o_grp *g) {
    const uint8_t *qs = blk + 2 + 8 * ib;
    const uint32_t aux = (uint32_t)blk[66 + 4 * ib] | ((uint32_t)blk[67 + 4 * ib] << 8) |
                         ((uint32_t)blk[68 + 4 * ib] << 16) | ((uint32_t)blk[69 + 4 * ib] << 24);
    g->neg = 0;
    for (int l = 0; l < 4; l++) {          /* eight values: two codebook entries, one sign byte */
        g->neg |= (uint32_t)q4o_sign8((aux >> (7 * l)) & 127u) << (8 * l);
        for (int h = 0; h < 2; h++) {
            const uint16_t code = q4b_iq3xxs_codes[qs[2 * l + h]];
            for (int j = 0; j < 4; j++) g->mag[8 * l + 4 * h + j] = q4o_iq3xxs_levels[(code >> (3 * j)) & 7];
        }
    }
    for (int lane = 0; lane < 8; lane++) g->ls[lane] = (int32_t)(aux >> 28);   /* raw 4-bit scale */
    return mv_f16(blk);
}

static float iq2s_group(const uint8_t *blk, int ib, q4o_grp *g) {
    const uint8_t *qs = blk + 2 + 4 * ib, *signs = blk + 34 + 4 * ib;
    const uint32_t qh = blk[66 + ib], sb = blk[74 + ib];
    g->neg = 0;
    for (int l = 0; l < 4; l++) {          /* eight values: one codebook entry, one sign byte */
        const uint32_t idx = qs[l] | ((qh << (8 - 2 * l)) & 0x300u);
        const uint16_t code = q4b_iq2s_codes[idx];
        for (int j = 0; j < 8; j++) g->mag[8 * l + j] = q4o_iq2s_levels[(code >> (2 * j)) & 3];
        g->neg |= (uint32_t)signs[l] << (8 * l);
    }
    for (int lane = 0; lane < 8; lane++) g->ls[lane] = (int32_t)(lane < 4 ? (sb & 15u) : (sb >> 4));
    return mv_f16(blk);
}

/* src/q4_quant.c:424-452 (IQ3_XXS), :290-322 (IQ2_S), :177-188 (Q2_0) */
void q4o_dequant_row_x(uint32_t type, const uint8_t *src, uint64_t n, float *dst) {
    if (type == Q4O_T_Q2_0) {
        for (uint64_t b = 0; b < n / 64; b++) {
            const uint8_t *blk = src + b * 18;
            const float d = mv_f16(blk);
            for (int j = 0; j < 64; j++)
                dst[64 * b + j] = d * (float)((int)((blk[2 + j / 4] >> ((j % 4) * 2)) & 3) - 1);
        }
        return;
    }
    const uint32_t bb = type == Q4O_T_IQ3_XXS ? 98 : 82;
    for (uint64_t b = 0; b < n / Q4O_QK_K; b++)
        for (int ib = 0; ib < 8; ib++) {
            q4o_grp g;
            const float d = type == Q4O_T_IQ3_XXS ? iq3xxs_group(src + b * bb, ib, &g) : iq2s_group(src + b * bb, ib, &g);
            for (int i = 0; i < 32; i++) {
                const float sub = 0.5f + (float)g.ls[i >> 2];
                const float db = type == Q4O_T_IQ3_XXS ? d * sub * 0.5f : d * sub * 0.25f;
                dst[256 * b + 32 * ib + i] = db * (float)g.mag[i] * ((g.neg >> i) & 1u ? -1.f : 1.f);
            }
        }
}

void q4o_group_idot_x(uint32_t type, const uint8_t *row, const q4o_q8 *x, uint64_t n, int32_t *I) {
    if (type == Q4O_T_Q2_0) {              /* per 32 values: sum of code x q (codes 0..3, value = code - 1) */
        for (uint64_t gi = 0; gi < n / 32; gi++) {
            const uint8_t *qs = row + (gi / 2) * 18 + 2 + 8 * (gi & 1);
            int32_t s = 0;
            for (int i = 0; i < 32; i++) s += (int32_t)((qs[i / 4] >> ((i % 4) * 2)) & 3) * x[gi].q[i];
            I[gi] = s;
        }
        return;
    }
    const uint32_t bb = type == Q4O_T_IQ3_XXS ? 98 : 82;
    for (uint64_t gi = 0; gi < n / 32; gi++) {          /* sum of sign x magnitude x q, before the sub-scales */
        q4o_grp g;
        if (type == Q4O_T_IQ3_XXS) iq3xxs_group(row + (gi / 8) * bb, (int)(gi & 7), &g);
        else iq2s_group(row + (gi / 8) * bb, (int)(gi & 7), &g);
        int32_t s = 0;
        for (int i = 0; i < 32; i++) s += ((g.neg >> i) & 1u ? -1 : 1) * (int32_t)g.mag[i] * x[gi].q[i];
        I[gi] = s;
    }
}

/* The CPU path's row dots: src/q4_cpuexp.c:895-931 (IQ3_XXS), :814-852 (IQ2_S), :1113-1145 (Q2_0).
 * Eight fp32 lanes, one fused multiply-add per lane and 32-group with the exact integer
 * lane sum x (2 ls + 1), the final tree of cpx_hsum (:39-46). */
float q4o_dot8_x(uint32_t type, const uint8_t *row, const q4o_q8 *x, uint64_t n) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (type == Q4O_T_Q2_0) {
        float cs = 0.f;
        for (uint64_t b = 0; b < n / 64; b++) {
            const uint8_t *blk = row + b * 18;
            const float d = mv_f16(blk);
            for (int h = 0; h < 2; h++) {
                const q4o_q8 *xg = x + 2 * b + h;
                const float dd = d * xg->d;
                for (int lane = 0; lane < 8; lane++) {
                    const uint32_t byte = blk[2 + 8 * h + lane];        /* four 2-bit codes */
                    int32_t s = 0;
                    for (int t = 0; t < 4; t++) s += (int32_t)((byte >> (2 * t)) & 3) * xg->q[4 * lane + t];
                    acc[lane] = fmaf(dd, (float)s, acc[lane]);
                }
                /* the offset term, accumulated as a scalar beside the lanes (:1141; the compiler fuses
                 * the multiply-add at the reference's optimisation level) */
                cs = fmaf(dd, (float)xg->bs, cs);
            }
        }
        return (((acc[0] + acc[4]) + (acc[2] + acc[6])) + ((acc[1] + acc[5]) + (acc[3] + acc[7]))) - cs;
    }
    const uint32_t bb = type == Q4O_T_IQ3_XXS ? 98 : 82;
    for (uint64_t b = 0; b < n / Q4O_QK_K; b++)
        for (int ib = 0; ib < 8; ib++) {
            q4o_grp g;
            const float d16 = type == Q4O_T_IQ3_XXS ? iq3xxs_group(row + b * bb, ib, &g) : iq2s_group(row + b * bb, ib, &g);
            const float d = d16 * (type == Q4O_T_IQ3_XXS ? 0.25f : 0.125f);
            const q4o_q8 *xg = x + 8 * b + ib;
            const float dd = d * xg->d;
            for (int lane = 0; lane < 8; lane++) {
                int32_t s = 0;
                for (int t = 0; t < 4; t++) {
                    const int i = 4 * lane + t;
                    s += ((g.neg >> i) & 1u ? -1 : 1) * (int32_t)g.mag[i] * xg->q[i];
                }
                acc[lane] = fmaf(dd, (float)(s * (2 * g.ls[lane] + 1)), acc[lane]);
            }
        }
    return ((acc[0] + acc[4]) + (acc[2] + acc[6])) + ((acc[1] + acc[5]) + (acc[3] + acc[7]));
}
