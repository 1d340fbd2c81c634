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

uint64_t q4o_row_bytes(uint32_t type, uint64_t ncols) {
    if (type == Q4O_T_IQ4_NL) return (ncols / 32) * Q4O_IQ4NL_BYTES;
    if (type == Q4O_T_IQ4_XS) return (ncols / Q4O_QK_K) * Q4O_IQ4XS_BYTES;
    return (ncols / Q4O_QK_K) * Q4O_IQ3S_BYTES;
}

float q4o_dot8_t(uint32_t type, const uint8_t *row, const q4o_q8 *x, uint64_t n) {
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
