// Decode-path kernels on the engine's packed-expert layout (110-byte IQ3_S
// super-blocks, any device pointer): activation quantiser, RMSNorm, router,
// gate/up + SwiGLU rows, down rows + weighted combine.  These serve the
// fine-grained entry points (q4_hip_moe_exec and friends) and the stage tests.
//
// Reference counterparts: xq8_k (src/q4_rocm.cu:5149), wmoe_iq3_gu_q8
// (:3912-3989), wmoe_iq3_ya_q8 (:4081-4120), softmax_topk_k (:12703),
// grouped_rms_k (:11285); arithmetic contract: src/q4_cpuexp.c:605-637,855-892.
#include "q4b_tile.cuh"

#include <atomic>

#include "../../include/q4cuda.h"

extern std::atomic<uint64_t> g_q4b_launches;
bool q4b_ptr_tiled(const void *p);
bool q4b_moe_decode_fused(const uint8_t *, uint64_t, uint64_t, uint64_t, uint64_t, int32_t, const float *,
                          const float *, float, const float *, uint32_t, uint32_t, uint32_t, uint32_t,
                          float *, int32_t *, float *, float *, uint32_t *, uint32_t, const float *);
float *q4b_host_alias(const void *h);
bool q4b_wait_flag(uint32_t epoch);
uint32_t q4b_next_flag_epoch();
static bool decode_fused_on();

#define Q4B_X_SLICE 64u  // scratch slice that holds the quantised input row

namespace {

// ------------------------------------------------------------------ Q8-A
// One warp per 32 values.  Slice s reads x + s*xs, writes group s*gps + g.
__global__ void quant8_k(const float *__restrict__ x, uint64_t xs, uint32_t gps,
                         uint64_t n_groups, int8_t *__restrict__ q, float *__restrict__ d,
                         int32_t *__restrict__ bs, uint64_t q_slice, uint64_t d_slice,
                         const int32_t *__restrict__ n_dev) {
    const uint64_t g = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (g >= n_groups) return;
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t s = g / gps, gl = g - s * gps;
    if (n_dev && s >= (uint64_t)*n_dev) return;
    const float v = x[s * xs + gl * 32u + lane];
    const float a = q4b_warp_max(fabsf(v));
    const float sc = a > 0.f ? __fdiv_rn(127.f, a) : 0.f;
    int qi = __float2int_rn(__fmul_rn(v, sc));
    qi = max(-128, min(127, qi));
    int sum = qi;
#pragma unroll
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    q[s * q_slice + gl * 32u + lane] = (int8_t)qi;
    if (lane == 0) {
        d[s * d_slice + gl] = __fdiv_rn(a, 127.f);
        if (bs) bs[s * d_slice + gl] = sum;
    }
}

// ------------------------------------------------------------------ RMSNorm (+ Q8-A)
// One block of 256 per (group, token) row.  The sum of squares is kept in
// fp64 like the scalar reference (src/q4_quant.c:697-706).
__global__ void rms_q8_k(const float *__restrict__ x, const float *__restrict__ w,
                         float *__restrict__ y, uint32_t n, uint32_t hc, float eps,
                         int8_t *__restrict__ q, float *__restrict__ d, int32_t *__restrict__ bs,
                         uint64_t q_slice, uint64_t d_slice) {
    const uint32_t c = blockIdx.x, tok = blockIdx.y;
    const uint64_t row = (uint64_t)tok * hc + c;
    const float *xc = x + row * n;
    const float *wc = w ? w + (uint64_t)c * n : nullptr;
    double ss = 0.0;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) ss += (double)xc[i] * (double)xc[i];
    __shared__ double sh[8];
#pragma unroll
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31u) == 0) sh[threadIdx.x >> 5] = ss;
    __syncthreads();
    double tot = 0.0;
    for (uint32_t i = 0; i < (blockDim.x >> 5); i++) tot += sh[i];
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn((float)(tot / (double)n), eps)));
    const uint32_t lane = threadIdx.x & 31u;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        float v = __fmul_rn(xc[i], scale);
        if (wc) v = __fmul_rn(v, wc[i]);
        if (y) y[row * n + i] = v;
        if (q) {  // n % 32 == 0 and blockDim % 32 == 0: a warp holds one whole group
            const float a = q4b_warp_max(fabsf(v));
            const float sc = a > 0.f ? __fdiv_rn(127.f, a) : 0.f;
            int qi = __float2int_rn(__fmul_rn(v, sc));
            qi = max(-128, min(127, qi));
            int sum = qi;
#pragma unroll
            for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            q[row * q_slice + i] = (int8_t)qi;
            if (lane == 0) {
                d[row * d_slice + (i >> 5)] = __fdiv_rn(a, 127.f);
                bs[row * d_slice + (i >> 5)] = sum;
            }
        }
    }
}

// ------------------------------------------------------------------ hyper-connection streams
// A token carries hc residual streams of n floats.  After a block, stream c takes the block's
// output row times 2 sigmoid(inject[c] / hc); the next block's input is the RMSNorm of every
// updated stream (reference: hc_combine_k and hc_comb_rms_k, src/q4_rocm.cu:11341-11408).
// One CTA per (stream, token).  NORM: the update and the norm in one pass -- a thread squares
// the values it has just formed, in the element order rms_q8_k squares them in, so the sum,
// the scale and the normalised row are bit for bit those of the update followed by the norm
// as two launches.  hy: a second row added to the block's (exactly: b + hy).
__device__ __forceinline__ float hc_stream_factor(const float *inject, uint32_t tok, uint32_t hc, uint32_t c) {
    const float t = inject[(uint64_t)tok * hc + c] / (float)hc;
    return 2.f * (1.f / (1.f + expf(-t)));
}
template <bool NORM>
__global__ void __launch_bounds__(256) hc_streams_k(float *__restrict__ res, const float *__restrict__ block,
                                                    const float *__restrict__ hy,
                                                    const float *__restrict__ inject,
                                                    const float *__restrict__ wn, float *__restrict__ y,
                                                    uint32_t n, uint32_t hc, float eps) {
    const uint32_t c = blockIdx.x, tok = blockIdx.y;
    const uint64_t row = (uint64_t)tok * hc + c;
    float *rc = res + row * n;
    const float *bt = block + (uint64_t)tok * n;
    const float *ht = hy ? hy + (uint64_t)tok * n : nullptr;
    const float f = hc_stream_factor(inject, tok, hc, c);
    double ss = 0.0;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        const float b = ht ? __fadd_rn(bt[i], ht[i]) : bt[i];
        const float v = __fadd_rn(rc[i], __fmul_rn(b, f));
        rc[i] = v;
        ss += (double)v * (double)v;
    }
    if (!NORM) return;
    __shared__ double sh[8];
#pragma unroll
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31u) == 0) sh[threadIdx.x >> 5] = ss;
    __syncthreads();
    double tot = 0.0;
    for (uint32_t i = 0; i < (blockDim.x >> 5); i++) tot += sh[i];
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn((float)(tot / (double)n), eps)));
    const float *wc = wn ? wn + (uint64_t)c * n : nullptr;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {   // a thread re-reads what it wrote
        float v = __fmul_rn(rc[i], scale);
        if (wc) v = __fmul_rn(v, wc[i]);
        y[row * n + i] = v;
    }
}

// ------------------------------------------------------------------ fp32 GEMV (router)
// One warp per weight row; grid.y = batch.
__global__ void gemv_f32_k(const float *__restrict__ W, uint64_t nrows, uint64_t ncols,
                           const float *__restrict__ x, float *__restrict__ y, float scale) {
    const uint64_t r = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= nrows) return;
    const uint32_t lane = threadIdx.x & 31u;
    const float *wr = W + r * ncols;
    const float *xb = x + (uint64_t)blockIdx.y * ncols;
    float acc = 0.f;
    if ((ncols & 3u) == 0) {
        const float4 *w4 = reinterpret_cast<const float4 *>(wr);
        const float4 *x4 = reinterpret_cast<const float4 *>(xb);
        for (uint64_t i = lane; i < ncols / 4; i += 32) {
            const float4 a = __ldg(w4 + i), b = x4[i];
            acc += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
        }
    } else {
        for (uint64_t i = lane; i < ncols; i += 32) acc += wr[i] * xb[i];
    }
    acc = q4b_warp_sum(acc);
    if (lane == 0) y[(uint64_t)blockIdx.y * nrows + r] = scale * acc;
}

// The same GEMV for a batch of vectors with ncols == 2048: a warp keeps its weight row in
// registers (16 float4 per lane) and walks 16 vectors (grid.y = batch / 16), so W is read
// once per 16 vectors instead of once per vector.  Same products in the same order as
// gemv_f32_k, so a vector's result does not depend on the batch it comes in.
__global__ void __launch_bounds__(256) gemv_f32_x16_k(const float *__restrict__ W, uint64_t nrows,
                                                      const float *__restrict__ x, uint32_t n_batch,
                                                      float *__restrict__ y, float scale) {
    const uint64_t r = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= nrows) return;
    const uint32_t lane = threadIdx.x & 31u;
    const float4 *w4 = reinterpret_cast<const float4 *>(W + r * 2048u);
    float4 w[16];
#pragma unroll
    for (int j = 0; j < 16; j++) w[j] = __ldg(w4 + lane + 32 * j);
    const uint32_t t0 = blockIdx.y * 16u, t1 = min(n_batch, t0 + 16u);
    for (uint32_t t = t0; t < t1; t++) {
        const float4 *x4 = reinterpret_cast<const float4 *>(x + (uint64_t)t * 2048u);
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < 16; j++) {
            const float4 b = x4[lane + 32 * j];
            acc += w[j].x * b.x + w[j].y * b.y + w[j].z * b.z + w[j].w * b.w;
        }
        acc = q4b_warp_sum(acc);
        if (lane == 0) y[(uint64_t)t * nrows + r] = scale * acc;
    }
}

// fp32 product for many tokens at once (the router over a batch): y[t][e] = scale *
// sum_h x[t][h] W[e][h].  Shared-memory tiles of BM tokens x 64 weight rows x 16 columns,
// 256 threads, thread (ty, tx) owns BM/16 tokens x 4 weight rows (its tokens' values come as
// float4 from the transposed tile); h runs in ascending order inside every thread.  nrows % 64 == 0 and ncols % 16 == 0.
template <int BM>
__global__ void __launch_bounds__(256) gemm_f32_nt_k(const float *__restrict__ W, uint32_t nrows,
                                                     uint32_t ncols, const float *__restrict__ X,
                                                     uint32_t n_tok, float *__restrict__ Y, float scale) {
    constexpr int TM = BM / 16;      // tokens per thread: 4 or 8
    constexpr int NA = BM / 64;      // loader passes over the token tile
    __shared__ __align__(16) float As[16][BM + 4];
    __shared__ __align__(16) float Bs[16][64 + 4];
    const uint32_t tid = threadIdx.x, tx = tid & 15u, ty = tid >> 4;
    const uint32_t e0 = blockIdx.x * 64u, t0 = blockIdx.y * BM;
    const uint32_t lr = tid >> 2, lc = (tid & 3u) * 4u;   // loader: row of the tile, first of 4 columns
    float acc[TM][4];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
    const float *xa[NA];
    bool a_live[NA];
    float4 va[NA], vb;
#pragma unroll
    for (int p = 0; p < NA; p++) {
        a_live[p] = t0 + lr + 64u * p < n_tok;
        xa[p] = X + (uint64_t)(t0 + (a_live[p] ? lr + 64u * p : 0u)) * ncols + lc;
        va[p] = a_live[p] ? *reinterpret_cast<const float4 *>(xa[p]) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const float *wb = W + (uint64_t)(e0 + lr) * ncols + lc;
    vb = __ldg(reinterpret_cast<const float4 *>(wb));
    for (uint32_t h0 = 0; h0 < ncols; h0 += 16u) {
#pragma unroll
        for (int p = 0; p < NA; p++) {
            const uint32_t r = lr + 64u * p;
            As[lc][r] = va[p].x, As[lc + 1][r] = va[p].y, As[lc + 2][r] = va[p].z, As[lc + 3][r] = va[p].w;
        }
        Bs[lc][lr] = vb.x, Bs[lc + 1][lr] = vb.y, Bs[lc + 2][lr] = vb.z, Bs[lc + 3][lr] = vb.w;
        __syncthreads();
        if (h0 + 16u < ncols) {   // the next tile's loads fly under this tile's products
#pragma unroll
            for (int p = 0; p < NA; p++)
                if (a_live[p]) va[p] = *reinterpret_cast<const float4 *>(xa[p] + h0 + 16u);
            vb = __ldg(reinterpret_cast<const float4 *>(wb + h0 + 16u));
        }
#pragma unroll
        for (int k = 0; k < 16; k++) {
            float a[TM];
#pragma unroll
            for (int i = 0; i < TM; i += 4) {
                const float4 t = *reinterpret_cast<const float4 *>(&As[k][ty * TM + i]);
                a[i] = t.x, a[i + 1] = t.y, a[i + 2] = t.z, a[i + 3] = t.w;
            }
            const float4 b = *reinterpret_cast<const float4 *>(&Bs[k][tx * 4u]);
#pragma unroll
            for (int i = 0; i < TM; i++) {
                acc[i][0] = fmaf(a[i], b.x, acc[i][0]);
                acc[i][1] = fmaf(a[i], b.y, acc[i][1]);
                acc[i][2] = fmaf(a[i], b.z, acc[i][2]);
                acc[i][3] = fmaf(a[i], b.w, acc[i][3]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; i++) {
        const uint32_t t = t0 + ty * TM + i;
        if (t < n_tok)
            *reinterpret_cast<float4 *>(Y + (uint64_t)t * nrows + e0 + tx * 4u) =
                make_float4(scale * acc[i][0], scale * acc[i][1], scale * acc[i][2], scale * acc[i][3]);
    }
}

// ------------------------------------------------------------------ IQ3_S helpers
struct Iq3Group {
    uint32_t qs_lo, qs_hi, qh, sg, ls;
};
// Fields of sub-block ib of the super-block at blk (2-byte aligned address).
__device__ __forceinline__ Iq3Group iq3_load_group(const uint8_t *blk, uint32_t ib) {
    Iq3Group g;
    g.qs_lo = q4b_ld_u32_a2(blk + 2 + 8 * ib);
    g.qs_hi = q4b_ld_u32_a2(blk + 6 + 8 * ib);
    g.qh = blk[66 + ib];
    g.sg = q4b_ld_u32_a2(blk + 74 + 4 * ib);
    const uint32_t sb = blk[106 + (ib >> 1)];
    g.ls = 1u + 2u * ((ib & 1u) ? (sb >> 4) : (sb & 15u));
    return g;
}
__device__ __forceinline__ float iq3_block_d(const uint8_t *blk) {
    return __half2float(__ushort_as_half((unsigned short)q4b_ld_u16(blk)));
}

// The same fields addressed by block number within a matrix, for either storage
// format.  mat = first byte of the matrix, bi = super-block number (row-major),
// ib = sub-block.  TILED: the library's arena format (q4b_tile.cuh), where the
// sign word comes back bit-permuted; otherwise the engine's 110-byte records.
struct Iq3Fields {
    uint32_t qs_lo, qs_hi, qh, sg, ls;
    float d;
};
template <bool TILED>
__device__ __forceinline__ Iq3Fields iq3_fields(const uint8_t *mat, uint64_t bi, uint32_t ib) {
    Iq3Fields f;
    if (TILED) {
        const uint8_t *t = mat + (bi >> 3) * Q4B_TILE_BYTES;
        const uint32_t b = (uint32_t)(bi & 7u);
        const uint2 qs = *reinterpret_cast<const uint2 *>(t + Q4B_TILE_OFF_QS + 64u * b + 8u * ib);
        f.qs_lo = qs.x;
        f.qs_hi = qs.y;
        f.qh = t[Q4B_TILE_OFF_QH + 8u * b + ib];
        f.sg = *reinterpret_cast<const uint32_t *>(t + Q4B_TILE_OFF_SG + 32u * b + 4u * ib);
        const uint32_t sb = t[Q4B_TILE_OFF_SC + 4u * b + (ib >> 1)];
        f.ls = 1u + 2u * ((ib & 1u) ? (sb >> 4) : (sb & 15u));
        f.d = __half2float(*reinterpret_cast<const __half *>(t + 2u * b));
    } else {
        const uint8_t *blk = mat + bi * Q4B_IQ3S_BYTES;
        const Iq3Group g = iq3_load_group(blk, ib);
        f.qs_lo = g.qs_lo;
        f.qs_hi = g.qs_hi;
        f.qh = g.qh;
        f.sg = g.sg;
        f.ls = g.ls;
        f.d = iq3_block_d(blk);
    }
    return f;
}
// Sign of element e (0..31) of a group from its sign word.
template <bool TILED>
__device__ __forceinline__ bool iq3_neg(uint32_t sg, uint32_t e) {
    return TILED ? ((sg >> (8u * (e & 3u) + 7u - (e >> 2))) & 1u) : ((sg >> e) & 1u);
}
template <bool TILED>
__device__ __forceinline__ int32_t iq3_idot(const Iq3Fields &f, const uint32_t *tab, const int *q,
                                            int32_t qsum) {
    return TILED ? q4b_tile_group_idot<1>(f.qs_lo, f.qs_hi, f.qh, f.sg, tab, q, qsum)
                 : q4b_group_idot(f.qs_lo, f.qs_hi, f.qh, f.sg, tab, q, qsum);
}

// fp32 dequantisation, one thread per 32-weight sub-block.
template <bool TILED>
__global__ void iq3s_dequant_k(const uint8_t *__restrict__ w, uint64_t n_groups,
                               float *__restrict__ out) {
    __shared__ uint32_t tab[512];
    q4b_fill_code_table(tab);
    __syncthreads();
    const uint64_t g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= n_groups) return;
    const Iq3Fields f = iq3_fields<TILED>(w, g >> 3, (uint32_t)(g & 7u));
    // src/q4_quant.c:397-409: db = d * (1 + 2 s); value = db * magnitude * (+-1)
    const float db = __fmul_rn(f.d, (float)f.ls);
    float *o = out + g * 32u;
    for (int k = 0; k < 8; k++) {
        const uint32_t wq = k < 4 ? f.qs_lo : f.qs_hi;
        const uint32_t idx = ((wq >> (8 * (k & 3))) & 0xffu) | (((f.qh >> k) & 1u) << 8);
        const uint32_t c = tab[idx];
        for (int j = 0; j < 4; j++) {
            const float mag = (float)(2u * ((c >> (8 * j)) & 0xffu) + 1u);
            o[4 * k + j] = __fmul_rn(__fmul_rn(db, mag), iq3_neg<TILED>(f.sg, 4 * k + j) ? -1.f : 1.f);
        }
    }
}

// Per-group integer dots of nrows rows against one quantised vector.
template <bool TILED>
__global__ void iq3s_idot_k(const uint8_t *__restrict__ w, uint64_t nrows, uint32_t ng,
                            const int8_t *__restrict__ q, int32_t *__restrict__ I) {
    __shared__ uint32_t tab[512];
    q4b_fill_code_table(tab);
    __syncthreads();
    const uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= nrows * ng) return;
    const uint64_t r = t / ng;
    const uint32_t g = (uint32_t)(t - r * ng);
    const Iq3Fields f = iq3_fields<TILED>(w, r * (ng >> 3) + (g >> 3), g & 7u);
    const int *qg = reinterpret_cast<const int *>(q) + g * 8u;
    int qv[8];
    int qsum = 0;
    for (int k = 0; k < 8; k++) {
        qv[k] = qg[k];
        qsum = __dp4a(qv[k], 0x01010101, qsum);
    }
    I[t] = iq3_idot<TILED>(f, tab, qv, qsum);
}

// ------------------------------------------------------------------ router softmax + top-k
// One warp per token.  p = softmax(logits); k picks by descending p, equal
// values keep the lower index; weights renormalised over the picks in rank
// order (src/q4_quant.c:715-755).  Optionally appends the shared expert's slot
// with weight 1 and writes the entry count.
__device__ __forceinline__ void softmax_topk_warp(const float *__restrict__ l, uint32_t n, uint32_t k,
                                                  int32_t *__restrict__ ids, float *__restrict__ wts,
                                                  int32_t shared_slot, int32_t *__restrict__ n_out,
                                                  float *p, float *wsel, uint32_t lane) {
    float m = -INFINITY;
    for (uint32_t i = lane; i < n; i += 32) m = fmaxf(m, __ldcg(l + i));
    m = q4b_warp_max(m);
    float s = 0.f;
    for (uint32_t i = lane; i < n; i += 32) {
        const float e = expf(__ldcg(l + i) - m);
        p[i] = e;
        s += e;
    }
    s = q4b_warp_sum(s);
    const float inv = s > 0.f ? __fdiv_rn(1.0f, s) : 0.f;
    for (uint32_t i = lane; i < n; i += 32) p[i] = __fmul_rn(p[i], inv);
    __syncwarp();
    // key: value bits above, inverted index below -> max key = largest value,
    // lowest index among equals.  p >= 0 so the bit pattern orders like the value.
    auto scan = [&]() {
        unsigned long long best = 0ull;
        for (uint32_t i = lane; i < n; i += 32) {
            const float v = p[i];
            if (v < 0.f) continue;  // taken
            const unsigned long long key =
                ((unsigned long long)__float_as_uint(v) << 32) | (0xffffffffu - i);
            best = key > best ? key : best;
        }
        return best;
    };
    unsigned long long mine = scan();
    if (k > n) k = n;
    for (uint32_t t = 0; t < k; t++) {
        unsigned long long best = mine;
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
            best = other > best ? other : best;
        }
        const uint32_t idx = 0xffffffffu - (uint32_t)(best & 0xffffffffu);
        if (lane == 0) {
            ids[t] = (int32_t)idx;
            wsel[t] = __uint_as_float((uint32_t)(best >> 32));
        }
        if ((idx & 31u) == lane) {
            p[idx] = -1.f;
            mine = scan();
        }
    }
    __syncwarp();
    if (lane == 0) {
        float sum = 0.f;
        for (uint32_t t = 0; t < k; t++) sum = __fadd_rn(sum, wsel[t]);
        const float wi = sum > 0.f ? __fdiv_rn(1.0f, sum) : 1.f;
        for (uint32_t t = 0; t < k; t++) wts[t] = sum > 0.f ? __fmul_rn(wsel[t], wi) : wsel[t];
        uint32_t cnt = k;
        if (shared_slot >= 0) {
            ids[k] = shared_slot;
            wts[k] = 1.0f;
            cnt++;
        }
        if (n_out) *n_out = (int32_t)cnt;
    }
}
__global__ void softmax_topk_k(const float *__restrict__ logits, uint32_t n, uint32_t k,
                               int32_t *__restrict__ ids, float *__restrict__ wts,
                               uint32_t out_stride, int32_t shared_slot,
                               int32_t *__restrict__ n_out) {
    __shared__ float p[1024];
    __shared__ float wsel[64];
    softmax_topk_warp(logits + (uint64_t)blockIdx.x * n, n, k, ids + (uint64_t)blockIdx.x * out_stride,
                      wts + (uint64_t)blockIdx.x * out_stride, shared_slot, n_out ? n_out + blockIdx.x : nullptr, p,
                      wsel, threadIdx.x);
}

// RMSNorm, router product and softmax / top-k of a batch of tokens in ONE launch (n_embd == 2048): what
// rms_q8_k (norm only), gemv_f32_x16_k and softmax_topk_k do as three, with the same products and sums
// in the same order (the sum of squares is formed in double in another order, which does not change
// its float value).  grid (router rows / 8, tokens / 8): a CTA normalises its group's eight rows (a
// warp per row, all loads in flight at once) into shared memory, then a warp takes one router row
// through the eight tokens; the CTA that finishes a group last (a counter per group, no waiting) runs
// the group's top-k, one warp per token.
__global__ void __launch_bounds__(256) route_small_k(const float *__restrict__ x, const float *__restrict__ norm_w,
                                                     float eps, const float *__restrict__ W, uint32_t n_expert,
                                                     uint32_t n_tok, uint32_t topk, float *__restrict__ xn_out,
                                                     float *__restrict__ logits, int32_t *__restrict__ ids,
                                                     float *__restrict__ wts, unsigned int *__restrict__ counters) {
    extern __shared__ __align__(16) float rs_rows[];   // [8][2048]; the last CTA reuses it for the probabilities
    __shared__ float wsel[8][64];
    __shared__ uint32_t is_last;
    constexpr uint32_t n = 2048;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t t0 = blockIdx.y * 8u, nt = min(8u, n_tok - t0);
    if (warp < nt) {
        const float4 *x4 = reinterpret_cast<const float4 *>(x + (uint64_t)(t0 + warp) * n);
        float4 v[16];
#pragma unroll
        for (int j = 0; j < 16; j++) v[j] = x4[lane + 32 * j];
        double ss = 0.0;
#pragma unroll
        for (int j = 0; j < 16; j++)
            ss += (double)v[j].x * (double)v[j].x + (double)v[j].y * (double)v[j].y +
                  (double)v[j].z * (double)v[j].z + (double)v[j].w * (double)v[j].w;
#pragma unroll
        for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn((float)(ss / (double)n), eps)));
        float4 *r4 = reinterpret_cast<float4 *>(rs_rows + warp * n);
        float4 *o4 = blockIdx.x == 0 ? reinterpret_cast<float4 *>(xn_out + (uint64_t)(t0 + warp) * n) : nullptr;
#pragma unroll
        for (int j = 0; j < 16; j++) {
            float4 u;
            u.x = __fmul_rn(v[j].x, scale), u.y = __fmul_rn(v[j].y, scale);
            u.z = __fmul_rn(v[j].z, scale), u.w = __fmul_rn(v[j].w, scale);
            if (norm_w) {
                const float4 g = __ldg(reinterpret_cast<const float4 *>(norm_w) + lane + 32 * j);
                u.x = __fmul_rn(u.x, g.x), u.y = __fmul_rn(u.y, g.y);
                u.z = __fmul_rn(u.z, g.z), u.w = __fmul_rn(u.w, g.w);
            }
            r4[lane + 32 * j] = u;
            if (o4) o4[lane + 32 * j] = u;
        }
    }
    __syncthreads();
    const uint32_t r = blockIdx.x * 8u + warp;
    if (r < n_expert) {
        const float4 *w4 = reinterpret_cast<const float4 *>(W + (uint64_t)r * n);
        float4 w[16];
#pragma unroll
        for (int j = 0; j < 16; j++) w[j] = __ldg(w4 + lane + 32 * j);
        for (uint32_t t = 0; t < nt; t++) {
            const float4 *x4 = reinterpret_cast<const float4 *>(rs_rows + t * n);
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const float4 b = x4[lane + 32 * j];
                acc += w[j].x * b.x + w[j].y * b.y + w[j].z * b.z + w[j].w * b.w;
            }
            acc = q4b_warp_sum(acc);
            if (lane == 0) logits[(uint64_t)(t0 + t) * n_expert + r] = 1.0f * acc;
        }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0)   // wraps to 0 by itself
        is_last = atomicInc(counters + blockIdx.y, gridDim.x - 1u) == gridDim.x - 1u ? 1u : 0u;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (warp < nt)
        softmax_topk_warp(logits + (uint64_t)(t0 + warp) * n_expert, n_expert, topk, ids + (uint64_t)(t0 + warp) * topk,
                          wts + (uint64_t)(t0 + warp) * topk, -1, nullptr, rs_rows + warp * 1024u, wsel[warp], lane);
}

// ------------------------------------------------------------------ gate/up + SwiGLU
// grid (n_ff/8, experts), 8 warps per block, one warp per hidden unit f:
// h[e][f] = silu(gate_f . xq) * (up_f . xq).
template <bool TILED>
__global__ void moe_gu_k(const uint8_t *__restrict__ bg, const uint8_t *__restrict__ bu,
                         uint64_t stride, const int32_t *__restrict__ slots,
                         const int32_t *__restrict__ n_dev, const int8_t *__restrict__ xq,
                         const float *__restrict__ xd, const int32_t *__restrict__ xbs,
                         uint32_t in_dim, uint32_t n_ff, float *__restrict__ h) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint32_t *tab = reinterpret_cast<uint32_t *>(smem);
    int *sq = reinterpret_cast<int *>(smem + 2048);
    const uint32_t ng = in_dim >> 5;
    float *sd = reinterpret_cast<float *>(smem + 2048 + in_dim);
    int *sb = reinterpret_cast<int *>(smem + 2048 + in_dim + 4 * ng);
    const uint32_t e = blockIdx.y;
    if (n_dev && e >= (uint32_t)*n_dev) return;
    q4b_fill_code_table(tab);
    for (uint32_t i = threadIdx.x; i < in_dim / 4; i += blockDim.x)
        sq[i] = reinterpret_cast<const int *>(xq)[i];
    for (uint32_t i = threadIdx.x; i < ng; i += blockDim.x) {
        sd[i] = xd[i];
        sb[i] = xbs[i];
    }
    __syncthreads();
    const uint32_t f = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (f >= n_ff) return;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t nbr = in_dim >> 8;  // super-blocks per row
    const uint8_t *wg = bg + (uint64_t)slots[e] * stride, *wu = bu + (uint64_t)slots[e] * stride;
    float ag = 0.f, au = 0.f;
    for (uint32_t g = lane; g < ng; g += 32) {
        const uint64_t bi = (uint64_t)f * nbr + (g >> 3);
        const int *qv = sq + g * 8u;
        const float dx = sd[g];
        const int qsum = sb[g];
        {
            const Iq3Fields fg = iq3_fields<TILED>(wg, bi, g & 7u);
            const int I = iq3_idot<TILED>(fg, tab, qv, qsum);
            ag = fmaf(__fmul_rn(fg.d, dx), (float)(I * (int)fg.ls), ag);
        }
        {
            const Iq3Fields fg = iq3_fields<TILED>(wu, bi, g & 7u);
            const int I = iq3_idot<TILED>(fg, tab, qv, qsum);
            au = fmaf(__fmul_rn(fg.d, dx), (float)(I * (int)fg.ls), au);
        }
    }
    ag = q4b_warp_sum(ag);
    au = q4b_warp_sum(au);
    if (lane == 0) h[(uint64_t)e * n_ff + f] = q4b_swiglu(ag, au);
}

// ------------------------------------------------------------------ down + weighted combine
// grid (n_embd/8), one warp per output row r:
// y[r] += sum_e wts[e] * (down_e[r] . hq_e), experts visited in list order by a
// fixed lane assignment, so the result is reproducible run to run.
template <bool TILED>
__global__ void moe_ya_k(const uint8_t *__restrict__ bd, uint64_t stride,
                         const int32_t *__restrict__ slots, const float *__restrict__ wts,
                         uint32_t n_host, const int32_t *__restrict__ n_dev,
                         const int8_t *__restrict__ hq, const float *__restrict__ hd,
                         const int32_t *__restrict__ hbs, uint64_t q_slice, uint64_t d_slice,
                         uint32_t n_ff, uint32_t n_embd, float *__restrict__ y) {
    __shared__ uint32_t tab[512];
    q4b_fill_code_table(tab);
    __syncthreads();
    const uint32_t r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= n_embd) return;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t n = n_dev ? (uint32_t)*n_dev : n_host;
    const uint32_t ng = n_ff >> 5;
    const uint32_t nbr = n_ff >> 8;
    float acc = 0.f;
    for (uint32_t it = lane; it < n * ng; it += 32) {
        const uint32_t e = it / ng, g = it - e * ng;
        const Iq3Fields fg = iq3_fields<TILED>(bd + (uint64_t)slots[e] * stride,
                                              (uint64_t)r * nbr + (g >> 3), g & 7u);
        const int *qg = reinterpret_cast<const int *>(hq + (uint64_t)e * q_slice) + g * 8u;
        int qv[8];
#pragma unroll
        for (int k = 0; k < 8; k++) qv[k] = qg[k];
        const int I = iq3_idot<TILED>(fg, tab, qv, hbs[(uint64_t)e * d_slice + g]);
        const float dd = __fmul_rn(fg.d, hd[(uint64_t)e * d_slice + g]);
        acc = fmaf(__fmul_rn(wts[e], dd), (float)(I * (int)fg.ls), acc);
    }
    acc = q4b_warp_sum(acc);
    if (lane == 0) y[r] += acc;
}

// ------------------------------------------------------------------ IQ4_NL and IQ4_XS
// Both index the same 16-value table with 4-bit codes, 16 code bytes per 32 weights (low nibbles
// = weights 0..15, high nibbles = 16..31).  IQ4_NL: 18-byte blocks, fp16 d + codes
// (src/q4_quant.c:270-290).  IQ4_XS: 136-byte super-blocks of 256, fp16 d, u16 scales_h,
// scales_l[4], qs[128]; group scale = d * (ls - 32), ls six bits (src/q4_quant.c:455-480).
// The kernels keep a 256-entry table in shared memory: code byte -> (low value, high value).
__device__ __forceinline__ void iq4_fill_pair_table(uint16_t *pair) {
    const int8_t kv[16] = Q4B_IQ4NL_VALUES;
    for (uint32_t b = threadIdx.x; b < 256u; b += blockDim.x)
        pair[b] = (uint16_t)((uint8_t)kv[b & 15u] | ((uint16_t)(uint8_t)kv[b >> 4] << 8));
}
// Integer dot of 16 code bytes (2-byte aligned) with their 32 activation bytes: exact int32.
__device__ __forceinline__ int32_t iq4_codes_idot(const uint8_t *codes, const uint16_t *pair, const int *q) {
    int32_t acc = 0;
#pragma unroll
    for (int w = 0; w < 4; w++) {       // four code bytes -> weights 4w..4w+3 and 16+4w..16+4w+3
        const uint32_t c01 = q4b_ld_u16(codes + 4 * w), c23 = q4b_ld_u16(codes + 4 * w + 2);
        const uint32_t p0 = pair[c01 & 0xffu], p1 = pair[c01 >> 8], p2 = pair[c23 & 0xffu], p3 = pair[c23 >> 8];
        const uint32_t lo = (p0 & 0xffu) | ((p1 & 0xffu) << 8) | ((p2 & 0xffu) << 16) | ((p3 & 0xffu) << 24);
        const uint32_t hi = (p0 >> 8) | ((p1 >> 8) << 8) | ((p2 >> 8) << 16) | ((p3 >> 8) << 24);
        acc = __dp4a((int)lo, q[w], acc);
        acc = __dp4a((int)hi, q[4 + w], acc);
    }
    return acc;
}
// Group g (32 weights) of a row of type T (20 or 23): where its codes are, its integer scale
// factor and the fp16 block scale.
template <uint32_t T>
__device__ __forceinline__ const uint8_t *iq4_group(const uint8_t *row, uint32_t g, int *lsf, float *d) {
    if (T == Q4_T_IQ4_NL) {
        const uint8_t *blk = row + (uint64_t)g * 18u;
        *lsf = 1;
        *d = __half2float(__ushort_as_half((unsigned short)q4b_ld_u16(blk)));
        return blk + 2;
    }
    const uint8_t *blk = row + (uint64_t)(g >> 3) * 136u;
    const uint32_t ib = g & 7u;
    const uint32_t sh = q4b_ld_u16(blk + 2);
    *lsf = (int)(((blk[4 + (ib >> 1)] >> (4u * (ib & 1u))) & 0xfu) | (((sh >> (2u * ib)) & 3u) << 4)) - 32;
    *d = __half2float(__ushort_as_half((unsigned short)q4b_ld_u16(blk)));
    return blk + 8 + 16u * ib;
}
__host__ __device__ inline uint64_t iq4_row_bytes(uint32_t type, uint64_t ncols) {
    return type == Q4_T_IQ4_NL ? (ncols / 32u) * 18u : (ncols / 256u) * 136u;
}

template <uint32_t T>
__global__ void iq4_dequant_k(const uint8_t *__restrict__ w, uint64_t n_groups, uint32_t gpr,
                              float *__restrict__ out) {
    const int8_t kv[16] = Q4B_IQ4NL_VALUES;
    const uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_groups) return;
    const uint64_t r = t / gpr;
    int lsf;
    float d;
    const uint8_t *codes = iq4_group<T>(w + r * iq4_row_bytes(T, 32ull * gpr), (uint32_t)(t - r * gpr), &lsf, &d);
    const float dl = T == Q4_T_IQ4_NL ? d : __fmul_rn(d, (float)lsf);
    for (int j = 0; j < 16; j++) {
        out[t * 32u + j] = __fmul_rn(dl, (float)kv[codes[j] & 15u]);
        out[t * 32u + j + 16] = __fmul_rn(dl, (float)kv[codes[j] >> 4]);
    }
}

// I[r][g] for nrows rows of gpr groups against one quantised vector.
template <uint32_t T>
__global__ void iq4_idot_k(const uint8_t *__restrict__ w, uint64_t nrows, uint32_t gpr,
                           const int8_t *__restrict__ q, int32_t *__restrict__ I) {
    __shared__ uint16_t pair[256];
    iq4_fill_pair_table(pair);
    __syncthreads();
    const uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= nrows * gpr) return;
    const uint64_t r = t / gpr;
    const uint32_t g = (uint32_t)(t - r * gpr);
    int qv[8];
    for (int k = 0; k < 8; k++) qv[k] = reinterpret_cast<const int *>(q)[g * 8u + k];
    int lsf;
    float d;
    const uint8_t *codes = iq4_group<T>(w + r * iq4_row_bytes(T, 32ull * gpr), g, &lsf, &d);
    I[t] = iq4_codes_idot(codes, pair, qv);
}

// Gate/up + SwiGLU with rows of type T: one warp per (expert, hidden unit); the counterpart of
// moe_gu_k.  h[e][f] = silu(gate_f . xq) * (up_f . xq).
template <uint32_t T>
__global__ void moe_gu4_k(const uint8_t *__restrict__ bg, const uint8_t *__restrict__ bu, uint64_t stride,
                          const int32_t *__restrict__ slots, const int32_t *__restrict__ n_dev,
                          const int8_t *__restrict__ xq, const float *__restrict__ xd, uint32_t in_dim,
                          uint32_t n_ff, float *__restrict__ h) {
    __shared__ uint16_t pair[256];
    iq4_fill_pair_table(pair);
    __syncthreads();
    const uint32_t e = blockIdx.y;
    if (n_dev && e >= (uint32_t)*n_dev) return;
    const uint32_t f = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (f >= n_ff) return;
    const uint32_t lane = threadIdx.x & 31u, ng = in_dim >> 5;
    const uint64_t rb = iq4_row_bytes(T, in_dim);
    const uint8_t *rg = bg + (uint64_t)slots[e] * stride + (uint64_t)f * rb;
    const uint8_t *ru = bu + (uint64_t)slots[e] * stride + (uint64_t)f * rb;
    float ag = 0.f, au = 0.f;
    for (uint32_t g = lane; g < ng; g += 32) {
        int qv[8];
#pragma unroll
        for (int k = 0; k < 8; k++) qv[k] = reinterpret_cast<const int *>(xq)[g * 8u + k];
        const float dx = xd[g];
        int lsf;
        float d;
        const uint8_t *cg = iq4_group<T>(rg, g, &lsf, &d);
        ag = fmaf(__fmul_rn(d, dx), (float)(iq4_codes_idot(cg, pair, qv) * lsf), ag);
        const uint8_t *cu = iq4_group<T>(ru, g, &lsf, &d);
        au = fmaf(__fmul_rn(d, dx), (float)(iq4_codes_idot(cu, pair, qv) * lsf), au);
    }
    ag = q4b_warp_sum(ag);
    au = q4b_warp_sum(au);
    if (lane == 0) h[(uint64_t)e * n_ff + f] = q4b_swiglu(ag, au);
}

// Down projection with rows of type T: the counterpart of moe_ya_k (same reduction shape).
template <uint32_t T>
__global__ void moe_ya4_k(const uint8_t *__restrict__ bd, uint64_t stride, const int32_t *__restrict__ slots,
                          const float *__restrict__ wts, uint32_t n_host, const int32_t *__restrict__ n_dev,
                          const int8_t *__restrict__ hq, const float *__restrict__ hd, uint64_t q_slice,
                          uint64_t d_slice, uint32_t n_ff, uint32_t n_embd, float *__restrict__ y) {
    __shared__ uint16_t pair[256];
    iq4_fill_pair_table(pair);
    __syncthreads();
    const uint32_t r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= n_embd) return;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t n = n_dev ? (uint32_t)*n_dev : n_host;
    const uint32_t ng = n_ff >> 5;
    const uint64_t rb = iq4_row_bytes(T, n_ff);
    float acc = 0.f;
    for (uint32_t it = lane; it < n * ng; it += 32) {
        const uint32_t e = it / ng, g = it - e * ng;
        const int *qg = reinterpret_cast<const int *>(hq + (uint64_t)e * q_slice) + g * 8u;
        int qv[8];
#pragma unroll
        for (int k = 0; k < 8; k++) qv[k] = qg[k];
        int lsf;
        float d;
        const uint8_t *codes = iq4_group<T>(bd + (uint64_t)slots[e] * stride + (uint64_t)r * rb, g, &lsf, &d);
        const int I = iq4_codes_idot(codes, pair, qv);
        const float dd = __fmul_rn(d, hd[(uint64_t)e * d_slice + g]);
        acc = fmaf(__fmul_rn(wts[e], dd), (float)(I * lsf), acc);
    }
    acc = q4b_warp_sum(acc);
    if (lane == 0) y[r] += acc;
}

// IQ3_S row r times an fp32 vector, one warp (every lane gets its partial sum; the caller
// reduces).  Lane l takes groups l, l + 32, ...; tab = the 512 byte-expanded codes.
template <bool TILED>
__device__ __forceinline__ float iq3s_row_dot_f32(const uint8_t *__restrict__ w, uint64_t r, uint32_t ncols,
                                                  const float *__restrict__ xb, const uint32_t *tab,
                                                  uint32_t lane) {
    const uint32_t ng = ncols >> 5;
    float acc = 0.f;
    for (uint32_t g = lane; g < ng; g += 32) {
        const Iq3Fields f = iq3_fields<TILED>(w, r * (uint64_t)(ncols >> 8) + (g >> 3), g & 7u);
        const float db = f.d * (float)f.ls;
        float sub = 0.f;
        for (int k = 0; k < 8; k++) {
            const uint32_t wq = k < 4 ? f.qs_lo : f.qs_hi;
            const uint32_t idx = ((wq >> (8 * (k & 3))) & 0xffu) | (((f.qh >> k) & 1u) << 8);
            const uint32_t c = tab[idx];
            for (int j = 0; j < 4; j++) {
                const float mag = (float)(2u * ((c >> (8 * j)) & 0xffu) + 1u);
                const float xv = xb[g * 32u + 4 * k + j];
                sub += iq3_neg<TILED>(f.sg, 4 * k + j) ? -mag * xv : mag * xv;
            }
        }
        acc += db * sub;
    }
    return acc;
}

// IQ3_S rows times fp32 activations (shared-expert style GEMV), warp per row.
template <bool TILED>
__global__ void gemv_iq3s_f32_k(const uint8_t *__restrict__ w, uint64_t nrows, uint32_t ncols,
                                const float *__restrict__ x, float *__restrict__ y, float scale) {
    __shared__ uint32_t tab[512];
    q4b_fill_code_table(tab);
    __syncthreads();
    const uint64_t r = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= nrows) return;
    const uint32_t lane = threadIdx.x & 31u;
    float acc = iq3s_row_dot_f32<TILED>(w, r, ncols, x + (uint64_t)blockIdx.y * ncols, tab, lane);
    acc = q4b_warp_sum(acc);
    if (lane == 0) y[(uint64_t)blockIdx.y * nrows + r] = scale * acc;
}

#include "q4b_small_formats.cuh"

// ------------------------------------------------------------------ host side
// gate and up of one type out of IQ3_S, IQ4_NL, IQ4_XS, IQ3_XXS, IQ2_S; down out of IQ3_S, IQ4_NL,
// IQ4_XS, Q2_0 (of the formats the engine's call sites accept, src/q4_rocm.cu:4926-4944, the ones its
// deployed models use for these projections)
bool gu_type_ok(uint32_t t) {
    return t == Q4_T_IQ3_S || t == Q4_T_IQ4_NL || t == Q4_T_IQ4_XS || t == Q4_T_IQ3_XXS || t == Q4_T_IQ2_S;
}
bool down_type_ok(uint32_t t) { return t == Q4_T_IQ3_S || t == Q4_T_IQ4_NL || t == Q4_T_IQ4_XS || t == Q4_T_Q2_0; }
bool shape_ok(uint32_t gt, uint32_t ut, uint32_t dt, uint32_t in_dim, uint32_t n_ff) {
    return gt == ut && gu_type_ok(gt) && down_type_ok(dt) && in_dim && n_ff && (in_dim % Q4B_QK) == 0 &&
           (n_ff % Q4B_QK) == 0 && in_dim <= Q4B_XQ_MAXLEN && n_ff <= Q4B_XQ_MAXLEN;
}

// A pack with a part that is not IQ3_S cannot live in a tiled arena (the tiling regroups IQ3_S bytes).
bool place_ok(uint32_t gt, uint32_t dt, const void *base) {
    return (gt == Q4_T_IQ3_S && dt == Q4_T_IQ3_S) || !q4b_ptr_tiled(base);
}
// In a tiled arena a matrix must start on a tile: the kernels address whole 880-byte tiles.
bool tile_offsets_ok(const void *base, uint64_t stride, uint64_t og, uint64_t ou, uint64_t od) {
    if (!q4b_ptr_tiled(base)) return true;
    return (stride % Q4B_TILE_BYTES) == 0 && (og % Q4B_TILE_BYTES) == 0 && (ou % Q4B_TILE_BYTES) == 0 &&
           (od % Q4B_TILE_BYTES) == 0;
}

bool launch_quant8(const float *x, uint64_t xs, uint32_t slen, uint32_t ns, int8_t *q, float *d,
                   int32_t *bs, uint64_t q_slice, uint64_t d_slice, const int32_t *n_dev) {
    const uint32_t gps = slen >> 5;
    const uint64_t ngr = (uint64_t)gps * ns;
    quant8_k<<<(unsigned)((ngr + 7) / 8), 256, 0, g_q4b.stream>>>(x, xs, gps, ngr, q, d, bs,
                                                                 q_slice, d_slice, n_dev);
    g_q4b_launches++;
    return q4b_launch_ok("quant8");
}

// The common tail of every exec variant: d_x is already quantised into the
// scratch slice Q4B_X_SLICE.
bool moe_exec_tail(const uint8_t *base, uint64_t stride, const int32_t *d_slots,
                   const float *d_wts, uint32_t n_host, const int32_t *d_n, uint64_t og,
                   uint64_t ou, uint64_t od, float *d_h, float *d_y, uint32_t n_ff,
                   uint32_t in_dim, uint32_t n_embd, uint32_t dt = Q4_T_IQ3_S,
                   uint32_t gt = Q4_T_IQ3_S) {
    Q4bState &s = g_q4b;
    const uint32_t ne = d_n ? 64u : n_host;
    const int8_t *xq = s.xq + (size_t)Q4B_X_SLICE * Q4B_XQ_MAXLEN;
    const float *xd = s.xd + (size_t)Q4B_X_SLICE * (Q4B_XQ_MAXLEN / 32);
    const int32_t *xbs = s.xbs + (size_t)Q4B_X_SLICE * (Q4B_XQ_MAXLEN / 32);
    const size_t sm = 2048 + in_dim + 8 * (in_dim >> 5);
    const bool tiled = q4b_ptr_tiled(base);
    if (gt == Q4_T_IQ3_XXS)
        moe_gux_k<Q4_T_IQ3_XXS><<<dim3((n_ff + 7) / 8, ne), 256, 0, s.stream>>>(
            base + og, base + ou, stride, d_slots, d_n, xq, xd, in_dim, n_ff, s.grid3xxs_d, s.grid2s_d, d_h);
    else if (gt == Q4_T_IQ2_S)
        moe_gux_k<Q4_T_IQ2_S><<<dim3((n_ff + 7) / 8, ne), 256, 0, s.stream>>>(
            base + og, base + ou, stride, d_slots, d_n, xq, xd, in_dim, n_ff, s.grid3xxs_d, s.grid2s_d, d_h);
    else if (gt == Q4_T_IQ4_NL)
        moe_gu4_k<Q4_T_IQ4_NL><<<dim3((n_ff + 7) / 8, ne), 256, 0, s.stream>>>(
            base + og, base + ou, stride, d_slots, d_n, xq, xd, in_dim, n_ff, d_h);
    else if (gt == Q4_T_IQ4_XS)
        moe_gu4_k<Q4_T_IQ4_XS><<<dim3((n_ff + 7) / 8, ne), 256, 0, s.stream>>>(
            base + og, base + ou, stride, d_slots, d_n, xq, xd, in_dim, n_ff, d_h);
    else if (tiled)
        moe_gu_k<true><<<dim3((n_ff + 7) / 8, ne), 256, sm, s.stream>>>(
            base + og, base + ou, stride, d_slots, d_n, xq, xd, xbs, in_dim, n_ff, d_h);
    else
        moe_gu_k<false><<<dim3((n_ff + 7) / 8, ne), 256, sm, s.stream>>>(
            base + og, base + ou, stride, d_slots, d_n, xq, xd, xbs, in_dim, n_ff, d_h);
    g_q4b_launches++;
    if (!q4b_launch_ok("moe_gu")) return false;
    if (!launch_quant8(d_h, n_ff, n_ff, ne, s.xq, s.xd, s.xbs, Q4B_XQ_MAXLEN, Q4B_XQ_MAXLEN / 32,
                       d_n))
        return false;
    if (dt == Q4_T_Q2_0)
        moe_ya20_k<<<(n_embd + 7) / 8, 256, 0, s.stream>>>(base + od, stride, d_slots, d_wts, n_host, d_n, s.xq, s.xd,
                                                          s.xbs, Q4B_XQ_MAXLEN, Q4B_XQ_MAXLEN / 32, n_ff, n_embd, d_y);
    else if (dt == Q4_T_IQ4_NL)
        moe_ya4_k<Q4_T_IQ4_NL><<<(n_embd + 7) / 8, 256, 0, s.stream>>>(
            base + od, stride, d_slots, d_wts, n_host, d_n, s.xq, s.xd, Q4B_XQ_MAXLEN, Q4B_XQ_MAXLEN / 32, n_ff,
            n_embd, d_y);
    else if (dt == Q4_T_IQ4_XS)
        moe_ya4_k<Q4_T_IQ4_XS><<<(n_embd + 7) / 8, 256, 0, s.stream>>>(
            base + od, stride, d_slots, d_wts, n_host, d_n, s.xq, s.xd, Q4B_XQ_MAXLEN, Q4B_XQ_MAXLEN / 32, n_ff,
            n_embd, d_y);
    else if (tiled)
        moe_ya_k<true><<<(n_embd + 7) / 8, 256, 0, s.stream>>>(
            base + od, stride, d_slots, d_wts, n_host, d_n, s.xq, s.xd, s.xbs, Q4B_XQ_MAXLEN,
            Q4B_XQ_MAXLEN / 32, n_ff, n_embd, d_y);
    else
        moe_ya_k<false><<<(n_embd + 7) / 8, 256, 0, s.stream>>>(
            base + od, stride, d_slots, d_wts, n_host, d_n, s.xq, s.xd, s.xbs, Q4B_XQ_MAXLEN,
            Q4B_XQ_MAXLEN / 32, n_ff, n_embd, d_y);
    g_q4b_launches++;
    return q4b_launch_ok("moe_ya");
}

bool quant_x(const float *d_x, uint32_t in_dim) {
    Q4bState &s = g_q4b;
    return launch_quant8(d_x, 0, in_dim, 1, s.xq + (size_t)Q4B_X_SLICE * Q4B_XQ_MAXLEN,
                         s.xd + (size_t)Q4B_X_SLICE * (Q4B_XQ_MAXLEN / 32),
                         s.xbs + (size_t)Q4B_X_SLICE * (Q4B_XQ_MAXLEN / 32), 0, 0, nullptr);
}

}  // namespace

extern "C" bool q4_hip_moe_tok_ok(uint32_t gt, uint32_t ut, uint32_t dt, uint32_t in_dim,
                                  uint32_t n_ff) {
    return g_q4b.ok && shape_ok(gt, ut, dt, in_dim, n_ff);
}

extern "C" bool q4_hip_moe_stage(const int32_t *slots, const float *wts, uint32_t n) {
    if (!g_q4b.ok || !slots || !wts || n == 0 || n > 64) return false;
    memcpy(g_q4b.es_h, slots, n * sizeof(int32_t));
    memcpy(g_q4b.ew_h, wts, n * sizeof(float));
    *g_q4b.en_h = (int32_t)n;
    return true;
}

extern "C" bool q4_hip_moe_exec_staged(const uint8_t *base, uint64_t stride, uint32_t gt,
                                       uint64_t og, uint32_t ut, uint64_t ou, uint32_t dt,
                                       uint64_t od, const float *d_x, float *d_h, float *d_h2,
                                       float *d_down, float *d_y, uint32_t n_ff, uint32_t in_dim,
                                       uint32_t n_embd) {
    (void)d_h2;
    (void)d_down;
    if (!g_q4b.ok || !base || !d_x || !d_h || !d_y || !n_embd) return false;
    if (!shape_ok(gt, ut, dt, in_dim, n_ff) || !place_ok(gt, dt, base) || !tile_offsets_ok(base, stride, og, ou, od))
        return false;
    if (!quant_x(d_x, in_dim)) return false;
    return moe_exec_tail(base, stride, g_q4b.es_d, g_q4b.ew_d, 0, g_q4b.en_d, og, ou, od, d_h, d_y,
                         n_ff, in_dim, n_embd, dt, gt);
}

extern "C" bool q4_hip_moe_exec(const uint8_t *base, uint64_t stride, const int32_t *slots,
                                const float *wts, uint32_t n, uint32_t gt, uint64_t og,
                                uint32_t ut, uint64_t ou, uint32_t dt, uint64_t od,
                                const float *d_x, float *d_h, float *d_h2, float *d_down,
                                float *d_y, uint32_t n_ff, uint32_t in_dim, uint32_t n_embd) {
    (void)d_h2;
    (void)d_down;
    if (!g_q4b.ok || !base || !slots || !wts || !n || n > 64 || !d_x || !d_h || !d_y || !n_embd)
        return false;
    if (!shape_ok(gt, ut, dt, in_dim, n_ff) || !place_ok(gt, dt, base) || !tile_offsets_ok(base, stride, og, ou, od))
        return false;
    // Like the reference (src/q4_rocm.cu:5441-5445) the list goes through mapped
    // host memory: the kernels fetch it themselves, no copy node on the stream.
    // The previous exec must have finished reading it.
    if (cudaStreamSynchronize(g_q4b.stream) != cudaSuccess) return false;
    memcpy(g_q4b.es_h, slots, n * sizeof(int32_t));
    memcpy(g_q4b.ew_h, wts, n * sizeof(float));
    *g_q4b.en_h = (int32_t)n;
    if (!quant_x(d_x, in_dim)) return false;
    return moe_exec_tail(base, stride, g_q4b.es_d, g_q4b.ew_d, n, nullptr, og, ou, od, d_h, d_y,
                         n_ff, in_dim, n_embd, dt, gt);
}

extern "C" bool q4_hip_moe_exec_dev(const uint8_t *base, uint64_t stride, const int32_t *d_es,
                                    const float *d_ew, const int32_t *d_nhit, uint32_t gt,
                                    uint64_t og, uint32_t ut, uint64_t ou, uint32_t dt, uint64_t od,
                                    const float *d_x, float *d_h, float *d_h2, float *d_down,
                                    float *d_y, uint32_t n_ff, uint32_t in_dim, uint32_t n_embd) {
    (void)d_h2;
    (void)d_down;
    if (!g_q4b.ok || !base || !d_es || !d_ew || !d_nhit || !d_x || !d_h || !d_y || !n_embd)
        return false;
    if (!shape_ok(gt, ut, dt, in_dim, n_ff) || !place_ok(gt, dt, base) || !tile_offsets_ok(base, stride, og, ou, od))
        return false;
    if (!quant_x(d_x, in_dim)) return false;
    return moe_exec_tail(base, stride, d_es, d_ew, 0, d_nhit, og, ou, od, d_h, d_y, n_ff, in_dim,
                         n_embd, dt, gt);
}

extern "C" bool q4_hip_softmax_topk_launch(const float *d_logits, uint32_t n, uint32_t k,
                                           int32_t *d_ids, float *d_wts) {
    if (!g_q4b.ok || !d_logits || !d_ids || !d_wts || n == 0 || n > 1024 || k == 0 || k > 64)
        return false;
    softmax_topk_k<<<1, 32, 0, g_q4b.stream>>>(d_logits, n, k, d_ids, d_wts, k, -1, nullptr);
    g_q4b_launches++;
    return q4b_launch_ok("softmax_topk");
}

extern "C" bool q4_hip_softmax_topk(const float *d_logits, uint32_t n, uint32_t k, int32_t *h_ids,
                                    float *h_wts) {
    if (!h_ids || !h_wts) return false;
    Q4bState &s = g_q4b;
    if (!q4_hip_softmax_topk_launch(d_logits, n, k, s.topk_ids_d, s.topk_wts_d)) return false;
    const uint32_t kk = k > n ? n : k;
    Q4B_CHECK(cudaMemcpyAsync(s.topk_ids_h, s.topk_ids_d, kk * 4, cudaMemcpyDeviceToHost, s.stream));
    Q4B_CHECK(cudaMemcpyAsync(s.topk_wts_h, s.topk_wts_d, kk * 4, cudaMemcpyDeviceToHost, s.stream));
    Q4B_CHECK(cudaStreamSynchronize(s.stream));
    memcpy(h_ids, s.topk_ids_h, kk * 4);
    memcpy(h_wts, s.topk_wts_h, kk * 4);
    return true;
}

extern "C" bool q4_hip_grouped_rms_n(const float *x, const float *w, float *y, uint32_t n_embd,
                                     uint32_t hc, float eps, uint32_t n_tok) {
    if (!g_q4b.ok || !x || !y || n_embd == 0 || hc == 0 || n_tok == 0) return false;
    rms_q8_k<<<dim3(hc, n_tok), 256, 0, g_q4b.stream>>>(x, w, y, n_embd, hc, eps, nullptr, nullptr,
                                                       nullptr, 0, 0);
    g_q4b_launches++;
    return q4b_launch_ok("grouped_rms");
}
// Stream update alone (reference q4_hip_hc_combine[_n], src/q4.h:1366,1376).
extern "C" bool q4_hip_hc_combine_n(float *res, const float *block, const float *inject, uint32_t n_embd,
                                    uint32_t hc, uint32_t n_tok) {
    if (!g_q4b.ok || !res || !block || !inject || n_embd == 0 || hc == 0) return false;
    hc_streams_k<false><<<dim3(hc, n_tok ? n_tok : 1), 256, 0, g_q4b.stream>>>(res, block, nullptr, inject, nullptr,
                                                                               nullptr, n_embd, hc, 0.f);
    g_q4b_launches++;
    return q4b_launch_ok("hc_combine");
}
extern "C" bool q4_hip_hc_combine(float *res, const float *block, const float *inject, uint32_t n_embd,
                                  uint32_t hc) {
    return q4_hip_hc_combine_n(res, block, inject, n_embd, hc, 1);
}
// Update + norm in one launch (reference q4_hip_hc_comb_rms[_n], src/q4.h:1368-1375); y == NULL:
// the update only (with the hy merge).
extern "C" bool q4_hip_hc_comb_rms_n(float *res, const float *block, const float *hy, const float *inject,
                                     const float *wn, float *y, uint32_t n_embd, uint32_t hc, float eps,
                                     uint32_t n_tok) {
    if (!g_q4b.ok || !res || !block || !inject || !n_tok || n_embd == 0 || hc == 0) return false;
    const dim3 grid(hc, n_tok);
    if (y)
        hc_streams_k<true><<<grid, 256, 0, g_q4b.stream>>>(res, block, hy, inject, wn, y, n_embd, hc, eps);
    else
        hc_streams_k<false><<<grid, 256, 0, g_q4b.stream>>>(res, block, hy, inject, nullptr, nullptr, n_embd, hc, eps);
    g_q4b_launches++;
    return q4b_launch_ok("hc_comb_rms");
}
extern "C" bool q4_hip_hc_comb_rms(float *res, const float *block, const float *inject, const float *wn,
                                   float *y, uint32_t n_embd, uint32_t hc, float eps) {
    if (!y) return false;
    return q4_hip_hc_comb_rms_n(res, block, nullptr, inject, wn, y, n_embd, hc, eps, 1);
}
extern "C" bool q4_hip_grouped_rms(const float *x, const float *w, float *y, uint32_t n_embd,
                                   uint32_t hc, float eps) {
    return q4_hip_grouped_rms_n(x, w, y, n_embd, hc, eps, 1);
}

extern "C" bool q4_hip_gemv_dd_n(uint32_t ggml_type, const uint8_t *d_w, uint64_t nrows,
                                 uint64_t ncols, const float *d_x, float *d_y, float scale,
                                 uint32_t n_batch) {
    if (!g_q4b.ok || !d_w || !d_x || !d_y || nrows == 0 || ncols == 0 || n_batch == 0) return false;
    const dim3 grid((unsigned)((nrows + 7) / 8), n_batch);
    if (ggml_type == Q4_T_F32 && n_batch >= 512 && (nrows % 64u) == 0 && (ncols % 16u) == 0 &&
        nrows <= 0xffffffffull && ncols <= 0xffffffffull) {
        // a large batch: one tiled product instead of n_batch matrix-vector passes over W
        gemm_f32_nt_k<128><<<dim3((unsigned)(nrows / 64), (n_batch + 127) / 128), 256, 0, g_q4b.stream>>>(
            reinterpret_cast<const float *>(d_w), (uint32_t)nrows, (uint32_t)ncols, d_x, n_batch, d_y, scale);
    } else if (ggml_type == Q4_T_F32 && n_batch >= 2 && ncols == 2048) {
        gemv_f32_x16_k<<<dim3((unsigned)((nrows + 7) / 8), (n_batch + 15) / 16), 256, 0, g_q4b.stream>>>(
            reinterpret_cast<const float *>(d_w), nrows, d_x, n_batch, d_y, scale);
    } else if (ggml_type == Q4_T_F32) {
        gemv_f32_k<<<grid, 256, 0, g_q4b.stream>>>(reinterpret_cast<const float *>(d_w), nrows,
                                                  ncols, d_x, d_y, scale);
    } else if (ggml_type == Q4_T_IQ3_S) {
        if (ncols % Q4B_QK) return false;
        if (q4b_ptr_tiled(d_w))
            gemv_iq3s_f32_k<true><<<grid, 256, 0, g_q4b.stream>>>(d_w, nrows, (uint32_t)ncols, d_x, d_y, scale);
        else
            gemv_iq3s_f32_k<false><<<grid, 256, 0, g_q4b.stream>>>(d_w, nrows, (uint32_t)ncols, d_x, d_y, scale);
    } else {
        return false;
    }
    g_q4b_launches++;
    return q4b_launch_ok("gemv");
}
extern "C" bool q4_hip_gemv_dd(uint32_t ggml_type, const uint8_t *d_w, uint64_t nrows,
                               uint64_t ncols, const float *d_x, float *d_y, float scale) {
    return q4_hip_gemv_dd_n(ggml_type, d_w, nrows, ncols, d_x, d_y, scale, 1);
}

extern "C" bool q4_cuda_quant8(const float *d_x, uint64_t n, int8_t *d_q, float *d_d,
                               int32_t *d_bs) {
    if (!g_q4b.ok || !d_x || !d_q || !d_d || n == 0 || (n & 31u)) return false;
    const uint64_t ngr = n / 32;
    quant8_k<<<(unsigned)((ngr + 7) / 8), 256, 0, g_q4b.stream>>>(d_x, 0, (uint32_t)ngr, ngr, d_q,
                                                                 d_d, d_bs, 0, 0, nullptr);
    g_q4b_launches++;
    return q4b_launch_ok("quant8");
}

extern "C" bool q4_cuda_iq3s_dequant(const uint8_t *d_w, uint64_t nrows, uint64_t ncols,
                                     float *d_out) {
    if (!g_q4b.ok || !d_w || !d_out || nrows == 0 || ncols == 0 || (ncols % Q4B_QK)) return false;
    const uint64_t ngr = nrows * ncols / 32;
    if (q4b_ptr_tiled(d_w))
        iq3s_dequant_k<true><<<(unsigned)((ngr + 255) / 256), 256, 0, g_q4b.stream>>>(d_w, ngr, d_out);
    else
        iq3s_dequant_k<false><<<(unsigned)((ngr + 255) / 256), 256, 0, g_q4b.stream>>>(d_w, ngr, d_out);
    g_q4b_launches++;
    return q4b_launch_ok("iq3s_dequant");
}

// Stage tests for the 4-bit formats: type 20 (IQ4_NL) or 23 (IQ4_XS).
extern "C" bool q4_cuda_iq4_dequant(uint32_t type, const uint8_t *d_w, uint64_t nrows, uint64_t ncols,
                                    float *d_out) {
    if (!g_q4b.ok || !d_w || !d_out || nrows == 0 || ncols == 0) return false;
    if (!(type == Q4_T_IQ4_NL && (ncols % 32u) == 0) && !(type == Q4_T_IQ4_XS && (ncols % 256u) == 0))
        return false;
    const uint32_t gpr = (uint32_t)(ncols / 32u);
    const uint64_t n = nrows * gpr;
    if (type == Q4_T_IQ4_NL)
        iq4_dequant_k<Q4_T_IQ4_NL><<<(unsigned)((n + 255) / 256), 256, 0, g_q4b.stream>>>(d_w, n, gpr, d_out);
    else
        iq4_dequant_k<Q4_T_IQ4_XS><<<(unsigned)((n + 255) / 256), 256, 0, g_q4b.stream>>>(d_w, n, gpr, d_out);
    g_q4b_launches++;
    return q4b_launch_ok("iq4_dequant");
}
extern "C" bool q4_cuda_iq4_idot(uint32_t type, const uint8_t *d_w, uint64_t nrows, uint64_t ncols,
                                 const int8_t *d_q, int32_t *d_I) {
    if (!g_q4b.ok || !d_w || !d_q || !d_I || nrows == 0 || ncols == 0) return false;
    if (!(type == Q4_T_IQ4_NL && (ncols % 32u) == 0) && !(type == Q4_T_IQ4_XS && (ncols % 256u) == 0))
        return false;
    const uint32_t gpr = (uint32_t)(ncols / 32u);
    const uint64_t n = nrows * gpr;
    if (type == Q4_T_IQ4_NL)
        iq4_idot_k<Q4_T_IQ4_NL><<<(unsigned)((n + 255) / 256), 256, 0, g_q4b.stream>>>(d_w, nrows, gpr, d_q, d_I);
    else
        iq4_idot_k<Q4_T_IQ4_XS><<<(unsigned)((n + 255) / 256), 256, 0, g_q4b.stream>>>(d_w, nrows, gpr, d_q, d_I);
    g_q4b_launches++;
    return q4b_launch_ok("iq4_idot");
}
// Stage tests of IQ3_XXS (18), IQ2_S (22), Q2_0 (42): dequantised rows, and the exact integer part of
// every 32-group's dot with int8 activations (before the sub-scales; Q2_0: codes 0..3 x q).
extern "C" bool q4_cuda_fmt_dequant(uint32_t type, const uint8_t *d_w, uint64_t nrows, uint64_t ncols,
                                    float *d_out) {
    const uint32_t per = type == Q4_T_Q2_0 ? 64u : 256u;
    if (!g_q4b.ok || !d_w || !d_out || !nrows || !ncols || (ncols % per) ||
        (type != Q4_T_IQ3_XXS && type != Q4_T_IQ2_S && type != Q4_T_Q2_0))
        return false;
    const uint32_t gpr = (uint32_t)(ncols / 32u);
    const uint64_t n = nrows * gpr;
    const unsigned grid = (unsigned)((n + 255) / 256);
    if (type == Q4_T_IQ3_XXS)
        small_dequant_k<Q4_T_IQ3_XXS><<<grid, 256, 0, g_q4b.stream>>>(d_w, n, gpr, g_q4b.grid3xxs_d, g_q4b.grid2s_d, d_out);
    else if (type == Q4_T_IQ2_S)
        small_dequant_k<Q4_T_IQ2_S><<<grid, 256, 0, g_q4b.stream>>>(d_w, n, gpr, g_q4b.grid3xxs_d, g_q4b.grid2s_d, d_out);
    else
        small_dequant_k<Q4_T_Q2_0><<<grid, 256, 0, g_q4b.stream>>>(d_w, n, gpr, g_q4b.grid3xxs_d, g_q4b.grid2s_d, d_out);
    g_q4b_launches++;
    return q4b_launch_ok("fmt_dequant");
}
extern "C" bool q4_cuda_fmt_idot(uint32_t type, const uint8_t *d_w, uint64_t nrows, uint64_t ncols,
                                 const int8_t *d_q, int32_t *d_I) {
    const uint32_t per = type == Q4_T_Q2_0 ? 64u : 256u;
    if (!g_q4b.ok || !d_w || !d_q || !d_I || !nrows || !ncols || (ncols % per) ||
        (type != Q4_T_IQ3_XXS && type != Q4_T_IQ2_S && type != Q4_T_Q2_0))
        return false;
    const uint32_t gpr = (uint32_t)(ncols / 32u);
    const unsigned grid = (unsigned)((nrows * gpr + 255) / 256);
    if (type == Q4_T_IQ3_XXS)
        small_idot_k<Q4_T_IQ3_XXS><<<grid, 256, 0, g_q4b.stream>>>(d_w, nrows, gpr, g_q4b.grid3xxs_d, g_q4b.grid2s_d, d_q, d_I);
    else if (type == Q4_T_IQ2_S)
        small_idot_k<Q4_T_IQ2_S><<<grid, 256, 0, g_q4b.stream>>>(d_w, nrows, gpr, g_q4b.grid3xxs_d, g_q4b.grid2s_d, d_q, d_I);
    else
        small_idot_k<Q4_T_Q2_0><<<grid, 256, 0, g_q4b.stream>>>(d_w, nrows, gpr, g_q4b.grid3xxs_d, g_q4b.grid2s_d, d_q, d_I);
    g_q4b_launches++;
    return q4b_launch_ok("fmt_idot");
}

extern "C" bool q4_cuda_iq4nl_dequant(const uint8_t *d_w, uint64_t nrows, uint64_t ncols, float *d_out) {
    return q4_cuda_iq4_dequant(Q4_T_IQ4_NL, d_w, nrows, ncols, d_out);
}
extern "C" bool q4_cuda_iq4nl_idot(const uint8_t *d_w, uint64_t nrows, uint64_t ncols, const int8_t *d_q,
                                   int32_t *d_I) {
    return q4_cuda_iq4_idot(Q4_T_IQ4_NL, d_w, nrows, ncols, d_q, d_I);
}

extern "C" bool q4_cuda_iq3s_idot(const uint8_t *d_w, uint64_t nrows, uint64_t ncols,
                                  const int8_t *d_q, int32_t *d_I) {
    if (!g_q4b.ok || !d_w || !d_q || !d_I || nrows == 0 || ncols == 0 || (ncols % Q4B_QK))
        return false;
    const uint64_t items = nrows * (ncols / 32);
    if (q4b_ptr_tiled(d_w))
        iq3s_idot_k<true><<<(unsigned)((items + 255) / 256), 256, 0, g_q4b.stream>>>(
            d_w, nrows, (uint32_t)(ncols / 32), d_q, d_I);
    else
        iq3s_idot_k<false><<<(unsigned)((items + 255) / 256), 256, 0, g_q4b.stream>>>(
            d_w, nrows, (uint32_t)(ncols / 32), d_q, d_I);
    g_q4b_launches++;
    return q4b_launch_ok("iq3s_idot");
}

// One MoE layer, one token, as a chain of the kernels above (five launches,
// no host round trip).
extern "C" bool q4_cuda_moe_decode(const uint8_t *base, uint64_t stride, uint64_t og, uint64_t ou,
                                   uint64_t od, int32_t shared_slot, const float *d_x,
                                   const float *d_norm_w, float eps, const float *d_router,
                                   uint32_t n_expert, uint32_t topk, uint32_t n_embd,
                                   uint32_t n_ff, float *d_y, int32_t *d_ids, float *d_wts) {
    Q4bState &s = g_q4b;
    if (!s.ok || !base || !d_x || !d_router || !d_y) return false;
    if (!shape_ok(Q4_T_IQ3_S, Q4_T_IQ3_S, Q4_T_IQ3_S, n_embd, n_ff)) return false;
    if (n_expert == 0 || n_expert > 1024 || topk == 0 || topk > 63 || topk > n_expert) return false;
    // The single persistent kernel when it applies (Q4B_FUSED=0 forces the chain).
    const bool fused_on = decode_fused_on();
    if (fused_on && q4b_moe_decode_fused(base, stride, og, ou, od, shared_slot, d_x, d_norm_w, eps,
                                         d_router, n_expert, topk, n_embd, n_ff, d_y, d_ids, d_wts,
                                         nullptr, nullptr, 0, nullptr))
        return true;
    int8_t *xq = s.xq + (size_t)Q4B_X_SLICE * Q4B_XQ_MAXLEN;
    float *xd = s.xd + (size_t)Q4B_X_SLICE * (Q4B_XQ_MAXLEN / 32);
    int32_t *xbs = s.xbs + (size_t)Q4B_X_SLICE * (Q4B_XQ_MAXLEN / 32);
    rms_q8_k<<<dim3(1, 1), 256, 0, s.stream>>>(d_x, d_norm_w, s.xn, n_embd, 1, eps, xq, xd, xbs, 0,
                                              0);
    g_q4b_launches++;
    if (!q4b_launch_ok("rms_q8")) return false;
    gemv_f32_k<<<dim3((n_expert + 7) / 8, 1), 256, 0, s.stream>>>(d_router, n_expert, n_embd, s.xn,
                                                                 s.logits, 1.0f);
    g_q4b_launches++;
    if (!q4b_launch_ok("router_gemv")) return false;
    softmax_topk_k<<<1, 32, 0, s.stream>>>(s.logits, n_expert, topk, s.r_ids, s.r_wts, 64,
                                          shared_slot, s.r_cnt);
    g_q4b_launches++;
    if (!q4b_launch_ok("softmax_topk")) return false;
    if (cudaMemsetAsync(d_y, 0, (size_t)n_embd * sizeof(float), s.stream) != cudaSuccess)
        return false;
    if (!moe_exec_tail(base, stride, s.r_ids, s.r_wts, 0, s.r_cnt, og, ou, od, s.hbuf, d_y, n_ff,
                       n_embd, n_embd))
        return false;
    if (d_ids &&
        cudaMemcpyAsync(d_ids, s.r_ids, topk * 4, cudaMemcpyDeviceToDevice, s.stream) != cudaSuccess)
        return false;
    if (d_wts &&
        cudaMemcpyAsync(d_wts, s.r_wts, topk * 4, cudaMemcpyDeviceToDevice, s.stream) != cudaSuccess)
        return false;
    return true;
}

// The same layer call for a caller that holds host buffers: copies the hidden
// state in, runs the layer, copies the result out and waits for it.
extern "C" bool q4_cuda_moe_decode_host(const uint8_t *base, uint64_t stride, uint64_t og,
                                        uint64_t ou, uint64_t od, int32_t shared_slot,
                                        const float *h_x, const float *d_norm_w, float eps,
                                        const float *d_router, uint32_t n_expert, uint32_t topk,
                                        uint32_t n_embd, uint32_t n_ff, float *h_y) {
    Q4bState &s = g_q4b;
    if (!s.ok || !h_x || !h_y || n_embd == 0 || n_embd > Q4B_XQ_MAXLEN) return false;
    // staging rows: the last token row of the norm scratch (in) and the row before it (out)
    float *d_x = s.xn + (size_t)(Q4B_MAX_TOK - 1) * Q4B_XQ_MAXLEN;
    float *d_y = s.xn + (size_t)(Q4B_MAX_TOK - 2) * Q4B_XQ_MAXLEN;
    // Fast hand-off: when the result buffer is pinned, mapped host memory (q4_hip_host_alloc_coh)
    // the persistent kernel's last CTA writes y straight into it and raises a mapped flag the
    // host spins on -- no copy node, no stream wake-up.  Anything else takes copy + sync.
    const bool fused_on = decode_fused_on();
    // The alias of the result buffer is looked up on every call (about a microsecond): a cached
    // alias would outlive a buffer that was freed and whose address was handed out again.
    // q4_cuda_decode_plan_host keeps the alias with the plan instead.
    float *y_dev_alias = nullptr;
    if (fused_on && s.flag_h && base && d_router) y_dev_alias = q4b_host_alias(h_y);
    if (y_dev_alias && shape_ok(Q4_T_IQ3_S, Q4_T_IQ3_S, Q4_T_IQ3_S, n_embd, n_ff) && n_expert != 0 &&
        topk != 0 && topk <= n_expert) {
        const uint32_t epoch = q4b_next_flag_epoch();
        // the hidden row goes in with the launch (kernel parameter block): no copy node either
        if (q4b_moe_decode_fused(base, stride, og, ou, od, shared_slot, d_x, d_norm_w, eps, d_router,
                                 n_expert, topk, n_embd, n_ff, d_y, nullptr, nullptr, y_dev_alias,
                                 s.flag_d, epoch, h_x))
            return q4b_wait_flag(epoch);
    }
    Q4B_CHECK(cudaMemcpyAsync(d_x, h_x, (size_t)n_embd * 4, cudaMemcpyHostToDevice, s.stream));
    if (!q4_cuda_moe_decode(base, stride, og, ou, od, shared_slot, d_x, d_norm_w, eps, d_router,
                            n_expert, topk, n_embd, n_ff, d_y, nullptr, nullptr))
        return false;
    Q4B_CHECK(cudaMemcpyAsync(h_y, d_y, (size_t)n_embd * 4, cudaMemcpyDeviceToHost, s.stream));
    Q4B_CHECK(cudaStreamSynchronize(s.stream));
    return true;
}

// ---- a layer's arguments bound once (the per-token call then takes the two buffers only) ----
struct Q4bDecodePlan {
    const uint8_t *base;
    uint64_t stride, og, ou, od;
    int32_t shared_slot;
    const float *d_norm_w, *d_router;
    float eps;
    uint32_t n_expert, topk, n_embd, n_ff;
    void *stack;    // the one-layer form of q4_cuda_decode_stack_plan when the persistent kernel takes the shape
};
static bool decode_fused_on() {
    static int on = -1;
    if (on < 0) {
        const char *e = getenv("Q4B_FUSED");
        on = !(e && e[0] == '0');
    }
    return on != 0;
}
extern "C" void *q4_cuda_decode_plan(const uint8_t *base, uint64_t stride, uint64_t og, uint64_t ou,
                                     uint64_t od, int32_t shared_slot, const float *d_norm_w, float eps,
                                     const float *d_router, uint32_t n_expert, uint32_t topk,
                                     uint32_t n_embd, uint32_t n_ff) {
    if (!g_q4b.ok || !base || !d_router) return nullptr;
    if (!shape_ok(Q4_T_IQ3_S, Q4_T_IQ3_S, Q4_T_IQ3_S, n_embd, n_ff)) return nullptr;
    if (n_expert == 0 || n_expert > 1024 || topk == 0 || topk > 63 || topk > n_expert) return nullptr;
    Q4bDecodePlan *p = new Q4bDecodePlan{base, stride, og, ou, od, shared_slot, d_norm_w, d_router,
                                         eps, n_expert, topk, n_embd, n_ff, nullptr};
    if (decode_fused_on()) {
        const q4_cuda_stack_layer_t one = {base, d_norm_w, d_router};
        p->stack = q4_cuda_decode_stack_plan(&one, 1, stride, og, ou, od, shared_slot, eps, n_expert, topk,
                                             n_embd, n_ff);
    }
    return p;
}
extern "C" void q4_cuda_decode_plan_free(void *plan) {
    Q4bDecodePlan *p = (Q4bDecodePlan *)plan;
    if (!p) return;
    if (p->stack) q4_cuda_decode_stack_free(p->stack);
    delete p;
}
extern "C" bool q4_cuda_decode_plan_dev(void *plan, const float *d_x, float *d_y, int32_t *d_ids,
                                        float *d_wts) {
    const Q4bDecodePlan *p = (const Q4bDecodePlan *)plan;
    if (!p) return false;
    if (p->stack) return q4_cuda_decode_stack_dev(p->stack, d_x, d_y, d_ids, d_wts);
    return q4_cuda_moe_decode(p->base, p->stride, p->og, p->ou, p->od, p->shared_slot, d_x, p->d_norm_w,
                              p->eps, p->d_router, p->n_expert, p->topk, p->n_embd, p->n_ff, d_y, d_ids,
                              d_wts);
}
extern "C" bool q4_cuda_decode_plan_host(void *plan, const float *h_x, float *h_y) {
    const Q4bDecodePlan *p = (const Q4bDecodePlan *)plan;
    if (!p) return false;
    if (p->stack) return q4_cuda_decode_stack_host(p->stack, h_x, h_y);
    return q4_cuda_moe_decode_host(p->base, p->stride, p->og, p->ou, p->od, p->shared_slot, h_x,
                                   p->d_norm_w, p->eps, p->d_router, p->n_expert, p->topk, p->n_embd,
                                   p->n_ff, h_y);
}

// ---- helpers shared with the many-token path (q4b_grouped.cu) ----
bool q4b_route_tokens(const float *d_rlog, int32_t *d_ids, float *d_wts, uint32_t n_tok,
                      uint32_t n_exp, uint32_t topk) {
    softmax_topk_k<<<n_tok, 32, 0, g_q4b.stream>>>(d_rlog, n_exp, topk, d_ids, d_wts, topk, -1, nullptr);
    g_q4b_launches++;
    return q4b_launch_ok("route_tokens");
}
// norm + router + top-k of up to ROUTE_MAX_TOK tokens in one launch; false: the shape is not this kernel's (nothing
// queued, the caller issues the three launches)
static unsigned int *g_route_counter = nullptr;   // one counter per group of eight tokens
constexpr uint32_t ROUTE_MAX_TOK = 256;
bool q4b_route_small_warm() {
    if (g_route_counter) return true;
    if (cudaMalloc(&g_route_counter, (ROUTE_MAX_TOK / 8u) * sizeof(unsigned int)) != cudaSuccess ||
        cudaMemset(g_route_counter, 0, (ROUTE_MAX_TOK / 8u) * sizeof(unsigned int)) != cudaSuccess ||
        cudaFuncSetAttribute(route_small_k, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 2048 * 4) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return true;
}
void q4b_route_small_shutdown() {
    cudaFree(g_route_counter);
    g_route_counter = nullptr;
}
bool q4b_route_small(const float *x, const float *norm_w, float eps, const float *router, uint32_t n_expert,
                     uint32_t topk, uint32_t n_embd, uint32_t n_tok, float *xn, float *logits, int32_t *ids,
                     float *wts) {
    if (!g_route_counter || n_embd != 2048u || n_tok == 0 || n_tok > ROUTE_MAX_TOK || n_expert > 1024u ||
        topk > 64u || (((uintptr_t)router | (uintptr_t)x | (uintptr_t)norm_w | (uintptr_t)xn) & 15u))
        return false;
    route_small_k<<<dim3((n_expert + 7u) / 8u, (n_tok + 7u) / 8u), 256, 8u * 2048u * 4u, g_q4b.stream>>>(
        x, norm_w, eps, router, n_expert, n_tok, topk, xn, logits, ids, wts, g_route_counter);
    g_q4b_launches++;
    return q4b_launch_ok("route_small");
}
bool q4b_rms_rows(const float *x, const float *w, float *y, uint32_t n_embd, float eps,
                  uint32_t n_tok) {
    rms_q8_k<<<dim3(1, n_tok), 256, 0, g_q4b.stream>>>(x, w, y, n_embd, 1, eps, nullptr, nullptr,
                                                      nullptr, 0, 0);
    g_q4b_launches++;
    return q4b_launch_ok("rms_rows");
}
