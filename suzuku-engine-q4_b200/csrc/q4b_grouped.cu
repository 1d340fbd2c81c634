// The many-token path: rows grouped by expert, every weight tile decoded once
// and dotted with all the rows of its expert.
//
// This is the engine's prefill / verify-window call sequence
// (src/q4_moe.c:3166-3251, 3697-3748, 3887) behind the same entry points:
//   q4_hip_route_pf      per-token softmax + top-k            (src/q4_rocm.cu:6383)
//   q4_hip_assign_pf     rows sorted by expert per token group (src/q4_rocm.cu:6483)
//   q4_mmq_quantize      activation rows -> 8-bit blocks       (src/q4_mmq.cu:365)
//   q4_mmq_mul_id        grouped IQ3_S x int8 product          (src/q4_mmq.cu:387)
//   q4_mmq_swiglu        h = silu(g) * u                       (src/q4_mmq.cu:603)
//   q4_hip_expert_reduce y[t] += sum_k rw * pd[rsrc]           (src/q4_rocm.cu:15739)
// plus q4_hip_moe_exec_win (2..8 tokens, src/q4_rocm.cu:7444) and the fused
// q4_cuda_moe_layer_n built from them.
//
// Arithmetic: activations are quantised with Q8-A (src/q4_cpuexp.c:605-637), so a
// row's result is the same whatever batch it arrives in (the reference's window
// path has the same property, src/q4_cpuexp.c:1727-1730).  The grouped product
// here is the CUDA-core form: right for the few rows per expert of decode,
// verify windows and expert-parallel shards.
#include "q4b_tile.cuh"

#include <atomic>

#include "../../include/q4cuda.h"

extern std::atomic<uint64_t> g_q4b_launches;
bool q4b_ptr_tiled(const void *p);
// defined in q4b_decode.cu
bool q4b_route_tokens(const float *d_rlog, int32_t *d_ids, float *d_wts, uint32_t n_tok,
                      uint32_t n_exp, uint32_t topk);
bool q4b_route_small(const float *x, const float *norm_w, float eps, const float *router, uint32_t n_expert,
                     uint32_t topk, uint32_t n_embd, uint32_t n_tok, float *xn, float *logits, int32_t *ids,
                     float *wts);
bool q4b_rms_rows(const float *x, const float *w, float *y, uint32_t n_embd, float eps,
                  uint32_t n_tok);

namespace grouped {

// Quantised activation rows, planar: int8 q[rows][cols], then float d[rows][cols/32],
// then int32 bs[rows][cols/32]; then scratch of the tensor-core product, which that product
// fills itself: two fp16 planes [rows][cols] and one float per row.  Each section 256-byte aligned.
struct Q8View {
    const int8_t *q;
    const float *d;
    const int32_t *bs;
    __half *h1, *h2;
    float *rs;
};
__host__ __device__ inline uint64_t align256(uint64_t v) { return (v + 255u) & ~(uint64_t)255u; }
__host__ __device__ inline uint64_t q8_bytes(uint64_t rows, uint64_t cols) {
    return align256(rows * cols) + 2u * align256(rows * (cols / 32) * 4u) + 2u * align256(rows * cols * 2u) +
           align256(rows * 4u) + 256u;
}
__host__ __device__ inline Q8View q8_view(const void *buf, uint64_t rows, uint64_t cols) {
    Q8View v;
    uint8_t *p = (uint8_t *)buf;
    v.q = (const int8_t *)p;
    p += align256(rows * cols);
    v.d = (const float *)p;
    p += align256(rows * (cols / 32) * 4u);
    v.bs = (const int32_t *)p;
    p += align256(rows * (cols / 32) * 4u);
    v.h1 = (__half *)p;
    p += align256(rows * cols * 2u);
    v.h2 = (__half *)p;
    p += align256(rows * cols * 2u);
    v.rs = (float *)p;
    return v;
}

// The two 8-bit quantisers of activation rows.  Q8-A (the product's own; the reference's CPU path):
// d = amax / 127, q = round-to-nearest-even(x * (127 / amax)).  Q8-C (COMPAT = true; ggml's q8_1, what
// the reference's grouped device product quantises with, quantize.cu:491-553 of its vendored ggml):
// d_inv = 127 / amax, q = round-half-away(x * d_inv), d = 1 / d_inv.  They differ on exact halves and
// in the last bit of d.
template <bool COMPAT> __device__ __forceinline__ int q8_round(float v, float sc) {
    const float t = __fmul_rn(v, sc);
    return max(-128, min(127, COMPAT ? (int)roundf(t) : __float2int_rn(t)));
}
template <bool COMPAT> __device__ __forceinline__ float q8_scale(float amax, float sc) {
    return COMPAT ? (sc > 0.f ? __fdiv_rn(1.0f, sc) : 0.f) : __fdiv_rn(amax, 127.f);
}
int g_q8_compat = 0;   // q4_cuda_mmq_q8_compat

// Four lanes per 32 values of one gathered row, eight values each (a negative source row
// gives zeros).
template <bool COMPAT>
__global__ void quantize_rows_k(const float *__restrict__ x, const int32_t *__restrict__ ids,
                                uint64_t cols, uint64_t rows, int8_t *__restrict__ q,
                                float *__restrict__ d, int32_t *__restrict__ bs) {
    const uint32_t gpr = (uint32_t)(cols >> 5);
    const uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t g = t >> 2;                       // 32-group
    const uint32_t part = (uint32_t)t & 3u;          // eight values of it
    const bool live = g < rows * gpr;                // whole quads are live or not
    const uint64_t r = live ? g / gpr : 0, gl = live ? g - r * gpr : 0;
    const int64_t src = !live ? -1 : (ids ? (int64_t)ids[r] : (int64_t)r);
    float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
    if (src >= 0) {
        const float4 *p = reinterpret_cast<const float4 *>(x + (uint64_t)src * cols + gl * 32u + part * 8u);
        v0 = __ldg(p);
        v1 = __ldg(p + 1);
    }
    float a = fmaxf(fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v0.z), fabsf(v0.w))),
                    fmaxf(fmaxf(fabsf(v1.x), fabsf(v1.y)), fmaxf(fabsf(v1.z), fabsf(v1.w))));
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 2));
    const float sc = a > 0.f ? __fdiv_rn(127.f, a) : 0.f;
    auto qz = [&](float v) { return q8_round<COMPAT>(v, sc); };
    const int q0 = qz(v0.x), q1 = qz(v0.y), q2 = qz(v0.z), q3 = qz(v0.w);
    const int q4 = qz(v1.x), q5 = qz(v1.y), q6 = qz(v1.z), q7 = qz(v1.w);
    int sum = q0 + q1 + q2 + q3 + q4 + q5 + q6 + q7;
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if (!live) return;
    uint2 o;
    o.x = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) |
          ((uint32_t)(q3 & 0xff) << 24);
    o.y = (uint32_t)(q4 & 0xff) | ((uint32_t)(q5 & 0xff) << 8) | ((uint32_t)(q6 & 0xff) << 16) |
          ((uint32_t)(q7 & 0xff) << 24);
    *reinterpret_cast<uint2 *>(q + r * cols + gl * 32u + part * 8u) = o;
    if (part == 0) {
        d[g] = q8_scale<COMPAT>(a, sc);
        bs[g] = sum;
    }
}

// One 32-weight group -> eight words of sign-applied code bytes c' (weight = 2c'+1).
template <bool TILED>
__device__ __forceinline__ void decode_group(const Iq3Fields &f, const uint32_t *tab, uint32_t *cw) {
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const uint32_t wq = k < 4 ? f.qs_lo : f.qs_hi;
        const uint32_t idx = ((wq >> (8 * (k & 3))) & 0xffu) | (((f.qh >> k) & 1u) << 8);
        uint32_t m;
        if (TILED) {
            const uint32_t t = f.sg << k;
            m = q4b_prmt(t, t, 0xba98u);
        } else {
            m = q4b_sign_mask4(f.sg >> (4 * k));
        }
        cw[k] = tab[idx] ^ m;
    }
}

// Grouped product.  Entry i (blockIdx.y) owns activation rows [bounds[i], bounds[i+1])
// and the weight matrix w + slot * expert_stride with slot = act ? act[i] : i; entries
// at or beyond *n_act (when given) do nothing.  One warp takes eight consecutive
// super-blocks (one tile): lane l owns block l/4 and sub-block pair l%4.  With B blocks
// per weight row a tile spans 8/B whole rows when B is 1, 2, 4 or 8 (rows summed by
// shuffles, reproducible); for any other B a row's blocks lie in several warps and the
// per-block partial sums are added with atomics into dst, which the caller zeroes.
template <bool TILED>
__global__ void __launch_bounds__(256) grouped_rows_k(
    const uint8_t *__restrict__ w, uint64_t expert_stride, const int32_t *__restrict__ act,
    const uint32_t *__restrict__ n_act, const int32_t *__restrict__ bounds, Q8View xq,
    uint32_t cols, uint32_t w_rows, float *__restrict__ dst, uint64_t ld_dst,
    const uint32_t *__restrict__ codes) {
    __shared__ uint32_t tab[512];
    const uint32_t entry = blockIdx.y;
    if (n_act && entry >= *n_act) return;
    const int32_t r0 = bounds[entry], r1 = bounds[entry + 1];
    if (r1 <= r0) return;
    tab[threadIdx.x] = __ldg(codes + threadIdx.x);
    tab[threadIdx.x + 256u] = __ldg(codes + threadIdx.x + 256u);
    __syncthreads();
    const uint32_t B = cols >> 8;                        // super-blocks per weight row
    const uint32_t n_tiles = (w_rows * B) >> 3;
    const uint32_t lane = threadIdx.x & 31u, p = lane & 3u;
    const uint8_t *mat = w + (uint64_t)(act ? act[entry] : (int32_t)entry) * expert_stride;
    const uint32_t ngr = cols >> 5;
    const bool pow2 = B == 1 || B == 2 || B == 4 || B == 8;
    const uint32_t lanes_per_row = 4u * B;
    const uint32_t t_step = gridDim.x * (blockDim.x >> 5);
    uint32_t ti = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (ti >= n_tiles) return;
    // the tile after this one is fetched while this one is decoded and used
    Iq3Fields f0 = iq3_fields<TILED>(mat, ti * 8u + (lane >> 2), 2u * p);
    Iq3Fields f1 = iq3_fields<TILED>(mat, ti * 8u + (lane >> 2), 2u * p + 1u);
    for (; ti < n_tiles; ti += t_step) {
        const uint32_t bi = ti * 8u + (lane >> 2);           // this lane's super-block in the matrix
        const uint32_t wrow = bi / B, brow = bi - wrow * B;  // weight row, block within the row
        uint32_t cw[16];
        decode_group<TILED>(f0, tab, cw);
        decode_group<TILED>(f1, tab, cw + 8);
        const int ls0 = (int)f0.ls, ls1 = (int)f1.ls;
        const float dblk = f0.d;
        if (ti + t_step < n_tiles) {
            const uint32_t bn = (ti + t_step) * 8u + (lane >> 2);
            f0 = iq3_fields<TILED>(mat, bn, 2u * p);
            f1 = iq3_fields<TILED>(mat, bn, 2u * p + 1u);
        }
        const uint32_t gcol = brow * 8u + 2u * p;         // first of the lane's two 32-groups
        for (int32_t r = r0; r < r1; r++) {
            const int4 *qp = reinterpret_cast<const int4 *>(xq.q + (uint64_t)r * cols + gcol * 32u);
            const int4 q0 = __ldg(qp), q1 = __ldg(qp + 1), q2 = __ldg(qp + 2), q3 = __ldg(qp + 3);
            const uint64_t go = (uint64_t)r * ngr + gcol;
            const float2 dx = __ldg(reinterpret_cast<const float2 *>(xq.d + go));
            const int2 bsv = __ldg(reinterpret_cast<const int2 *>(xq.bs + go));
            int a0 = 0, a1 = 0;
            a0 = __dp4a((int)cw[0], q0.x, a0);
            a0 = __dp4a((int)cw[1], q0.y, a0);
            a0 = __dp4a((int)cw[2], q0.z, a0);
            a0 = __dp4a((int)cw[3], q0.w, a0);
            a0 = __dp4a((int)cw[4], q1.x, a0);
            a0 = __dp4a((int)cw[5], q1.y, a0);
            a0 = __dp4a((int)cw[6], q1.z, a0);
            a0 = __dp4a((int)cw[7], q1.w, a0);
            a1 = __dp4a((int)cw[8], q2.x, a1);
            a1 = __dp4a((int)cw[9], q2.y, a1);
            a1 = __dp4a((int)cw[10], q2.z, a1);
            a1 = __dp4a((int)cw[11], q2.w, a1);
            a1 = __dp4a((int)cw[12], q3.x, a1);
            a1 = __dp4a((int)cw[13], q3.y, a1);
            a1 = __dp4a((int)cw[14], q3.z, a1);
            a1 = __dp4a((int)cw[15], q3.w, a1);
            const int I0 = 2 * a0 + bsv.x, I1 = 2 * a1 + bsv.y;  // sum sign*(2c+1)*q = 2 sum c'q + sum q
            float v = dblk * ((float)(I0 * ls0) * dx.x + (float)(I1 * ls1) * dx.y);
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            float *o = dst + (uint64_t)r * ld_dst + wrow;
            if (pow2) {  // a weight row is 4*B neighbouring lanes of this warp
                if (B >= 2) v += __shfl_xor_sync(0xffffffffu, v, 4);
                if (B >= 4) v += __shfl_xor_sync(0xffffffffu, v, 8);
                if (B >= 8) v += __shfl_xor_sync(0xffffffffu, v, 16);
                if ((lane & (lanes_per_row - 1u)) == 0) *o = v;
            } else if (p == 0) {
                atomicAdd(o, v);  // other widths: a row is spread over warps, one add per block
            }
        }
    }
}

__global__ void swiglu_rows_k(const float *__restrict__ gu, float *__restrict__ h, uint64_t rows,
                              uint64_t n_ff) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * n_ff) return;
    const uint64_t r = i / n_ff, k = i - r * n_ff;
    h[i] = q4b_swiglu(gu[r * 2 * n_ff + k], gu[r * 2 * n_ff + n_ff + k]);
}

// h = silu(g) * u and its Q8-A quantisation in one pass (the values swiglu_rows_k followed by
// quantize_rows_k would give): four lanes per 32 hidden values, eight each.
template <bool COMPAT>
__global__ void swiglu_quant_rows_k(const float *__restrict__ gu, uint64_t rows, uint64_t n_ff,
                                    int8_t *__restrict__ q, float *__restrict__ d,
                                    int32_t *__restrict__ bs) {
    const uint32_t gpr = (uint32_t)(n_ff >> 5);
    const uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t g = t >> 2;
    const uint32_t part = (uint32_t)t & 3u;
    const bool live = g < rows * gpr;
    const uint64_t r = live ? g / gpr : 0, gl = live ? g - r * gpr : 0;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = 0.f;
    if (live) {
        const float4 *pg = reinterpret_cast<const float4 *>(gu + r * 2 * n_ff + gl * 32u + part * 8u);
        const float4 *pu = reinterpret_cast<const float4 *>(gu + r * 2 * n_ff + n_ff + gl * 32u + part * 8u);
        const float4 g0 = __ldg(pg), g1 = __ldg(pg + 1), u0 = __ldg(pu), u1 = __ldg(pu + 1);
        v[0] = q4b_swiglu(g0.x, u0.x), v[1] = q4b_swiglu(g0.y, u0.y);
        v[2] = q4b_swiglu(g0.z, u0.z), v[3] = q4b_swiglu(g0.w, u0.w);
        v[4] = q4b_swiglu(g1.x, u1.x), v[5] = q4b_swiglu(g1.y, u1.y);
        v[6] = q4b_swiglu(g1.z, u1.z), v[7] = q4b_swiglu(g1.w, u1.w);
    }
    float a = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) a = fmaxf(a, fabsf(v[i]));
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 2));
    const float sc = a > 0.f ? __fdiv_rn(127.f, a) : 0.f;
    int qi[8], sum = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        qi[i] = q8_round<COMPAT>(v[i], sc);
        sum += qi[i];
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if (!live) return;
    uint2 o;
    o.x = (uint32_t)(qi[0] & 0xff) | ((uint32_t)(qi[1] & 0xff) << 8) | ((uint32_t)(qi[2] & 0xff) << 16) |
          ((uint32_t)(qi[3] & 0xff) << 24);
    o.y = (uint32_t)(qi[4] & 0xff) | ((uint32_t)(qi[5] & 0xff) << 8) | ((uint32_t)(qi[6] & 0xff) << 16) |
          ((uint32_t)(qi[7] & 0xff) << 24);
    *reinterpret_cast<uint2 *>(q + r * n_ff + gl * 32u + part * 8u) = o;
    if (part == 0) {
        d[g] = q8_scale<COMPAT>(a, sc);
        bs[g] = sum;
    }
}

// y[t][c] (+)= sum_k rw[t][k] * pd[rsrc[t][k]][c], picks in order k = 0..topk-1; ADD = false
// overwrites y (same value as adding to a zeroed y).
template <bool ADD>
__global__ void expert_reduce_k(float *__restrict__ y, const float *__restrict__ pd,
                                const int32_t *__restrict__ rsrc, const float *__restrict__ rw,
                                uint32_t topk, uint32_t n_embd) {
    const uint32_t t = blockIdx.y;
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= n_embd) return;
    float acc = 0.f;
    for (uint32_t k = 0; k < topk; k++) {
        const int32_t p = rsrc[(uint64_t)t * topk + k];
        if (p >= 0) acc += rw[(uint64_t)t * topk + k] * pd[(uint64_t)p * n_embd + c];
    }
    if (ADD)
        y[(uint64_t)t * n_embd + c] += acc;
    else
        y[(uint64_t)t * n_embd + c] = 0.f + acc;
}
// The same sums four columns per thread (n_embd % 4 == 0, 16-byte aligned rows): the picks'
// rows are read as float4, each column still adds its picks in the order k = 0..topk-1.
template <bool ADD>
__global__ void __launch_bounds__(256) expert_reduce4_k(float *__restrict__ y, const float *__restrict__ pd,
                                                        const int32_t *__restrict__ rsrc,
                                                        const float *__restrict__ rw, uint32_t topk,
                                                        uint32_t n_embd) {
    const uint32_t t = blockIdx.y;
    const uint32_t c4 = blockIdx.x * blockDim.x + threadIdx.x;
    if (c4 >= n_embd / 4u) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t k = 0; k < topk; k++) {
        const int32_t p = rsrc[(uint64_t)t * topk + k];
        if (p >= 0) {
            const float w = rw[(uint64_t)t * topk + k];
            const float4 v = __ldcs(reinterpret_cast<const float4 *>(pd + (uint64_t)p * n_embd) + c4);
            acc.x += w * v.x;
            acc.y += w * v.y;
            acc.z += w * v.z;
            acc.w += w * v.w;
        }
    }
    float4 *o = reinterpret_cast<float4 *>(y + (uint64_t)t * n_embd) + c4;
    if (ADD) {
        const float4 old = *o;
        *o = make_float4(old.x + acc.x, old.y + acc.y, old.z + acc.z, old.w + acc.w);
    } else {
        *o = make_float4(0.f + acc.x, 0.f + acc.y, 0.f + acc.z, 0.f + acc.w);
    }
}
template <bool ADD>
static void launch_expert_reduce(float *y, const float *pd, const int32_t *rsrc, const float *rw, uint32_t n_tok,
                                 uint32_t topk, uint32_t n_embd) {
    if ((n_embd & 3u) == 0 && (((uintptr_t)y | (uintptr_t)pd) & 15u) == 0)
        expert_reduce4_k<ADD><<<dim3((n_embd / 4u + 255u) / 256u, n_tok), 256, 0, g_q4b.stream>>>(y, pd, rsrc, rw,
                                                                                                topk, n_embd);
    else
        expert_reduce_k<ADD><<<dim3((n_embd + 255) / 256, n_tok), 256, 0, g_q4b.stream>>>(y, pd, rsrc, rw, topk,
                                                                                         n_embd);
}

// One block (256 threads, or 1024 for a large group) per group of gsz tokens: a stable counting
// sort of the group's picks by expert.  Each warp owns a contiguous run of picks; per-warp histograms, a
// prefix over warps and over experts, then every warp places its own run 32 picks at a
// time, each lane finding its place among the lanes of the warp that picked the same
// expert.  Rows of one expert therefore keep (token, pick) order.
__global__ void __launch_bounds__(1024) assign_k(
    const int32_t *__restrict__ ids, const float *__restrict__ wts, int32_t *__restrict__ a_tok,
    int32_t *__restrict__ rsrc, float *__restrict__ rw, int32_t *__restrict__ stg,
    uint32_t *__restrict__ stgn, uint32_t *__restrict__ ek, int32_t *__restrict__ cbounds,
    uint32_t gsz, uint32_t topk, uint32_t n_exp, uint32_t n_tok, uint32_t ek_stride,
    uint32_t topk_in, int32_t extra_id, int32_t own_first, uint32_t own_count, uint32_t tok_first,
    uint32_t tok_count, int32_t *__restrict__ bounds_full) {
    // ids/wts hold topk_in columns per token; when topk == topk_in + 1 the last pick of every
    // token is extra_id with weight 1 (the shared expert), not read from memory.
    // own_count != 0 (expert parallelism): only picks of experts [own_first, own_first +
    // own_count) are placed, renumbered from 0, and the extra pick only for tokens
    // [tok_first, tok_first + tok_count).  bounds_full (optional) receives the first row of
    // every expert and the total: n_exp + 1 values.  Rows of a_tok beyond the total get -1.
    extern __shared__ uint32_t sh[];  // hist[nw][n_exp], cnt[n_exp], rank[n_exp], wsum[40]
    const uint32_t nw = blockDim.x >> 5;
    uint32_t *hist = sh, *cnt = sh + nw * n_exp, *rank = cnt + n_exp, *wsum = rank + n_exp;
    const uint32_t g = blockIdx.x, tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t t0 = g * gsz, t1 = min(t0 + gsz, n_tok);
    const uint32_t seg = g * gsz * topk, rows = (t1 - t0) * topk;
    const uint32_t run = ((rows + nw - 1u) / nw + 31u) & ~31u;  // picks per warp, a multiple of 32
    const uint32_t i_lo = warp * run, i_hi = min(rows, i_lo + run);
    auto pick_id = [&](uint32_t i) -> int32_t {   // i = pick index within the group
        const uint32_t t = i / topk, k = i - t * topk;
        if (k >= topk_in)
            return (own_count && (t0 + t < tok_first || t0 + t >= tok_first + tok_count)) ? -1 : extra_id;
        int32_t e = ids[(uint64_t)(t0 + t) * topk_in + k];
        if (own_count) {
            e -= own_first;
            if (e < 0 || (uint32_t)e >= own_count) e = -1;
        }
        return e;
    };
    for (uint32_t i = tid; i < nw * n_exp; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (uint32_t i0 = i_lo; i0 < i_hi; i0 += 32u) {   // one add per distinct expert of the 32 picks
        const uint32_t i = i0 + lane;
        int32_t e = i < i_hi ? pick_id(i) : -1;
        if (e < 0 || (uint32_t)e >= n_exp) e = -1;
        const uint32_t same = __match_any_sync(0xffffffffu, e);
        if (e >= 0 && (same & ((1u << lane) - 1u)) == 0) hist[warp * n_exp + e] += __popc(same);
        __syncwarp();
    }
    __syncthreads();
    // per expert: exclusive prefix over the warps, total in cnt
    for (uint32_t e = tid; e < n_exp; e += blockDim.x) {
        uint32_t tot = 0;
        for (uint32_t wv = 0; wv < nw; wv++) {
            const uint32_t c = hist[wv * n_exp + e];
            hist[wv * n_exp + e] = tot;
            tot += c;
        }
        cnt[e] = tot;
        if (ek) ek[g * ek_stride + e] = tot;
    }
    __syncthreads();
    // exclusive prefix over experts of (count, used): thread t owns experts [t*per, t*per+per)
    const uint32_t per = (n_exp + blockDim.x - 1u) / blockDim.x;
    uint32_t my_c = 0, my_u = 0;
    for (uint32_t k = 0; k < per; k++) {
        const uint32_t e = tid * per + k;
        if (e < n_exp) {
            my_c += cnt[e];
            my_u += cnt[e] ? 1u : 0u;
        }
    }
    uint32_t pack = (my_c << 10) | my_u;  // rows < 2^22, used experts <= 1023
    uint32_t inc = pack;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t v = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= (uint32_t)o) inc += v;
    }
    if (lane == 31u) wsum[warp] = inc;
    __syncthreads();
    uint32_t off = 0;
    for (uint32_t wv = 0; wv < warp; wv++) off += wsum[wv];
    uint32_t excl = off + inc - pack;
    uint32_t b = excl >> 10, nu = excl & 1023u;
    for (uint32_t k = 0; k < per; k++) {
        const uint32_t e = tid * per + k;
        if (e < n_exp) {
            const uint32_t c = cnt[e];
            rank[e] = b;  // first row of expert e
            if (c) {
                if (stg) stg[g * ek_stride + nu] = (int32_t)e;
                if (cbounds) cbounds[g * (ek_stride + 1) + nu] = (int32_t)b;
                nu++;
            }
            b += c;
        }
    }
    if (tid == blockDim.x - 1u) {  // totals
        if (cbounds) cbounds[g * (ek_stride + 1) + nu] = (int32_t)b;
        if (stgn) stgn[g] = nu;
        wsum[32] = b;
    }
    __syncthreads();
    if (bounds_full)
        for (uint32_t e = tid; e <= n_exp; e += blockDim.x)
            bounds_full[g * (n_exp + 1) + e] = (int32_t)(e < n_exp ? rank[e] : wsum[32]);
    for (uint32_t i = wsum[32] + tid; i < rows; i += blockDim.x) a_tok[seg + i] = -1;   // unused rows
    for (uint32_t i0 = i_lo; i0 < i_hi; i0 += 32u) {
        const uint32_t i = i0 + lane;
        int32_t e = -1;
        uint32_t t = 0, k = 0;
        if (i < i_hi) {
            t = t0 + i / topk;
            k = i % topk;
            e = pick_id(i);
            if (e < 0 || (uint32_t)e >= n_exp) e = -1;
        }
        const uint32_t same = __match_any_sync(0xffffffffu, e);
        if (e >= 0) {
            const uint32_t before = __popc(same & ((1u << lane) - 1u));
            const uint32_t pos = rank[e] + hist[warp * n_exp + e] + before;
            a_tok[seg + pos] = (int32_t)t;
            rsrc[(uint64_t)t * topk + k] = (int32_t)pos;
            rw[(uint64_t)t * topk + k] = k < topk_in ? wts[(uint64_t)t * topk_in + k] : 1.0f;
        } else if (i < i_hi) {
            rsrc[(uint64_t)t * topk + k] = -1;
            rw[(uint64_t)t * topk + k] = 0.f;
        }
        __syncwarp();
        if (e >= 0 && (same & ((1u << lane) - 1u)) == 0) hist[warp * n_exp + e] += __popc(same);
        __syncwarp();
    }
}

// Verify window: per-token slot lists (stride 64, count per token; n_tok <= 8) ->
// entries = distinct slots in order of first appearance, their rows in (token, pick)
// order, bounds per entry.  One block of 512 threads, one per possible pick.
__global__ void __launch_bounds__(512) win_assign_k(
    const int32_t *__restrict__ es, const float *__restrict__ ew, const int32_t *__restrict__ nh,
    uint32_t n_tok, int32_t *__restrict__ act, uint32_t *__restrict__ n_act,
    int32_t *__restrict__ bounds, int32_t *__restrict__ a_tok, int32_t *__restrict__ rsrc,
    float *__restrict__ rw) {
    __shared__ int32_t slot[512];
    __shared__ int32_t lead[512];   // index of the first pick with the same slot, or -1 (invalid)
    __shared__ int32_t ent[512];    // entry number of a leader
    __shared__ int32_t size[513];
    const uint32_t i = threadIdx.x, t = i >> 6, k = i & 63u;
    const bool valid = t < n_tok && (int32_t)k < nh[t];
    slot[i] = valid ? es[i] : -1;
    __syncthreads();
    int32_t first = -1, before = 0;
    if (valid) {
        for (uint32_t j = 0; j < i; j++)
            if (slot[j] == slot[i]) {
                if (first < 0) first = (int32_t)j;
                before++;
            }
        if (first < 0) first = (int32_t)i;
    }
    lead[i] = first;
    __syncthreads();
    // entry number of leader i = number of leaders before it
    int32_t my_ent = 0;
    if (valid && first == (int32_t)i) {
        for (uint32_t j = 0; j < i; j++) my_ent += lead[j] == (int32_t)j ? 1 : 0;
        ent[i] = my_ent;
        act[my_ent] = slot[i];
    }
    size[i] = 0;
    if (i == 0) size[512] = 0;
    __syncthreads();
    if (valid) atomicAdd(&size[ent[first]], 1);
    __syncthreads();
    if (i == 0) {
        int32_t n = 0, b = 0;
        for (uint32_t j = 0; j < 512; j++) n += lead[j] == (int32_t)j ? 1 : 0;
        for (int32_t j = 0; j < n; j++) {
            bounds[j] = b;
            b += size[j];
            size[j] = bounds[j];   // becomes the entry's first row
        }
        bounds[n] = b;
        *n_act = (uint32_t)n;
    }
    __syncthreads();
    if (valid) {
        const int32_t pos = size[ent[first]] + before;
        a_tok[pos] = (int32_t)t;
        rsrc[i] = pos;
        rw[i] = ew[i];
    } else {
        rsrc[i] = -1;
        rw[i] = 0.f;
    }
}

// The grouped product for IQ4_NL / IQ4_XS weights (type T; arenas in the engine's byte order): one
// warp per weight row of an entry.  A lane owns the row's 32-groups lane, lane + 32, ... (at most
// four: rows up to 4096 wide), turns their 4-bit codes into table values once, and dots them with
// every activation row of the entry; a row's 32 lane sums are added by the butterfly.  Integer parts
// exact (codes x int8 by dp4a); the result is the sum over groups of (d * dx) * (I * ls).
template <uint32_t T>
__global__ void __launch_bounds__(256) grouped_rows4_k(const uint8_t *__restrict__ w, uint64_t expert_stride,
                                                       const int32_t *__restrict__ act,
                                                       const uint32_t *__restrict__ n_act,
                                                       const int32_t *__restrict__ bounds, Q8View xq, uint32_t cols,
                                                       uint32_t w_rows, float *__restrict__ dst, uint64_t ld_dst) {
    __shared__ uint16_t pair[256];
    iq4_fill_pair_table(pair);
    __syncthreads();
    const uint32_t entry = blockIdx.y;
    if (n_act && entry >= *n_act) return;
    const int32_t r0 = bounds[entry], r1 = bounds[entry + 1];
    const uint32_t wrow = blockIdx.x * 8u + (threadIdx.x >> 5), lane = threadIdx.x & 31u;
    if (r1 <= r0 || wrow >= w_rows) return;
    const uint32_t ng = cols >> 5;
    const uint8_t *row = w + (uint64_t)(act ? act[entry] : (int32_t)entry) * expert_stride +
                         (uint64_t)wrow * iq4_row_bytes(T, cols);
    constexpr uint32_t GPL = 4;          // groups per lane
    uint32_t wv[GPL][8];                 // table values: words 0..3 = weights 0..15, 4..7 = weights 16..31
    float dl[GPL];                       // d * ls of the group
#pragma unroll
    for (uint32_t k = 0; k < GPL; k++) {
        const uint32_t g = lane + 32u * k;
        dl[k] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) wv[k][i] = 0u;
        if (g < ng) {
            int lsf;
            float d;
            const uint8_t *codes = iq4_group<T>(row, g, &lsf, &d);
            dl[k] = __fmul_rn(d, (float)lsf);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t c01 = q4b_ld_u16(codes + 4 * i), c23 = q4b_ld_u16(codes + 4 * i + 2);
                const uint32_t p0 = pair[c01 & 0xffu], p1 = pair[c01 >> 8], p2 = pair[c23 & 0xffu], p3 = pair[c23 >> 8];
                wv[k][i] = (p0 & 0xffu) | ((p1 & 0xffu) << 8) | ((p2 & 0xffu) << 16) | ((p3 & 0xffu) << 24);
                wv[k][4 + i] = (p0 >> 8) | ((p1 >> 8) << 8) | ((p2 >> 8) << 16) | ((p3 >> 8) << 24);
            }
        }
    }
    for (int32_t r = r0; r < r1; r++) {
        float acc = 0.f;
#pragma unroll
        for (uint32_t k = 0; k < GPL; k++) {
            const uint32_t g = lane + 32u * k;
            if (g < ng) {
                const int4 *qp = reinterpret_cast<const int4 *>(xq.q + (uint64_t)r * cols + g * 32u);
                const int4 q0 = __ldg(qp), q1 = __ldg(qp + 1);
                int I = __dp4a((int)wv[k][0], q0.x, 0);
                I = __dp4a((int)wv[k][1], q0.y, I);
                I = __dp4a((int)wv[k][2], q0.z, I);
                I = __dp4a((int)wv[k][3], q0.w, I);
                I = __dp4a((int)wv[k][4], q1.x, I);
                I = __dp4a((int)wv[k][5], q1.y, I);
                I = __dp4a((int)wv[k][6], q1.z, I);
                I = __dp4a((int)wv[k][7], q1.w, I);
                acc = fmaf(__fmul_rn(dl[k], __ldg(xq.d + (uint64_t)r * ng + g)), (float)I, acc);
            }
        }
        acc = q4b_warp_sum(acc);
        if (lane == 0) dst[(uint64_t)r * ld_dst + wrow] = acc;
    }
}

bool launch_grouped4(uint32_t type, const uint8_t *w, uint64_t expert_stride, const int32_t *act,
                     const uint32_t *n_act, uint32_t n_entries, const int32_t *bounds, Q8View xq, uint32_t cols,
                     uint32_t w_rows, float *dst, uint64_t ld_dst) {
    const dim3 grid((w_rows + 7u) / 8u, n_entries);
    if (type == Q4_T_IQ4_NL)
        grouped_rows4_k<Q4_T_IQ4_NL><<<grid, 256, 0, g_q4b.stream>>>(w, expert_stride, act, n_act, bounds, xq, cols,
                                                                    w_rows, dst, ld_dst);
    else
        grouped_rows4_k<Q4_T_IQ4_XS><<<grid, 256, 0, g_q4b.stream>>>(w, expert_stride, act, n_act, bounds, xq, cols,
                                                                    w_rows, dst, ld_dst);
    g_q4b_launches++;
    return q4b_launch_ok("grouped_rows4");
}

bool launch_grouped(const uint8_t *w, uint64_t expert_stride, const int32_t *act,
                    const uint32_t *n_act, uint32_t n_entries, const int32_t *bounds, Q8View xq,
                    uint32_t cols, uint32_t w_rows, float *dst, uint64_t ld_dst) {
    const uint32_t B = cols >> 8;
    const uint32_t n_tiles = (w_rows * B) >> 3;
    // eight tiles per warp (64 per CTA) where the matrix has that many: the code table and
    // the CTA start-up are paid once per 56 KB of weights
    const uint32_t ctas = (n_tiles + 7u) / 8u;
    const dim3 grid(ctas > 8u ? (ctas + 7u) / 8u : 1u, n_entries);
    if (q4b_ptr_tiled(w))
        grouped_rows_k<true><<<grid, 256, 0, g_q4b.stream>>>(w, expert_stride, act, n_act, bounds, xq,
                                                            cols, w_rows, dst, ld_dst, g_q4b.codes_d);
    else
        grouped_rows_k<false><<<grid, 256, 0, g_q4b.stream>>>(w, expert_stride, act, n_act, bounds, xq,
                                                             cols, w_rows, dst, ld_dst, g_q4b.codes_d);
    g_q4b_launches++;
    return q4b_launch_ok("grouped_rows");
}

// Which grouped product runs.  The tensor-core kernel pays off once an expert has
// enough rows to fill a useful part of a 128 x 64 MMA tile; below that the streaming
// CUDA-core kernel (one decode, a handful of dot products from registers) is the
// better fit, and the general CUDA-core kernel takes what neither accepts (arenas in
// the engine's byte order, odd widths).  In the default mode a call is split by
// entry: entries with TC_MIN_ROWS rows or more go to the tensor cores, the rest to
// the streaming kernel; each kernel skips the other's entries.
int g_tc_mode = -1;  // -1 split by rows, 0 CUDA cores only, 1 tensor cores whenever the shape
                     // allows, 2 the general CUDA-core kernel only
// An entry goes to the tensor cores from 12 rows: beyond the three rows it keeps in registers the
// streaming kernel re-fetches the activation rows for every tile, which costs more than the
// tensor-core kernel's fixed work per tile.  Measured (48 layers of 64 tokens / 48 layers of 4
// tokens / one layer of 2048 tokens): split at 12: 18.7 / 3.53 / 1.19 ms, at 8: 18.7 / 3.53 /
// 1.17, at 4: 18.9 / 5.50 / 1.16 (a 4-token window's shared expert, weights cold, is the
// streaming kernel's case), everything streamed: 33 ms for the first.  At 8 the shared expert of
// an 8-way expert-parallel rank (8 own tokens, weights cold) moves to the tensor cores with its
// four helper launches per layer: 9.3 ms per step against 7.8 ms with the split at 12.
constexpr uint32_t TC_MIN_ROWS = 12;
bool launch_grouped_any(const uint8_t *w, uint64_t expert_stride, const int32_t *act,
                        const uint32_t *n_act, uint32_t n_entries, const int32_t *bounds, Q8View xq,
                        uint64_t total_rows, uint32_t cols, uint32_t w_rows, float *dst,
                        uint64_t ld_dst, uint64_t max_rows_hint, uint32_t type = Q4_T_IQ3_S) {
    if (type != Q4_T_IQ3_S)   // IQ4_NL / IQ4_XS: one CUDA-core kernel, engine byte order only
        return !q4b_ptr_tiled(w) &&
               launch_grouped4(type, w, expert_stride, act, n_act, n_entries, bounds, xq, cols, w_rows, dst, ld_dst);
    // max_rows_hint: the caller's bound on the rows of its largest entry (0 = unknown).  When
    // it says no entry reaches the tensor-core threshold that kernel is not launched at all;
    // should an entry exceed the hint anyway, the streaming kernel still takes it.
    if (max_rows_hint == 0 || max_rows_hint > total_rows) max_rows_hint = total_rows;
    const bool tiled = q4b_ptr_tiled(w);
    const bool tc_ok = g_tc_mode != 0 && g_tc_mode != 2 && mmqtc::g_ready && mmqtc::shape_ok(w_rows, cols);
    const bool few_ok = g_tc_mode != 2 && g_tc_mode != 1 && tiled && few::shape_ok(w_rows, cols, n_entries);
    // rows an entry needs before the tensor cores take it
    uint32_t tc_min = 0xffffffffu;
    // a prefill-sized call (thousands of rows): the tensor-core kernel is running anyway and takes
    // entries from 6 rows (2048 tokens: 1.083 ms against 1.097 at 12, 1.086 at 4 and at 8)
    const uint32_t split_rows = total_rows >= 4096u ? 6u : TC_MIN_ROWS;
    if (tc_ok) tc_min = g_tc_mode == 1 ? 1u : (few_ok ? split_rows : 0xffffffffu);
    if (tc_ok && g_tc_mode == -1 && !few_ok && total_rows >= 8ull * n_entries) tc_min = 1u;
    const bool run_tc = tc_min != 0xffffffffu && max_rows_hint >= tc_min;
    // When a call is split, the two kernels touch disjoint entries and rows: the tensor-core
    // kernel goes to a side stream forked off the compute stream and joined after the streaming
    // kernel, so a handful of many-row experts (a decode batch's shared expert) does not cost a
    // launch of its own length; the streaming kernel's CTAs on the SMs the other kernel holds
    // simply start a little later.
    const bool side = run_tc && tc_min > 1u && few_ok;
    if (run_tc) {
        cudaStream_t st = g_q4b.stream;
        if (side) {
            if (cudaEventRecord(g_q4b.ev_fork, g_q4b.stream) != cudaSuccess ||
                cudaStreamWaitEvent(g_q4b.aux_stream, g_q4b.ev_fork, 0) != cudaSuccess)
                return false;
            st = g_q4b.aux_stream;
        }
        const bool ok = mmqtc::launch(w, expert_stride, act, n_act, n_entries, bounds, xq.q, xq.d, xq.h1, xq.h2, xq.rs,
                                      total_rows, cols, w_rows, dst, ld_dst, tiled, tc_min, st);
        g_q4b_launches++;
        if (!ok || !q4b_launch_ok("mmq_tc")) return false;
        if (tc_min <= 1u) return true;
    }
    if (few_ok) {
        few::Args a;
        a.w = w;
        a.expert_stride = expert_stride;
        a.act = act;
        a.n_act = n_act;
        a.n_entries = n_entries;
        a.bounds = bounds;
        a.xq = xq.q;
        a.xd = xq.d;
        a.xbs = xq.bs;
        a.cols = cols;
        a.w_rows = w_rows;
        a.dst = dst;
        a.ld_dst = ld_dst;
        a.codes = g_q4b.codes_d;
        a.err = g_q4b.err_d;
        a.max_rows = run_tc ? tc_min - 1u : 0x7fffffffu;
        const bool ok = few::launch(a);
        g_q4b_launches++;
        if (!ok || !q4b_launch_ok("grouped_few")) return false;
        if (side && (cudaEventRecord(g_q4b.ev_join, g_q4b.aux_stream) != cudaSuccess ||
                     cudaStreamWaitEvent(g_q4b.stream, g_q4b.ev_join, 0) != cudaSuccess))
            return false;
        return true;
    }
    return launch_grouped(w, expert_stride, act, n_act, n_entries, bounds, xq, cols, w_rows, dst, ld_dst);
}

// bytes of one weight row of a type the grouped products take
uint64_t row_bytes_t(uint32_t type, uint64_t cols) {
    return type == Q4_T_IQ3_S ? (cols / 256u) * Q4B_IQ3S_BYTES : iq4_row_bytes(type, cols);
}
bool pow2_blocks(uint64_t w_cols) {
    const uint64_t B = w_cols / 256u;
    return B == 1 || B == 2 || B == 4 || B == 8;
}

bool shape_ok(uint32_t type, uint64_t w_rows, uint64_t w_cols) {
    if (type == Q4_T_IQ4_NL || type == Q4_T_IQ4_XS)
        return w_rows != 0 && w_cols != 0 && w_cols <= 4096u && (w_cols % (type == Q4_T_IQ4_NL ? 32u : 256u)) == 0;
    if (type != Q4_T_IQ3_S || w_rows == 0 || w_cols == 0 || (w_cols % 256u)) return false;
    const uint64_t B = w_cols / 256u;
    return ((w_rows * B) % 8u) == 0;
}

}  // namespace grouped

using namespace grouped;

// shared memory of assign_k with 32 warps and 1024 experts; the limit is raised once, at warm-up
constexpr size_t ASSIGN_SMEM_MAX = (34u * 1024u + 48u) * sizeof(uint32_t);
bool q4b_mmq_tc_warm() {
    if (cudaFuncSetAttribute(assign_k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ASSIGN_SMEM_MAX) !=
        cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    const bool f = few::warm();
    return mmqtc::warm() && f;
}
extern "C" bool q4_cuda_mmq_tc_mode(int mode) {
    if (mode < -1 || mode > 2 || (mode == 1 && !mmqtc::g_ready)) return false;
    grouped::g_tc_mode = mode;
    return true;
}
extern "C" int q4_mmq_on(void) { return g_q4b.ok ? 1 : 0; }
extern "C" uint32_t q4_mmq_group(void) { return 4096u; }
extern "C" bool q4_mmq_supported(uint32_t type, uint64_t w_rows) {
    if (!g_q4b.ok || w_rows == 0) return false;
    if (type == Q4_T_IQ4_NL || type == Q4_T_IQ4_XS) return true;   // weights in the engine's byte order
    return type == Q4_T_IQ3_S && (w_rows % 8u) == 0;
}
extern "C" uint64_t q4_mmq_q8_bytes(uint64_t rows, uint64_t cols) { return q8_bytes(rows, cols); }
extern "C" uint64_t q4_mmq_pad(uint64_t row_bytes) {
    (void)row_bytes;
    return 0;  // the kernels here never read past a matrix: no zero pad is needed
}

extern "C" bool q4_mmq_quantize(const float *x, const int32_t *ids, void *xq, uint32_t w_type,
                                uint64_t cols, uint64_t rows) {
    if (!g_q4b.ok || !x || !xq || rows == 0 || cols == 0 || (cols % 32u)) return false;
    if (w_type != Q4_T_IQ3_S && w_type != Q4_T_IQ4_NL && w_type != Q4_T_IQ4_XS) return false;
    const Q8View v = q8_view(xq, rows, cols);
    const uint64_t ngr = rows * (cols / 32u);
    if (g_q8_compat)
        quantize_rows_k<true><<<(unsigned)((ngr * 4 + 255) / 256), 256, 0, g_q4b.stream>>>(
            x, ids, cols, rows, (int8_t *)v.q, (float *)v.d, (int32_t *)v.bs);
    else
        quantize_rows_k<false><<<(unsigned)((ngr * 4 + 255) / 256), 256, 0, g_q4b.stream>>>(
            x, ids, cols, rows, (int8_t *)v.q, (float *)v.d, (int32_t *)v.bs);
    g_q4b_launches++;
    return q4b_launch_ok("quantize_rows");
}

extern "C" bool q4_mmq_mul_id(const void *w, uint32_t type, uint64_t w_rows, uint64_t w_cols,
                              uint64_t expert_stride_bytes, uint32_t n_expert, const void *xq,
                              const int32_t *bounds, uint32_t max_rows, uint64_t total_rows,
                              float *dst, uint64_t ld_dst) {
    if (!g_q4b.ok || !w || !xq || !bounds || !dst || n_expert == 0 || total_rows == 0) return false;
    if (!grouped::shape_ok(type, w_rows, w_cols) || ld_dst < w_rows) return false;
    if (type != Q4_T_IQ3_S && q4b_ptr_tiled(w)) return false;
    if (type == Q4_T_IQ3_S && !grouped::pow2_blocks(w_cols) &&
        cudaMemsetAsync(dst, 0, total_rows * ld_dst * sizeof(float), g_q4b.stream) != cudaSuccess)
        return false;
    return launch_grouped_any((const uint8_t *)w, expert_stride_bytes, nullptr, nullptr, n_expert, bounds,
                              q8_view(xq, total_rows, w_cols), total_rows, (uint32_t)w_cols,
                              (uint32_t)w_rows, dst, ld_dst, max_rows, type);
}

extern "C" bool q4_mmq_swiglu(const float *gu, float *h, uint64_t rows, uint64_t n_ff) {
    if (!g_q4b.ok || !gu || !h || rows == 0 || n_ff == 0) return false;
    const uint64_t n = rows * n_ff;
    swiglu_rows_k<<<(unsigned)((n + 255) / 256), 256, 0, g_q4b.stream>>>(gu, h, rows, n_ff);
    g_q4b_launches++;
    return q4b_launch_ok("swiglu_rows");
}

extern "C" bool q4_hip_expert_reduce(float *d_y, const float *d_pd, const int32_t *d_rsrc,
                                     const float *d_rw, uint32_t n_tok, uint32_t topk,
                                     uint32_t n_embd) {
    if (!g_q4b.ok || !d_y || !d_pd || !d_rsrc || !d_rw || !n_tok || !topk || !n_embd) return false;
    launch_expert_reduce<true>(d_y, d_pd, d_rsrc, d_rw, n_tok, topk, n_embd);
    g_q4b_launches++;
    return q4b_launch_ok("expert_reduce");
}
extern "C" bool q4_cuda_expert_reduce_set(float *d_y, const float *d_pd, const int32_t *d_rsrc,
                                          const float *d_rw, uint32_t n_tok, uint32_t topk,
                                          uint32_t n_embd) {
    if (!g_q4b.ok || !d_y || !d_pd || !d_rsrc || !d_rw || !n_tok || !topk || !n_embd) return false;
    launch_expert_reduce<false>(d_y, d_pd, d_rsrc, d_rw, n_tok, topk, n_embd);
    g_q4b_launches++;
    return q4b_launch_ok("expert_reduce_set");
}
extern "C" bool q4_cuda_mmq_swiglu_quantize(const float *gu, void *hq, uint64_t rows, uint64_t n_ff) {
    if (!g_q4b.ok || !gu || !hq || rows == 0 || n_ff == 0 || (n_ff % 32u)) return false;
    const Q8View v = q8_view(hq, rows, n_ff);
    const uint64_t ngr = rows * (n_ff / 32u);
    if (g_q8_compat)
        swiglu_quant_rows_k<true><<<(unsigned)((ngr * 4 + 255) / 256), 256, 0, g_q4b.stream>>>(
            gu, rows, n_ff, (int8_t *)v.q, (float *)v.d, (int32_t *)v.bs);
    else
        swiglu_quant_rows_k<false><<<(unsigned)((ngr * 4 + 255) / 256), 256, 0, g_q4b.stream>>>(
            gu, rows, n_ff, (int8_t *)v.q, (float *)v.d, (int32_t *)v.bs);
    g_q4b_launches++;
    return q4b_launch_ok("swiglu_quantize");
}

// Which quantiser the row buffers of the many-token sequence are filled with (q4_mmq_quantize,
// q4_cuda_mmq_swiglu_quantize, and through them q4_cuda_moe_layer_n): 0 = Q8-A (default), 1 = Q8-C,
// ggml's q8_1 rounding, for bit-level comparisons with the reference's grouped device product.
extern "C" void q4_cuda_mmq_q8_compat(int on) { g_q8_compat = on ? 1 : 0; }
// The sections of a row buffer (device pointers into xq): int8 q [rows][cols], float d and int32
// sums [rows][cols / 32].  For stage tests.
extern "C" bool q4_cuda_mmq_q8_sections(const void *xq, uint64_t rows, uint64_t cols, const int8_t **q,
                                        const float **d, const int32_t **sums) {
    if (!xq || !rows || !cols || (cols % 32u)) return false;
    const Q8View v = q8_view(xq, rows, cols);
    if (q) *q = v.q;
    if (d) *d = v.d;
    if (sums) *sums = v.bs;
    return true;
}

extern "C" bool q4_hip_route_pf(const float *d_rlog, int32_t *d_ids, float *d_wts, uint32_t n_tok,
                                uint32_t n_exp, uint32_t topk) {
    if (!g_q4b.ok || !d_rlog || !d_ids || !d_wts || !n_tok || n_exp == 0 || n_exp > 1024u || !topk ||
        topk > 64u)
        return false;
    return q4b_route_tokens(d_rlog, d_ids, d_wts, n_tok, n_exp, topk);
}

static bool launch_assign(const int32_t *d_ids, const float *d_wts, int32_t *d_atok, int32_t *d_rsrc,
                          float *d_rw, int32_t *d_stg, uint32_t *d_stgn, uint32_t *d_ek,
                          int32_t *d_cbounds, uint32_t gsz, uint32_t topk, uint32_t n_exp,
                          uint32_t n_tok, uint32_t ek_stride, uint32_t topk_in = 0,
                          int32_t extra_id = -1, int32_t own_first = 0, uint32_t own_count = 0,
                          uint32_t tok_first = 0, uint32_t tok_count = 0, int32_t *d_bounds_full = nullptr) {
    const uint32_t n_g = (n_tok + gsz - 1u) / gsz;
    // a large group gets 32 warps (a histogram per warp: up to 34 x n_exp words of shared memory)
    const uint64_t rows = (uint64_t)(gsz < n_tok ? gsz : n_tok) * topk;
    const uint32_t nt = rows > 4096u ? 1024u : 256u;
    const size_t sm = ((nt / 32u + 2u) * n_exp + 48u) * sizeof(uint32_t);
    if (sm > ASSIGN_SMEM_MAX) return false;
    assign_k<<<n_g, nt, sm, g_q4b.stream>>>(
        d_ids, d_wts, d_atok, d_rsrc, d_rw, d_stg, d_stgn, d_ek, d_cbounds, gsz, topk, n_exp, n_tok,
        ek_stride, topk_in ? topk_in : topk, extra_id, own_first, own_count, tok_first, tok_count,
        d_bounds_full);
    g_q4b_launches++;
    return q4b_launch_ok("assign");
}

extern "C" bool q4_hip_assign_pf(const int32_t *d_ids, const float *d_wts, int32_t *d_atok,
                                 int32_t *d_rsrc, float *d_rw, int32_t *d_stg, uint32_t *d_stgn,
                                 uint32_t *d_ek, uint32_t gsz, uint32_t topk, uint32_t n_exp,
                                 uint32_t n_tok) {
    if (!g_q4b.ok || !d_ids || !d_wts || !d_atok || !d_rsrc || !d_rw || !d_stg || !d_stgn || !d_ek ||
        !n_tok || !gsz || !topk || n_exp == 0 || n_exp > 512u || topk > 64u)
        return false;
    // tables are 512 entries per group, as in the reference (src/q4_rocm.cu:6545-6548)
    return launch_assign(d_ids, d_wts, d_atok, d_rsrc, d_rw, d_stg, d_stgn, d_ek, nullptr, gsz, topk,
                         n_exp, n_tok, 512u);
}

// Assignment for one rank of an expert-parallel layer: all n_tok tokens' picks (d_ids/d_wts,
// [n_tok][topk], global expert ids) -> rows of the experts this rank owns, renumbered from 0,
// plus (has_shared) one pick of local expert own_count, weight 1, for tokens [tok_first,
// tok_first + tok_count).  Outputs as q4_hip_assign_pf with topk + has_shared columns, one
// group; d_bounds receives own_count + has_shared + 1 row bounds.
extern "C" bool q4_cuda_assign_local(const int32_t *d_ids, const float *d_wts, int32_t *d_atok,
                                     int32_t *d_rsrc, float *d_rw, int32_t *d_bounds, uint32_t n_tok,
                                     uint32_t topk, uint32_t own_first, uint32_t own_count,
                                     int has_shared, uint32_t tok_first, uint32_t tok_count) {
    if (!g_q4b.ok || !d_ids || !d_wts || !d_atok || !d_rsrc || !d_rw || !d_bounds || !n_tok || !topk ||
        own_count == 0 || own_count + (has_shared ? 1u : 0u) > 1023u || topk > 63u)
        return false;
    const uint32_t k1 = topk + (has_shared ? 1u : 0u), n_e = own_count + (has_shared ? 1u : 0u);
    return launch_assign(d_ids, d_wts, d_atok, d_rsrc, d_rw, nullptr, nullptr, nullptr, nullptr, n_tok, k1,
                         n_e, n_tok, n_e, topk, has_shared ? (int32_t)own_count : -1, (int32_t)own_first,
                         own_count, tok_first, tok_count, d_bounds);
}

// ---- the whole layer for n_tok tokens ----
// Workspace carve-up (all sections 256-byte aligned).
namespace {
struct LayerWs {
    float *xn, *logits, *wts, *wts2, *rw, *gu, *h, *pd;
    int32_t *ids, *ids2, *atok, *rsrc, *cbounds, *stg;
    uint32_t *stgn;
    void *xq, *hq;
    uint64_t bytes;
};
LayerWs carve(uint8_t *p, uint32_t n_tok, uint32_t topk, uint32_t n_expert, uint32_t n_embd,
              uint32_t n_ff) {
    LayerWs w;
    uint64_t off = 0;
    const uint64_t k1 = topk + 1u, rows = (uint64_t)n_tok * k1;
    auto take = [&](uint64_t n) {
        uint8_t *r = p ? p + off : nullptr;
        off += align256(n);
        return r;
    };
    w.xn = (float *)take((uint64_t)n_tok * n_embd * 4);
    w.logits = (float *)take((uint64_t)n_tok * n_expert * 4);
    w.ids = (int32_t *)take((uint64_t)n_tok * topk * 4);
    w.wts = (float *)take((uint64_t)n_tok * topk * 4);
    w.ids2 = (int32_t *)take(rows * 4);
    w.wts2 = (float *)take(rows * 4);
    w.atok = (int32_t *)take(rows * 4);
    w.rsrc = (int32_t *)take(rows * 4);
    w.rw = (float *)take(rows * 4);
    w.cbounds = (int32_t *)take((uint64_t)(n_expert + 3) * 4);
    w.stg = (int32_t *)take((uint64_t)(n_expert + 2) * 4);
    w.stgn = (uint32_t *)take(256);
    w.xq = take(q8_bytes(rows, n_embd));
    w.gu = (float *)take(rows * 2 * n_ff * 4);
    w.h = (float *)take(rows * n_ff * 4);
    w.hq = take(q8_bytes(rows, n_ff));
    w.pd = (float *)take(rows * n_embd * 4);
    w.bytes = off;
    return w;
}
}  // namespace

extern "C" uint64_t q4_cuda_moe_layer_n_ws_bytes(uint32_t n_tok, uint32_t topk, uint32_t n_expert,
                                                 uint32_t n_embd, uint32_t n_ff) {
    return carve(nullptr, n_tok, topk, n_expert, n_embd, n_ff).bytes;
}

extern "C" bool q4_cuda_moe_layer_n(const uint8_t *base, uint64_t stride, uint64_t og, uint64_t ou,
                                    uint64_t od, int32_t shared_slot, const float *d_x,
                                    const float *d_norm_w, float eps, const float *d_router,
                                    uint32_t n_expert, uint32_t topk, uint32_t n_embd,
                                    uint32_t n_ff, uint32_t n_tok, float *d_y, int32_t *d_ids,
                                    float *d_wts, void *d_ws, uint64_t ws_bytes) {
    return q4_cuda_moe_layer_nt(base, stride, Q4_T_IQ3_S, og, ou, Q4_T_IQ3_S, od, shared_slot, d_x, d_norm_w, eps,
                                d_router, n_expert, topk, n_embd, n_ff, n_tok, d_y, d_ids, d_wts, d_ws, ws_bytes);
}

// RMSNorm, router product and softmax / top-k of up to 256 tokens in one launch (n_embd == 2048): the
// values of q4_hip_grouped_rms_n + q4_hip_gemv_dd_n + q4_hip_route_pf, bit for bit.  false: not this
// kernel's shape, nothing queued.
extern "C" bool q4_cuda_route_small(const float *d_x, const float *d_norm_w, float eps, const float *d_router,
                                    uint32_t n_expert, uint32_t topk, uint32_t n_embd, uint32_t n_tok, float *d_xn,
                                    float *d_logits, int32_t *d_ids, float *d_wts) {
    if (!g_q4b.ok || !d_x || !d_router || !d_xn || !d_logits || !d_ids || !d_wts || topk == 0 || topk > n_expert)
        return false;
    return q4b_route_small(d_x, d_norm_w, eps, d_router, n_expert, topk, n_embd, n_tok, d_xn, d_logits, d_ids, d_wts);
}

// The same with the experts' formats named: gate and up of type gt, down of type dt, each IQ3_S,
// IQ4_NL or IQ4_XS (a pack with a part that is not IQ3_S sits in an arena in the engine's byte order).
extern "C" bool q4_cuda_moe_layer_nt(const uint8_t *base, uint64_t stride, uint32_t gt, uint64_t og, uint64_t ou,
                                     uint32_t dt, uint64_t od, int32_t shared_slot, const float *d_x,
                                     const float *d_norm_w, float eps, const float *d_router,
                                     uint32_t n_expert, uint32_t topk, uint32_t n_embd, uint32_t n_ff,
                                     uint32_t n_tok, float *d_y, int32_t *d_ids, float *d_wts, void *d_ws,
                                     uint64_t ws_bytes) {
    if (!g_q4b.ok || !base || !d_x || !d_router || !d_y || !d_ws || n_tok == 0) return false;
    if (n_expert == 0 || n_expert >= 1024u || topk == 0 || topk > 63u || topk > n_expert) return false;
    if (!grouped::shape_ok(gt, 2ull * n_ff, n_embd) || !grouped::shape_ok(dt, n_embd, n_ff)) return false;
    if ((gt != Q4_T_IQ3_S || dt != Q4_T_IQ3_S) && q4b_ptr_tiled(base)) return false;
    if (ou != og + (uint64_t)n_ff * grouped::row_bytes_t(gt, n_embd)) return false;  // gate|up contiguous
    if (shared_slot >= 0 && (uint32_t)shared_slot != n_expert) return false;  // shared = slot n_expert
    const LayerWs w = carve((uint8_t *)d_ws, n_tok, topk, n_expert, n_embd, n_ff);
    if (ws_bytes < w.bytes) return false;
    cudaStream_t st = g_q4b.stream;
    const bool sh = shared_slot >= 0;
    const uint32_t k1 = topk + (sh ? 1u : 0u), n_e = n_expert + (sh ? 1u : 0u);
    const uint64_t rows = (uint64_t)n_tok * k1;
    const uint32_t n_entries = (uint32_t)(rows < n_e ? rows : n_e);  // used experts <= rows
    // up to 256 tokens: norm, router and top-k as one launch (same values); else the three launches
    if (!q4b_route_small(d_x, d_norm_w, eps, d_router, n_expert, topk, n_embd, n_tok, w.xn, w.logits, w.ids,
                         w.wts)) {
        if (!q4b_rms_rows(d_x, d_norm_w, w.xn, n_embd, eps, n_tok)) return false;
        if (!q4_hip_gemv_dd_n(Q4_T_F32, (const uint8_t *)d_router, n_expert, n_embd, w.xn, w.logits, 1.0f,
                              n_tok))
            return false;
        if (!q4b_route_tokens(w.logits, w.ids, w.wts, n_tok, n_expert, topk)) return false;
    }
    // the shared expert is one more pick (id n_expert, weight 1) of every token, added on the fly
    if (!launch_assign(w.ids, w.wts, w.atok, w.rsrc, w.rw, w.stg, w.stgn, nullptr, w.cbounds, n_tok, k1,
                       n_e, n_tok, n_e, topk, sh ? (int32_t)n_expert : -1))
        return false;
    if (!q4_mmq_quantize(w.xn, w.atok, w.xq, gt, n_embd, rows)) return false;
    if (gt == Q4_T_IQ3_S && !grouped::pow2_blocks(n_embd) &&
        cudaMemsetAsync(w.gu, 0, rows * 2 * n_ff * 4, st) != cudaSuccess)
        return false;
    if (!launch_grouped_any(base + og, stride, w.stg, w.stgn, n_entries, w.cbounds,
                            q8_view(w.xq, rows, n_embd), rows, n_embd, 2u * n_ff, w.gu, 2ull * n_ff,
                            n_tok, gt))
        return false;
    if (!q4_cuda_mmq_swiglu_quantize(w.gu, w.hq, rows, n_ff)) return false;
    if (dt == Q4_T_IQ3_S && !grouped::pow2_blocks(n_ff) &&
        cudaMemsetAsync(w.pd, 0, rows * n_embd * 4, st) != cudaSuccess)
        return false;
    if (!launch_grouped_any(base + od, stride, w.stg, w.stgn, n_entries, w.cbounds,
                            q8_view(w.hq, rows, n_ff), rows, n_ff, n_embd, w.pd, n_embd, n_tok, dt))
        return false;
    if (!q4_cuda_expert_reduce_set(d_y, w.pd, w.rsrc, w.rw, n_tok, k1, n_embd)) return false;
    if (d_ids && cudaMemcpyAsync(d_ids, w.ids, (uint64_t)n_tok * topk * 4, cudaMemcpyDeviceToDevice, st) !=
                     cudaSuccess)
        return false;
    if (d_wts && cudaMemcpyAsync(d_wts, w.wts, (uint64_t)n_tok * topk * 4, cudaMemcpyDeviceToDevice, st) !=
                     cudaSuccess)
        return false;
    return true;
}

// ---- verify window (2..8 tokens), reference entry point ----
extern "C" bool q4_hip_moe_win_ok(uint32_t gt, uint32_t ut, uint32_t dt, uint32_t in_dim,
                                  uint32_t n_ff, uint32_t n_tok) {
    // gate and up of one type, down of any; each IQ3_S, IQ4_NL or IQ4_XS (src/q4_rocm.cu:4926-4944
    // takes more formats; the others answer false here and the engine keeps its own path)
    return g_q4b.ok && gt == ut && n_tok >= 2 && n_tok <= 8 && in_dim <= 16384u && n_ff <= 4096u &&
           grouped::shape_ok(gt, n_ff, in_dim) && grouped::shape_ok(dt, in_dim, n_ff);
}

// Library-owned scratch of the window path (allocated by init / scratch_warm):
// 8 tokens x 64 picks, rows up to 16384 wide, hidden rows up to 4096.
static uint8_t *g_win_ws = nullptr;
static uint64_t g_win_ws_bytes = 0;
bool q4b_window_warm() {
    if (g_win_ws) return true;
    const uint64_t rows = 512;
    g_win_ws_bytes = 8 * align256(rows * 4) + align256(514 * 4) + q8_bytes(rows, 16384) +
                     align256(rows * 2 * 4096 * 4) + align256(rows * 4096 * 4) + q8_bytes(rows, 4096) +
                     align256(rows * 16384 * 4) + 4096;
    if (cudaMalloc(&g_win_ws, g_win_ws_bytes) != cudaSuccess) {
        cudaGetLastError();
        g_win_ws = nullptr;
        return false;
    }
    return true;
}

extern "C" bool q4_hip_moe_exec_win(const uint8_t *base, uint64_t stride, const int32_t *d_es,
                                    const float *d_ew, const int32_t *d_nh, uint32_t n_tok,
                                    uint32_t gt, uint64_t og, uint32_t ut, uint64_t ou, uint32_t dt,
                                    uint64_t od, const float *d_x, float *d_h, float *d_y,
                                    uint32_t n_ff, uint32_t in_dim, uint32_t n_embd) {
    (void)d_h;
    if (!g_q4b.ok || !base || !d_es || !d_ew || !d_nh || !d_x || !d_y) return false;
    if (!q4_hip_moe_win_ok(gt, ut, dt, in_dim, n_ff, n_tok) || n_embd > 16384u ||
        !grouped::shape_ok(dt, n_embd, n_ff))
        return false;
    if ((gt != Q4_T_IQ3_S || dt != Q4_T_IQ3_S) && q4b_ptr_tiled(base)) return false;
    if (!q4b_window_warm()) return false;
    cudaStream_t st = g_q4b.stream;
    const uint64_t rows = 512;  // 8 tokens x 64 picks; only the placed rows are touched
    uint8_t *p = g_win_ws;
    auto take = [&](uint64_t n) {
        uint8_t *r = p;
        p += align256(n);
        return r;
    };
    int32_t *act = (int32_t *)take(rows * 4);
    uint32_t *n_act = (uint32_t *)take(256);
    int32_t *atok = (int32_t *)take(rows * 4);
    int32_t *rsrc = (int32_t *)take(rows * 4);
    float *rw = (float *)take(rows * 4);
    int32_t *bounds = (int32_t *)take(514 * 4);
    void *xq = take(q8_bytes(rows, in_dim));
    float *gu = (float *)take(rows * 2 * n_ff * 4);
    float *h = (float *)take(rows * n_ff * 4);
    void *hq = take(q8_bytes(rows, n_ff));
    float *pd = (float *)take(rows * n_embd * 4);
    if ((uint64_t)(p - g_win_ws) > g_win_ws_bytes) return false;
    if (cudaMemsetAsync(atok, 0xff, rows * 4, st) != cudaSuccess) return false;  // -1: unplaced rows
    win_assign_k<<<1, 512, 0, st>>>(d_es, d_ew, d_nh, n_tok, act, n_act, bounds, atok, rsrc, rw);
    g_q4b_launches++;
    if (!q4b_launch_ok("win_assign")) return false;
    const uint32_t n_pairs = n_tok * 64u;
    if (!q4_mmq_quantize(d_x, atok, xq, gt, in_dim, n_pairs)) return false;
    const Q8View xv = q8_view(xq, n_pairs, in_dim);
    if (gt == Q4_T_IQ3_S && !grouped::pow2_blocks(in_dim) &&
        cudaMemsetAsync(gu, 0, (uint64_t)n_pairs * 2 * n_ff * 4, st) != cudaSuccess)
        return false;
    if (dt == Q4_T_IQ3_S && !grouped::pow2_blocks(n_ff) &&
        cudaMemsetAsync(pd, 0, (uint64_t)n_pairs * n_embd * 4, st) != cudaSuccess)
        return false;
    if (ou == og + (uint64_t)n_ff * grouped::row_bytes_t(gt, in_dim)) {
        if (!launch_grouped_any(base + og, stride, act, n_act, n_pairs, bounds, xv, n_pairs, in_dim,
                                2u * n_ff, gu, 2ull * n_ff, n_tok, gt))
            return false;
    } else if (!launch_grouped_any(base + og, stride, act, n_act, n_pairs, bounds, xv, n_pairs, in_dim, n_ff,
                                   gu, 2ull * n_ff, n_tok, gt) ||
               !launch_grouped_any(base + ou, stride, act, n_act, n_pairs, bounds, xv, n_pairs, in_dim, n_ff,
                                   gu + n_ff, 2ull * n_ff, n_tok, gt)) {
        return false;
    }
    if (!q4_mmq_swiglu(gu, h, n_pairs, n_ff)) return false;
    if (!q4_mmq_quantize(h, nullptr, hq, dt, n_ff, n_pairs)) return false;
    if (!launch_grouped_any(base + od, stride, act, n_act, n_pairs, bounds, q8_view(hq, n_pairs, n_ff),
                            n_pairs, n_ff, n_embd, pd, n_embd, n_tok, dt))
        return false;
    return q4_hip_expert_reduce(d_y, pd, rsrc, rw, n_tok, 64u, n_embd);
}
