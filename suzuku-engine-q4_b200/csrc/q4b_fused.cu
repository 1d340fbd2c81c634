// One MoE layer for one token as ONE persistent kernel (one CTA per SM):
//
//   phase 0  every CTA: RMSNorm of x, Q8-A quantisation, code table -> shared memory
//   phase 1  router: the CTAs split the fp32 router matrix into 2 KB chunks,
//            fetched with bulk async copies issued at kernel start
//            -- grid barrier --
//   phase 2  every CTA: softmax + top-k (redundantly, from the 512 logits);
//            gate/up rows of the picked experts and the shared expert, split
//            evenly over the CTAs as (expert, hidden unit) pairs; the CTA's
//            down-projection tiles are fetched meanwhile
//            -- grid barrier --
//   phase 3  every CTA: Q8-A of the hidden rows, down tiles x hq, weighted sum
//            over the experts in list order, y written
//
// Weight bytes cross HBM -> shared memory exactly once, by 1-D bulk async
// copies (cp.async.bulk, no multicast) that complete on mbarriers; nothing is
// re-read.  Replaces the reference's per-layer launch chain
// (src/q4_moe.c:2077-2133; kernels wmoe_iq3_gu_q8 / wmoe_iq3_ya_q8,
// src/q4_rocm.cu:3912-4120).  Needs the tiled arena format (q4b_tile.cuh),
// n_embd == 2048 and n_ff == 512.
#include "q4b_tile.cuh"

#include <atomic>

#include "../../include/q4cuda.h"

extern std::atomic<uint64_t> g_q4b_launches;
bool q4b_ptr_tiled(const void *p);

namespace fused {

constexpr uint32_t NT = 512;          // threads per CTA
constexpr uint32_t NW = NT / 32;      // warps
constexpr uint32_t H = 2048;          // n_embd
constexpr uint32_t F = 512;           // n_ff
constexpr uint32_t RCHUNK = 512;      // router chunk: 512 floats = 2 KB
constexpr uint32_t MAX_E = 40;        // experts per token incl. shared
constexpr uint32_t UCHUNK = 8;        // gate/up units per bulk-copy chunk
constexpr uint32_t MAX_CHUNKS = 12;
constexpr uint32_t WAIT_LIMIT = 1000000u;  // polls before a wait gives up

// error word bits
constexpr uint32_t ERR_MBAR = 1u, ERR_GRID = 2u, ERR_SHAPE = 4u;

struct Args {
    const uint8_t *base;
    uint64_t stride, og, ou, od;
    int32_t shared_slot;
    const float *x, *norm_w, *router;
    float eps;
    uint32_t n_expert, topk;
    float *y;
    int32_t *ids_out;
    float *wts_out;
    float *logit_part;            // [n_expert][H / RCHUNK]
    float *h;                     // [MAX_E][F]
    unsigned long long *bar;      // grid barrier counter
    uint32_t *err;
    // shared-memory carve-up (bytes from the 1024-aligned start)
    uint32_t off_stage, off_down, stage_bytes, down_bytes;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after WAIT_LIMIT polls and records it.
__device__ __forceinline__ void mbar_wait(uint64_t *bar, uint32_t parity, uint32_t *err) {
    for (uint32_t i = 0; i < WAIT_LIMIT; i++)
        if (mbar_try_wait(bar, parity)) return;
    atomicOr(err, ERR_MBAR);
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes,
                                         uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
            "r"(smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// All CTAs arrive; nobody leaves before the last one has.  The counter only
// grows: arrival number a belongs to barrier a / gridDim.x, so no reset is
// needed between barriers or launches.  Bounded: a CTA that waits too long
// records ERR_GRID and goes on (its results are then meaningless, but nothing
// hangs).
__device__ __forceinline__ void grid_barrier(unsigned long long *ctr, uint32_t *err) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned long long old = atomicAdd(ctr, 1ull);
        const unsigned long long target = (old / gridDim.x + 1ull) * gridDim.x;
        uint32_t i = 0;
        for (; i < WAIT_LIMIT; i++) {
            unsigned long long v;
            asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(ctr) : "memory");
            if (v >= target) break;
            __nanosleep(20);
        }
        if (i == WAIT_LIMIT) atomicOr(err, ERR_GRID);
        __threadfence();
    }
    __syncthreads();
}

__device__ __forceinline__ float block_reduce_max(float v, float *red) {
    v = q4b_warp_max(v);
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = red[0];
    for (uint32_t i = 1; i < NW; i++) r = fmaxf(r, red[i]);
    __syncthreads();
    return r;
}
__device__ __forceinline__ float block_reduce_sum(float v, float *red) {
    v = q4b_warp_sum(v);
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.f;
    for (uint32_t i = 0; i < NW; i++) r += red[i];
    __syncthreads();
    return r;
}

// Q8-A of 32 consecutive floats held four per lane by eight neighbouring lanes.
// Returns the packed int8x4 word; lane with (lane & 7) == 0 gets d and sum.
__device__ __forceinline__ uint32_t quant8_oct(float4 v, float *d_out, int *bs_out) {
    float a = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 2));
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 4));
    const float sc = a > 0.f ? __fdiv_rn(127.f, a) : 0.f;
    int q0 = max(-128, min(127, __float2int_rn(__fmul_rn(v.x, sc))));
    int q1 = max(-128, min(127, __float2int_rn(__fmul_rn(v.y, sc))));
    int q2 = max(-128, min(127, __float2int_rn(__fmul_rn(v.z, sc))));
    int q3 = max(-128, min(127, __float2int_rn(__fmul_rn(v.w, sc))));
    int s = q0 + q1 + q2 + q3;
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    *d_out = __fdiv_rn(a, 127.f);
    *bs_out = s;
    return (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) |
           ((uint32_t)(q3 & 0xff) << 24);
}

// Shared-memory layout (offsets from a 1024-byte aligned base):
//   [0, 65536)        code table, entry i replicated per lane: tab[32 i + lane]
//   [65536, +...)     small arrays (below), then the two staging regions
struct Small {
    uint64_t mbar[MAX_CHUNKS + 2];  // [0] router, [1..MAX_CHUNKS] gate/up chunks, [last] down
    alignas(16) float xn[H];        // normalised x (router input)
    alignas(16) uint32_t xq[H / 4];             // Q8-A of xn, int8x4 words
    float xd[H / 32];
    int xbs[H / 32];
    float p[1024];                  // softmax probabilities
    int32_t ids[MAX_E];
    float wts[MAX_E];
    float red[NW];
    double redd[NW];
    alignas(16) uint32_t hq[MAX_E][F / 4];  // Q8-A of the hidden rows
    float hd[MAX_E][F / 32];
    int hbs[MAX_E][F / 32];
    float part[64][4];              // phase-3 partial sums: [tile][row in tile]
};

__global__ void __launch_bounds__(NT, 1) moe_decode_fused_k(const Args a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *sm = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint32_t *tab = reinterpret_cast<uint32_t *>(sm);
    Small &S = *reinterpret_cast<Small *>(sm + 65536);
    uint8_t *stage = sm + a.off_stage;  // router chunks, then gate/up tiles
    uint8_t *dstage = sm + a.off_down;  // down tiles
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t cta = blockIdx.x, ncta = gridDim.x;
    const uint32_t ne = a.topk + (a.shared_slot >= 0 ? 1u : 0u);

    // ---- work split ----
    const uint32_t n_rchunks = a.n_expert * (H / RCHUNK);
    const uint32_t rc0 = (uint32_t)((uint64_t)cta * n_rchunks / ncta);
    const uint32_t rc1 = (uint32_t)((uint64_t)(cta + 1) * n_rchunks / ncta);
    const uint32_t n_units = ne * F;  // (expert, hidden unit) pairs
    const uint32_t u0 = (uint32_t)((uint64_t)cta * n_units / ncta);
    const uint32_t u1 = (uint32_t)((uint64_t)(cta + 1) * n_units / ncta);
    const uint32_t n_dtiles = (H / 4) * ne;  // (row quad, expert) pairs, expert fastest
    const uint32_t v0 = (uint32_t)((uint64_t)cta * n_dtiles / ncta);
    const uint32_t v1 = (uint32_t)((uint64_t)(cta + 1) * n_dtiles / ncta);

    if (tid == 0) {
        for (uint32_t i = 0; i < MAX_CHUNKS + 2; i++) mbar_init(&S.mbar[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // router chunks: contiguous in memory
    if (tid == 0 && rc1 > rc0) {
        const uint32_t bytes = (rc1 - rc0) * RCHUNK * 4u;
        mbar_expect_tx(&S.mbar[0], bytes);
        bulk_g2s(stage, a.router + (size_t)rc0 * RCHUNK, bytes, &S.mbar[0]);
    }

    // ---- phase 0: code table, y = 0, RMSNorm, Q8-A ----
    for (uint32_t i = 0; i < 32; i++) {
        const uint32_t idx = warp * 32u + i;
        tab[idx * 32u + lane] = q4b_code_bytes(c_iq3s_codes[idx]);
    }
    for (uint32_t r = cta * NT + tid; r < H; r += ncta * NT) a.y[r] = 0.f;
    {
        const float4 xv = reinterpret_cast<const float4 *>(a.x)[tid];
        double ss = (double)xv.x * xv.x + (double)xv.y * xv.y + (double)xv.z * xv.z +
                    (double)xv.w * xv.w;
#pragma unroll
        for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) S.redd[warp] = ss;
        __syncthreads();
        double tot = 0.0;
        for (uint32_t i = 0; i < NW; i++) tot += S.redd[i];
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn((float)(tot / (double)H), a.eps)));
        float4 v;
        v.x = __fmul_rn(xv.x, scale);
        v.y = __fmul_rn(xv.y, scale);
        v.z = __fmul_rn(xv.z, scale);
        v.w = __fmul_rn(xv.w, scale);
        if (a.norm_w) {
            const float4 wv = reinterpret_cast<const float4 *>(a.norm_w)[tid];
            v.x = __fmul_rn(v.x, wv.x);
            v.y = __fmul_rn(v.y, wv.y);
            v.z = __fmul_rn(v.z, wv.z);
            v.w = __fmul_rn(v.w, wv.w);
        }
        reinterpret_cast<float4 *>(S.xn)[tid] = v;
        float d;
        int bs;
        S.xq[tid] = quant8_oct(v, &d, &bs);
        if ((lane & 7u) == 0) {
            S.xd[tid >> 3] = d;
            S.xbs[tid >> 3] = bs;
        }
    }
    __syncthreads();

    // ---- phase 1: router partial dots ----
    if (rc1 > rc0) mbar_wait(&S.mbar[0], 0, a.err);
    for (uint32_t c = rc0 + warp; c < rc1; c += NW) {
        const float4 *w4 = reinterpret_cast<const float4 *>(stage + (size_t)(c - rc0) * RCHUNK * 4u);
        const uint32_t part = c % (H / RCHUNK);
        const float4 *x4 = reinterpret_cast<const float4 *>(S.xn + part * RCHUNK);
        float acc = 0.f;
#pragma unroll
        for (uint32_t i = 0; i < RCHUNK / 128; i++) {
            const float4 wv = w4[lane + 32 * i], xv = x4[lane + 32 * i];
            acc += wv.x * xv.x + wv.y * xv.y + wv.z * xv.z + wv.w * xv.w;
        }
        acc = q4b_warp_sum(acc);
        if (lane == 0) a.logit_part[c] = acc;
    }
    grid_barrier(a.bar, a.err);

    // ---- phase 2a: softmax + top-k (every CTA, same result) ----
    {
        float l[2] = {-INFINITY, -INFINITY};
        float m = -INFINITY;
        for (uint32_t j = 0, e = tid; e < a.n_expert; e += NT, j++) {
            const float4 pp = __ldcg(reinterpret_cast<const float4 *>(a.logit_part) + e);
            l[j] = (pp.x + pp.y) + (pp.z + pp.w);
            m = fmaxf(m, l[j]);
        }
        m = block_reduce_max(m, S.red);
        float s = 0.f;
        for (uint32_t j = 0, e = tid; e < a.n_expert; e += NT, j++) {
            l[j] = expf(l[j] - m);
            s += l[j];
        }
        s = block_reduce_sum(s, S.red);
        const float inv = s > 0.f ? __fdiv_rn(1.0f, s) : 0.f;
        for (uint32_t j = 0, e = tid; e < a.n_expert; e += NT, j++) S.p[e] = __fmul_rn(l[j], inv);
        __syncthreads();
        if (warp == 0) {
            // each lane keeps its strided values in registers; a pick is the
            // largest value, lowest index among equals
            float v[32];
            const uint32_t per = (a.n_expert + 31u) / 32u;
#pragma unroll
            for (uint32_t j = 0; j < 32; j++)
                v[j] = (j < per && lane + 32u * j < a.n_expert) ? S.p[lane + 32u * j] : -1.f;
            float wsum = 0.f;
            for (uint32_t t = 0; t < a.topk; t++) {
                float best = -1.f;
                uint32_t bj = 0;
#pragma unroll
                for (uint32_t j = 0; j < 32; j++)
                    if (j < per && v[j] > best) {
                        best = v[j];
                        bj = j;
                    }
                // values are >= 0 (or -1 when taken): compare as ordered bits
                const uint32_t key = best < 0.f ? 0u : __float_as_uint(best) + 1u;
                const uint32_t kmax = __reduce_max_sync(0xffffffffu, key);
                const uint32_t cand = key == kmax ? lane + 32u * bj : 0xffffffffu;
                const uint32_t idx = __reduce_min_sync(0xffffffffu, cand);
                if ((idx & 31u) == lane) {
#pragma unroll
                    for (uint32_t j = 0; j < 32; j++)
                        if (j == (idx >> 5)) v[j] = -1.f;
                }
                if (lane == 0) {
                    S.ids[t] = (int32_t)idx;
                    S.wts[t] = __uint_as_float(kmax - 1u);
                }
                wsum = __fadd_rn(wsum, __uint_as_float(kmax - 1u));
            }
            __syncwarp();
            if (lane < a.topk && wsum > 0.f)
                S.wts[lane] = __fmul_rn(S.wts[lane], __fdiv_rn(1.0f, wsum));
            if (lane == 0 && a.shared_slot >= 0) {
                S.ids[a.topk] = a.shared_slot;
                S.wts[a.topk] = 1.0f;
            }
            __syncwarp();
            if (cta == 0 && lane < a.topk) {
                if (a.ids_out) a.ids_out[lane] = S.ids[lane];
                if (a.wts_out) a.wts_out[lane] = S.wts[lane];
            }
        }
        __syncthreads();
    }

    // ---- phase 2b: fetch this CTA's gate/up tiles (chunks of UCHUNK units) and down tiles ----
    // unit u = e * F + f; chunk k covers units [u0 + k*UCHUNK, ...) cut at expert boundaries
    // staging: chunk k at stage + k * UCHUNK * 2 * 880: gate tiles then up tiles
    const uint32_t n_chunks = (u1 - u0 + UCHUNK - 1) / UCHUNK;
    if (warp == 0) {
        for (uint32_t k = lane; k < n_chunks; k += 32) {
            const uint32_t ua = u0 + k * UCHUNK, ub = min(ua + UCHUNK, u1);
            uint8_t *dst = stage + (size_t)k * UCHUNK * 2u * Q4B_TILE_BYTES;
            // a chunk may straddle two experts: copy each expert's run separately
            mbar_expect_tx(&S.mbar[1 + k], (ub - ua) * 2u * Q4B_TILE_BYTES);
            uint32_t u = ua;
            while (u < ub) {
                const uint32_t e = u / F, f = u - e * F;
                const uint32_t run = min(ub - u, F - f);
                const uint8_t *pk = a.base + (uint64_t)S.ids[e] * a.stride;
                bulk_g2s(dst + (size_t)(u - ua) * Q4B_TILE_BYTES, pk + a.og + (size_t)f * Q4B_TILE_BYTES,
                         run * Q4B_TILE_BYTES, &S.mbar[1 + k]);
                bulk_g2s(dst + (size_t)(UCHUNK + (u - ua)) * Q4B_TILE_BYTES,
                         pk + a.ou + (size_t)f * Q4B_TILE_BYTES, run * Q4B_TILE_BYTES, &S.mbar[1 + k]);
                u += run;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) mbar_expect_tx(&S.mbar[MAX_CHUNKS + 1], (v1 - v0) * Q4B_TILE_BYTES);
        __syncwarp();
        for (uint32_t v = v0 + lane; v < v1; v += 32) {
            const uint32_t rq = v / ne, e = v - rq * ne;
            bulk_g2s(dstage + (size_t)(v - v0) * Q4B_TILE_BYTES,
                     a.base + (uint64_t)S.ids[e] * a.stride + a.od + (size_t)rq * Q4B_TILE_BYTES,
                     Q4B_TILE_BYTES, &S.mbar[MAX_CHUNKS + 1]);
        }
    }

    // ---- phase 2c: gate/up dots, SwiGLU ----
    {
        int q[16];
#pragma unroll
        for (int i = 0; i < 16; i++) q[i] = (int)S.xq[16u * lane + i];
        const float dx0 = S.xd[2u * lane], dx1 = S.xd[2u * lane + 1];
        const int bs0 = S.xbs[2u * lane], bs1 = S.xbs[2u * lane + 1];
        const uint32_t *tl = tab + lane;
        for (uint32_t u = u0 + warp; u < u1; u += NW) {
            const uint32_t k = (u - u0) / UCHUNK, i = (u - u0) - k * UCHUNK;
            mbar_wait(&S.mbar[1 + k], 0, a.err);
            const uint8_t *tg = stage + ((size_t)k * UCHUNK * 2u + i) * Q4B_TILE_BYTES;
            const uint8_t *tu = tg + (size_t)UCHUNK * Q4B_TILE_BYTES;
            float g = q4b_tile_lane_dot(tg, lane, tl, q, dx0, dx1, bs0, bs1);
            float up = q4b_tile_lane_dot(tu, lane, tl, q, dx0, dx1, bs0, bs1);
            g = q4b_warp_sum(g);
            up = q4b_warp_sum(up);
            if (lane == 0) a.h[u] = q4b_swiglu(g, up);  // u = e * F + f
        }
    }
    grid_barrier(a.bar, a.err);

    // ---- phase 3a: Q8-A of the hidden rows (all experts; 8 lanes per group) ----
    for (uint32_t w4 = tid; w4 < ne * (F / 4); w4 += NT) {
        const float4 hv = __ldcg(reinterpret_cast<const float4 *>(a.h) + w4);
        float d;
        int bs;
        const uint32_t word = quant8_oct(hv, &d, &bs);
        const uint32_t e = w4 / (F / 4), i = w4 - e * (F / 4);
        S.hq[e][i] = word;
        if ((lane & 7u) == 0) {
            S.hd[e][i >> 3] = d;
            S.hbs[e][i >> 3] = bs;
        }
    }
    __syncthreads();

    // ---- phase 3b: down tiles; tile = 4 rows x 2 blocks; lane: block l/4 -> row (l/8), half (l/4)&1 ----
    mbar_wait(&S.mbar[MAX_CHUNKS + 1], 0, a.err);
    {
        const uint32_t *tl = tab + lane;
        const uint32_t col16 = 16u * (lane & 7u);  // first activation word of this lane's 64 columns
        for (uint32_t v = v0 + warp; v < v1; v += NW) {
            const uint32_t rq = v / ne, e = v - rq * ne;
            int q[16];
#pragma unroll
            for (int i = 0; i < 16; i += 4) {
                const uint4 t4 = *reinterpret_cast<const uint4 *>(&S.hq[e][col16 + i]);
                q[i] = (int)t4.x;
                q[i + 1] = (int)t4.y;
                q[i + 2] = (int)t4.z;
                q[i + 3] = (int)t4.w;
            }
            const uint32_t g0 = 2u * (lane & 7u);
            float r = q4b_tile_lane_dot(dstage + (size_t)(v - v0) * Q4B_TILE_BYTES, lane, tl, q,
                                        S.hd[e][g0], S.hd[e][g0 + 1], S.hbs[e][g0], S.hbs[e][g0 + 1]);
            r += __shfl_xor_sync(0xffffffffu, r, 1);
            r += __shfl_xor_sync(0xffffffffu, r, 2);
            r += __shfl_xor_sync(0xffffffffu, r, 4);
            if ((lane & 7u) == 0) S.part[v - v0][lane >> 3] = S.wts[e] * r;
        }
    }
    __syncthreads();
    // combine over the experts in list order; a row quad split between two CTAs is
    // finished with one atomic add from each (y starts at 0, so the sum of the two
    // parts does not depend on which lands first)
    {
        const uint32_t rq_first = v0 / ne, rq_last = (v1 - 1) / ne;
        for (uint32_t t = tid; t < (rq_last - rq_first + 1) * 4u && v1 > v0; t += NT) {
            const uint32_t rq = rq_first + (t >> 2), row = t & 3u;
            const uint32_t va = max(rq * ne, v0), vb = min((rq + 1) * ne, v1);
            float sum = 0.f;
            for (uint32_t v = va; v < vb; v++) sum += S.part[v - v0][row];
            if (vb - va == ne)
                a.y[rq * 4u + row] = sum;
            else
                atomicAdd(&a.y[rq * 4u + row], sum);
        }
    }
}

}  // namespace fused

// Scratch of the fused kernel (allocated once, by the first call or by warm).
static float *g_f_logit_part = nullptr;
static float *g_f_h = nullptr;
static unsigned long long *g_f_bar = nullptr;
static bool g_f_attr_set = false;

static bool fused_scratch() {
    if (g_f_bar) return true;
    Q4B_CHECK(cudaMalloc(&g_f_logit_part, 1024 * 4 * sizeof(float)));
    Q4B_CHECK(cudaMalloc(&g_f_h, (size_t)fused::MAX_E * fused::F * sizeof(float)));
    Q4B_CHECK(cudaMalloc(&g_f_bar, sizeof(unsigned long long)));
    Q4B_CHECK(cudaMemset(g_f_bar, 0, sizeof(unsigned long long)));
    return true;
}

bool q4b_fused_warm() { return fused_scratch(); }

void q4b_fused_reset_barrier() {
    if (g_f_bar) cudaMemsetAsync(g_f_bar, 0, sizeof(unsigned long long), g_q4b.stream);
}

// Returns false when the fused kernel does not apply (caller takes the chain).
bool q4b_moe_decode_fused(const uint8_t *base, uint64_t stride, uint64_t og, uint64_t ou,
                          uint64_t od, int32_t shared_slot, const float *d_x,
                          const float *d_norm_w, float eps, const float *d_router,
                          uint32_t n_expert, uint32_t topk, uint32_t n_embd, uint32_t n_ff,
                          float *d_y, int32_t *d_ids, float *d_wts) {
    using namespace fused;
    Q4bState &s = g_q4b;
    if (n_embd != H || n_ff != F || n_expert > 1024 || (n_expert % 4) || topk > 32) return false;
    if (!q4b_ptr_tiled(base) || (og % 16) || (ou % 16) || (od % 16) || (stride % 16)) return false;
    if (((uintptr_t)d_router % 16) || ((uintptr_t)d_x % 16) || (d_norm_w && ((uintptr_t)d_norm_w % 16)))
        return false;
    if (!fused_scratch()) return false;
    const uint32_t ncta = (uint32_t)s.n_sm;
    const uint32_t ne = topk + (shared_slot >= 0 ? 1u : 0u);
    const uint32_t max_units = (ne * F + ncta - 1) / ncta + 1;
    const uint32_t n_chunks = (max_units + UCHUNK - 1) / UCHUNK;
    const uint32_t max_dt = ((H / 4) * ne + ncta - 1) / ncta + 1;
    const uint32_t max_rc = (n_expert * (H / RCHUNK) + ncta - 1) / ncta + 1;
    if (n_chunks > MAX_CHUNKS || max_dt > 64 || ne > MAX_E) return false;
    Args a;
    a.base = base;
    a.stride = stride;
    a.og = og;
    a.ou = ou;
    a.od = od;
    a.shared_slot = shared_slot;
    a.x = d_x;
    a.norm_w = d_norm_w;
    a.router = d_router;
    a.eps = eps;
    a.n_expert = n_expert;
    a.topk = topk;
    a.y = d_y;
    a.ids_out = d_ids;
    a.wts_out = d_wts;
    a.logit_part = g_f_logit_part;
    a.h = g_f_h;
    a.bar = g_f_bar;
    a.err = s.err_d;
    uint32_t stage_bytes = n_chunks * UCHUNK * 2u * Q4B_TILE_BYTES;
    if (stage_bytes < max_rc * RCHUNK * 4u) stage_bytes = max_rc * RCHUNK * 4u;
    const uint32_t small = (uint32_t)((sizeof(Small) + 127) & ~127u);
    a.off_stage = 65536u + small;
    a.stage_bytes = (stage_bytes + 127u) & ~127u;
    a.off_down = a.off_stage + a.stage_bytes;
    a.down_bytes = max_dt * Q4B_TILE_BYTES;
    const size_t smem = (size_t)a.off_down + a.down_bytes + 1024;
    if (smem > 227u * 1024u) return false;
    if (!g_f_attr_set) {
        Q4B_CHECK(cudaFuncSetAttribute(moe_decode_fused_k, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       227 * 1024));
        g_f_attr_set = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ncta);
    cfg.blockDim = dim3(NT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s.stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident at once: the grid barrier needs it
    at[0].val.cooperative = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, moe_decode_fused_k, a) != cudaSuccess) {
        fprintf(stderr, "q4cuda: fused decode launch failed: %s\n", cudaGetErrorString(cudaGetLastError()));
        return false;
    }
    g_q4b_launches++;
    return true;
}
