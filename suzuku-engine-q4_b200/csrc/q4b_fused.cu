// One MoE layer for one token as ONE persistent kernel (one CTA per SM):
//
//   start    bulk async copies of this CTA's share of the router matrix and of the
//            shared expert's gate/up tiles are issued before anything else
//   phase 0  every CTA: code table -> shared memory, RMSNorm of x, Q8-A quantisation
//   phase 1  router: partial dots of this CTA's 2 KB router chunks
//            -- grid barrier 1: arrive; while the others arrive, this CTA computes
//               its share of the shared expert's gate/up rows (they do not depend
//               on the routing); then wait --
//   phase 2  every CTA: softmax + top-k (redundantly, from the logits); bulk copies
//            of this CTA's share of the picked experts' gate/up tiles, then of all
//            experts' down tiles; gate/up dots, SwiGLU, h -> global
//            -- grid barrier 2 --
//   phase 3  every CTA: Q8-A of the hidden rows, down tiles x hq, weighted sum
//            over the experts in list order, y written
//
// Weight bytes cross HBM -> shared memory exactly once, by 1-D bulk async copies
// (plain cp.async.bulk into this CTA only) that complete on mbarriers; nothing is re-read.
// Replaces the reference's per-layer launch chain (src/q4_moe.c:2077-2133;
// kernels wmoe_iq3_gu_q8 / wmoe_iq3_ya_q8, src/q4_rocm.cu:3912-4120).  Needs the
// tiled arena format (q4b_tile.cuh), n_embd == 2048, n_ff == 512,
// n_expert <= 768, topk <= 32.
#include "q4b_tile.cuh"

#include <atomic>

#include "../../include/q4cuda.h"

extern std::atomic<uint64_t> g_q4b_launches;
bool q4b_ptr_tiled(const void *p);

namespace fused {

constexpr uint32_t NT = 768;          // threads per CTA
constexpr uint32_t NW = NT / 32;      // warps
constexpr uint32_t H = 2048;          // n_embd
constexpr uint32_t F = 512;           // n_ff
constexpr uint32_t RCHUNK = 512;      // router chunk: 512 floats = 2 KB
constexpr uint32_t MAX_E = 24;        // experts per token incl. shared (more: the launch chain runs)
constexpr uint32_t UCHUNK = 8;        // gate/up units per bulk-copy chunk
constexpr uint32_t MAX_CHUNKS = 8;
constexpr uint32_t MAX_UNITS = 64;    // routed (expert, hidden unit) pairs per CTA
constexpr uint32_t MAX_SH = 8;        // shared-expert units per CTA
constexpr uint32_t MAX_DT = 64;       // down tiles per CTA
constexpr uint32_t WAIT_LIMIT = 1000000u;  // polls before a wait gives up

// mbarrier slots
constexpr uint32_t MB_ROUTER = 0, MB_SHARED = 1, MB_DOWN = 2, MB_CHUNK0 = 3;
constexpr uint32_t N_MBAR = MB_CHUNK0 + MAX_CHUNKS;

// error word bits
constexpr uint32_t ERR_MBAR = 1u, ERR_GRID = 2u;

struct Args {
    const uint8_t *base;
    uint64_t stride, og, ou, od;
    int32_t shared_slot;
    const float *x, *norm_w, *router;
    const uint32_t *codes;        // 512 byte-expanded codebook words (device memory)
    float eps;
    uint32_t n_expert, topk;
    float *y;
    int32_t *ids_out;
    float *wts_out;
    float *logit_part;            // [n_expert][H / RCHUNK]
    float *h;                     // [MAX_E][F]
    unsigned long long *bar;      // grid barrier counter
    uint32_t *err;
    unsigned long long *prof;     // optional [gridDim.x][16] phase time stamps (ns), or NULL
    float *y_host;                // optional: host-mapped copy of y, written by the last CTA to finish
    volatile uint32_t *flag_host; // host-mapped word that receives flag_val after y_host is complete
    uint32_t flag_val;
    // shared-memory carve-up (bytes from the 1024-aligned start)
    uint32_t off_stage, off_down, off_sh;
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

// Phase time stamp for the optional in-kernel profile.
__device__ __forceinline__ void stamp(const Args &a, uint32_t slot) {
    if (a.prof && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        a.prof[blockIdx.x * 16u + slot] = t;
    }
}

// Grid barrier in two halves.  The counter only grows: every CTA adds one per
// barrier, so barrier number k of this launch is complete when the counter
// reaches base + (k + 1) * gridDim.x, where base is the (multiple of gridDim.x)
// value the counter had when the launch began.  A CTA reads base at its start:
// it may already see a few arrivals of faster CTAs at the first barrier, so it
// rounds down.  No reset between barriers or launches.  The wait is bounded: a
// CTA that waits too long records ERR_GRID and goes on (its results are then
// meaningless, but nothing hangs).  Both halves are called by thread 0 only,
// with __syncthreads() before the arrive and after the wait.
__device__ __forceinline__ unsigned long long grid_barrier_base(const unsigned long long *ctr) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(ctr) : "memory");
    return v - v % gridDim.x;
}
__device__ __forceinline__ void grid_arrive(unsigned long long *ctr) {
    asm volatile("red.release.gpu.global.add.u64 [%0], 1;" ::"l"(ctr) : "memory");
}
__device__ __forceinline__ void grid_wait(const unsigned long long *ctr, unsigned long long target,
                                          uint32_t *err) {
    uint32_t i = 0;
    for (; i < WAIT_LIMIT; i++) {
        unsigned long long v;
        asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(ctr) : "memory");
        if (v >= target) break;
    }
    if (i == WAIT_LIMIT) atomicOr(err, ERR_GRID);
}

// Q8-A of 32 consecutive floats held four per lane by eight neighbouring lanes.
// Returns the packed int8x4 word; every lane gets the group's d and sum.
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
//   [65536, +...)     small arrays (below), then the staging regions
struct Small {
    uint32_t last;   // 1 in the CTA that finished last (host hand-off)
    uint64_t mbar[N_MBAR];
    alignas(16) float xn[H];            // normalised x (router input)
    alignas(16) uint32_t xq[H / 4];     // Q8-A of xn, int8x4 words
    float xd[H / 32];
    int xbs[H / 32];
    int32_t ids[MAX_E];
    float wts[MAX_E];
    float red[NW];
    double redd[NW];
    alignas(16) uint32_t hq[MAX_E][F / 4];  // Q8-A of the hidden rows
    float hd[MAX_E][F / 32];
    int hbs[MAX_E][F / 32];
    float part[MAX_DT][4];              // phase-3 partial sums: [tile][row in tile]
    float gu[MAX_UNITS][2];             // phase-2 gate and up dots of this CTA's units
    float gu_sh[MAX_SH][2];             // the same for its shared-expert units
    uint32_t ck[NW][32];                // routing: per-warp ordered candidates (key, index)
    uint32_t ci[NW][32];
};

__device__ __forceinline__ float block_reduce_max(float v, float *red) {
    v = q4b_warp_max(v);
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (uint32_t i = 1; i < NW; i++) r = fmaxf(r, red[i]);
    __syncthreads();
    return r;
}
__device__ __forceinline__ float block_reduce_sum(float v, float *red) {
    v = q4b_warp_sum(v);
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.f;
#pragma unroll
    for (uint32_t i = 0; i < NW; i++) r += red[i];
    __syncthreads();
    return r;
}

// Softmax over the logits and top-k by the whole CTA; thread i owns expert i
// (n_expert <= NT).  A pick is the largest probability, the lowest index among
// equal ones; weights are renormalised in rank order (src/q4_quant.c:715-755).
// Two stages, nothing indexed dynamically: every warp extracts the ordered
// top-k of its own 32 experts with warp reductions, then warp 0 merges the NW
// ordered lists (lane w walks list w).
__device__ __forceinline__ void route_block(const Args &a, Small &S, uint32_t tid, uint32_t cta) {
    const uint32_t lane = tid & 31u, warp = tid >> 5;
    float l = -INFINITY;
    if (tid < a.n_expert) {
        const float4 pp = __ldcg(reinterpret_cast<const float4 *>(a.logit_part) + tid);
        l = (pp.x + pp.y) + (pp.z + pp.w);
    }
    const float m = block_reduce_max(l, S.red);
    const float e = tid < a.n_expert ? expf(l - m) : 0.f;
    const float s = block_reduce_sum(e, S.red);
    const float inv = s > 0.f ? __fdiv_rn(1.0f, s) : 0.f;
    // probabilities are >= 0: their bit patterns order like the values; 0 = none
    uint32_t key = tid < a.n_expert ? __float_as_uint(__fmul_rn(e, inv)) + 1u : 0u;
    uint32_t my_key = 0u, my_idx = 0xffffffffu;
    if (warp * 32u < a.n_expert) {
        for (uint32_t r = 0; r < a.topk; r++) {
            const uint32_t kmax = __reduce_max_sync(0xffffffffu, key);
            const uint32_t imin = __reduce_min_sync(0xffffffffu, key == kmax ? tid : 0xffffffffu);
            if (lane == r) {
                my_key = kmax;
                my_idx = kmax ? imin : 0xffffffffu;
            }
            if (tid == imin) key = 0u;
        }
    }
    S.ck[warp][lane] = my_key;
    S.ci[warp][lane] = my_idx;
    __syncthreads();
    if (warp == 0) {
        uint32_t pos = 0;
        uint32_t hk = lane < NW ? S.ck[lane][0] : 0u;
        uint32_t hi = lane < NW ? S.ci[lane][0] : 0xffffffffu;
        float wsum = 0.f, my_w = 0.f;
        uint32_t my_id = 0;
        for (uint32_t t = 0; t < a.topk; t++) {
            const uint32_t kmax = __reduce_max_sync(0xffffffffu, hk);
            const uint32_t imin = __reduce_min_sync(0xffffffffu, hk == kmax ? hi : 0xffffffffu);
            if (hk == kmax && hi == imin) {  // this lane's list head was taken
                pos++;
                hk = pos < 32u ? S.ck[lane][pos] : 0u;
                hi = pos < 32u ? S.ci[lane][pos] : 0xffffffffu;
            }
            const float w = __uint_as_float(kmax - 1u);
            if (lane == t) {
                my_id = imin;
                my_w = w;
            }
            wsum = __fadd_rn(wsum, w);
        }
        if (lane < a.topk) {
            const float w = wsum > 0.f ? __fmul_rn(my_w, __fdiv_rn(1.0f, wsum)) : my_w;
            S.ids[lane] = (int32_t)my_id;
            S.wts[lane] = w;
            if (cta == 0) {
                if (a.ids_out) a.ids_out[lane] = (int32_t)my_id;
                if (a.wts_out) a.wts_out[lane] = w;
            }
        }
        if (lane == 0 && a.shared_slot >= 0) {
            S.ids[a.topk] = a.shared_slot;
            S.wts[a.topk] = 1.0f;
        }
    }
}

// The kernel body; xrow is the token's hidden row as H/4 float4: device memory for the
// device-pointer call, the kernel's own parameter block for the host-buffer call.
__device__ __forceinline__ void fused_body(const Args &a, const float4 *xrow) {
    // used directly (no integer round trip), so that the compiler keeps these as
    // shared-space accesses; dynamic shared memory starts on the declared alignment
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *sm = smem_raw;
    uint32_t *tab = reinterpret_cast<uint32_t *>(sm);
    Small &S = *reinterpret_cast<Small *>(sm + 65536);
    uint8_t *stage = sm + a.off_stage;  // router chunks, then routed gate/up tiles
    uint8_t *dstage = sm + a.off_down;  // down tiles
    uint8_t *sstage = sm + a.off_sh;    // shared-expert gate/up tiles
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t cta = blockIdx.x, ncta = gridDim.x;
    const bool has_sh = a.shared_slot >= 0;
    const uint32_t ne = a.topk + (has_sh ? 1u : 0u);

    // ---- work split ----
    const uint32_t n_rchunks = a.n_expert * (H / RCHUNK);
    const uint32_t rc0 = (uint32_t)((uint64_t)cta * n_rchunks / ncta);
    const uint32_t rc1 = (uint32_t)((uint64_t)(cta + 1) * n_rchunks / ncta);
    const uint32_t n_units = a.topk * F;  // routed (expert, hidden unit) pairs
    const uint32_t u0 = (uint32_t)((uint64_t)cta * n_units / ncta);
    const uint32_t u1 = (uint32_t)((uint64_t)(cta + 1) * n_units / ncta);
    const uint32_t s0 = has_sh ? (uint32_t)((uint64_t)cta * F / ncta) : 0u;  // shared-expert units
    const uint32_t s1 = has_sh ? (uint32_t)((uint64_t)(cta + 1) * F / ncta) : 0u;
    // down tiles = (row quad, expert) pairs, expert fastest; a CTA takes whole row quads, so every
    // output row is summed over the experts by one CTA, in list order, and written once
    const uint32_t v0 = (uint32_t)((uint64_t)cta * (H / 4) / ncta) * ne;
    const uint32_t v1 = (uint32_t)((uint64_t)(cta + 1) * (H / 4) / ncta) * ne;

    // loads with nothing before them in the dependency chain go first
    float4 xv = make_float4(0.f, 0.f, 0.f, 0.f), wv = make_float4(1.f, 1.f, 1.f, 1.f);
    uint32_t code = 0;
    if (tid < H / 4) {
        xv = xrow[tid];
        if (a.norm_w) wv = reinterpret_cast<const float4 *>(a.norm_w)[tid];
        code = a.codes[tid];
    }
    unsigned long long bar_base = 0;
    if (tid == 0) {
        bar_base = grid_barrier_base(a.bar);
        for (uint32_t i = 0; i < N_MBAR; i++) mbar_init(&S.mbar[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (tid == 0 && rc1 > rc0) {  // router chunks: contiguous in memory
        const uint32_t bytes = (rc1 - rc0) * RCHUNK * 4u;
        mbar_expect_tx(&S.mbar[MB_ROUTER], bytes);
        bulk_g2s(stage, a.router + (size_t)rc0 * RCHUNK, bytes, &S.mbar[MB_ROUTER]);
    }
    if (tid == 32 && s1 > s0) {   // shared expert: gate tiles then up tiles of units [s0, s1)
        const uint32_t bytes = (s1 - s0) * Q4B_TILE_BYTES;
        const uint8_t *pk = a.base + (uint64_t)a.shared_slot * a.stride;
        mbar_expect_tx(&S.mbar[MB_SHARED], 2u * bytes);
        bulk_g2s(sstage, pk + a.og + (size_t)s0 * Q4B_TILE_BYTES, bytes, &S.mbar[MB_SHARED]);
        bulk_g2s(sstage + (size_t)MAX_SH * Q4B_TILE_BYTES, pk + a.ou + (size_t)s0 * Q4B_TILE_BYTES,
                 bytes, &S.mbar[MB_SHARED]);
    }

    stamp(a, 0);
    // ---- phase 0: code table, y = 0, RMSNorm, Q8-A ----
    // table entry i replicated once per lane: thread t < 512 holds entry t, a warp
    // broadcasts its 32 entries one by one
    if (tid < 512) {
#pragma unroll 8
        for (uint32_t i = 0; i < 32; i++) {
            const uint32_t v = __shfl_sync(0xffffffffu, code, i);
            tab[(warp * 32u + i) * 32u + lane] = v;
        }
    }
    {
        double ss = (double)xv.x * xv.x + (double)xv.y * xv.y + (double)xv.z * xv.z +
                    (double)xv.w * xv.w;
#pragma unroll
        for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) S.redd[warp] = ss;
        __syncthreads();
        if (tid < H / 4) {
            // pairwise, so the sixteen partial sums are not one long dependent chain
            double t8[8];
#pragma unroll
            for (uint32_t i = 0; i < 8; i++) t8[i] = S.redd[2 * i] + S.redd[2 * i + 1];
            const double tot = ((t8[0] + t8[1]) + (t8[2] + t8[3])) + ((t8[4] + t8[5]) + (t8[6] + t8[7]));
            // H is a power of two: multiplying by 1/H is the exact division
            const float scale =
                __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn((float)(tot * (1.0 / (double)H)), a.eps)));
            float4 v;
            v.x = __fmul_rn(xv.x, scale);
            v.y = __fmul_rn(xv.y, scale);
            v.z = __fmul_rn(xv.z, scale);
            v.w = __fmul_rn(xv.w, scale);
            if (a.norm_w) {
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
    }
    __syncthreads();
    stamp(a, 1);

    // ---- phase 1: router partial dots ----
    if (rc1 > rc0) mbar_wait(&S.mbar[MB_ROUTER], 0, a.err);
    stamp(a, 2);
    for (uint32_t c = rc0 + warp; c < rc1; c += NW) {
        const float4 *w4 = reinterpret_cast<const float4 *>(stage + (size_t)(c - rc0) * RCHUNK * 4u);
        const uint32_t part = c % (H / RCHUNK);
        const float4 *x4 = reinterpret_cast<const float4 *>(S.xn + part * RCHUNK);
        float acc = 0.f;
#pragma unroll
        for (uint32_t i = 0; i < RCHUNK / 128; i++) {
            const float4 rw = w4[lane + 32 * i], rx = x4[lane + 32 * i];
            acc += rw.x * rx.x + rw.y * rx.y + rw.z * rx.z + rw.w * rx.w;
        }
        acc = q4b_warp_sum(acc);
        if (lane == 0) a.logit_part[c] = acc;
    }
    stamp(a, 3);
    __syncthreads();
    // the last warp signals (its thread waits for the CTA's stores to land), so that
    // warp 0 and the others go straight on to the shared expert's rows
    if (tid == NT - 32) grid_arrive(a.bar);

    // activations of this lane's 64 columns (lane l of a gate/up tile owns columns 64 l ..)
    int q[16];
#pragma unroll
    for (int i = 0; i < 16; i++) q[i] = (int)S.xq[16u * lane + i];
    const float dx0 = S.xd[2u * lane], dx1 = S.xd[2u * lane + 1];
    const int bs0 = S.xbs[2u * lane], bs1 = S.xbs[2u * lane + 1];
    const uint32_t *tl = tab + lane;

    // ---- while the grid gathers: the shared expert's gate/up rows ----
    if (s1 > s0) {
        mbar_wait(&S.mbar[MB_SHARED], 0, a.err);
        for (uint32_t t = warp; t < 2u * (s1 - s0); t += NW) {
            const uint32_t ul = t >> 1, which = t & 1u;
            const uint8_t *tile = sstage + ((size_t)which * MAX_SH + ul) * Q4B_TILE_BYTES;
            float r = q4b_tile_lane_dot(tile, lane, tl, q, dx0, dx1, bs0, bs1);
            r = q4b_warp_sum(r);
            if (lane == 0) S.gu_sh[ul][which] = r;
        }
    }
    __syncthreads();
    if (tid < s1 - s0) a.h[a.topk * F + s0 + tid] = q4b_swiglu(S.gu_sh[tid][0], S.gu_sh[tid][1]);
    if (tid == 0) grid_wait(a.bar, bar_base + ncta, a.err);
    __syncthreads();
    stamp(a, 4);

    // ---- phase 2a: softmax + top-k (every CTA, same result) ----
    route_block(a, S, tid, cta);
    __syncthreads();
    stamp(a, 5);

    // ---- phase 2b: fetch this CTA's routed gate/up tiles (chunks of UCHUNK units) ----
    // unit u = e * F + f; chunk k covers units [u0 + k*UCHUNK, ...), cut at expert boundaries;
    // staging: chunk k at stage + k * UCHUNK * 2 * 880: gate tiles then up tiles.
    // One warp per chunk issues its copies.
    const uint32_t n_chunks = (u1 - u0 + UCHUNK - 1) / UCHUNK;
    if (warp < n_chunks && lane == 0) {
        const uint32_t k = warp;
        const uint32_t ua = u0 + k * UCHUNK, ub = min(ua + UCHUNK, u1);
        uint8_t *dst = stage + (size_t)k * UCHUNK * 2u * Q4B_TILE_BYTES;
        mbar_expect_tx(&S.mbar[MB_CHUNK0 + k], (ub - ua) * 2u * Q4B_TILE_BYTES);
        uint32_t u = ua;
        while (u < ub) {  // a chunk may straddle two experts: one copy per expert's run
            const uint32_t e = u / F, f = u - e * F;
            const uint32_t run = min(ub - u, F - f);
            const uint8_t *pk = a.base + (uint64_t)S.ids[e] * a.stride;
            bulk_g2s(dst + (size_t)(u - ua) * Q4B_TILE_BYTES, pk + a.og + (size_t)f * Q4B_TILE_BYTES,
                     run * Q4B_TILE_BYTES, &S.mbar[MB_CHUNK0 + k]);
            bulk_g2s(dst + (size_t)(UCHUNK + (u - ua)) * Q4B_TILE_BYTES,
                     pk + a.ou + (size_t)f * Q4B_TILE_BYTES, run * Q4B_TILE_BYTES,
                     &S.mbar[MB_CHUNK0 + k]);
            u += run;
        }
    }
    stamp(a, 6);
    // ---- phase 2c: routed gate/up dots (one tile per warp task), SwiGLU ----
    for (uint32_t t = warp; t < 2u * (u1 - u0); t += NW) {
        const uint32_t ul = t >> 1, which = t & 1u;
        const uint32_t k = ul / UCHUNK, i = ul - k * UCHUNK;
        mbar_wait(&S.mbar[MB_CHUNK0 + k], 0, a.err);
        if (t == 0) stamp(a, 13);
        const uint8_t *tile = stage + ((size_t)k * UCHUNK * 2u + which * UCHUNK + i) * Q4B_TILE_BYTES;
        float r = q4b_tile_lane_dot(tile, lane, tl, q, dx0, dx1, bs0, bs1);
        r = q4b_warp_sum(r);
        if (lane == 0) S.gu[ul][which] = r;
        if (t == 0) stamp(a, 14);
    }
    if (n_chunks) mbar_wait(&S.mbar[MB_CHUNK0 + n_chunks - 1], 0, a.err);
    stamp(a, 15);
    // The down tiles are needed only after the next grid barrier: the last two warps
    // ask for them after their own gate/up work, when the last gate/up chunk has landed,
    // so that they do not compete with the tiles that are needed first.
    if (warp >= NW - 2) {
        if (n_chunks) mbar_wait(&S.mbar[MB_CHUNK0 + n_chunks - 1], 0, a.err);
        const uint32_t t64 = tid - (NW - 2) * 32;
        if (t64 == 0) mbar_expect_tx(&S.mbar[MB_DOWN], (v1 - v0) * Q4B_TILE_BYTES);
        for (uint32_t v = v0 + t64; v < v1; v += 64) {
            const uint32_t rq = v / ne, e = v - rq * ne;
            bulk_g2s(dstage + (size_t)(v - v0) * Q4B_TILE_BYTES,
                     a.base + (uint64_t)S.ids[e] * a.stride + a.od + (size_t)rq * Q4B_TILE_BYTES,
                     Q4B_TILE_BYTES, &S.mbar[MB_DOWN]);
        }
    }

    __syncthreads();
    if (tid < u1 - u0) a.h[u0 + tid] = q4b_swiglu(S.gu[tid][0], S.gu[tid][1]);
    stamp(a, 7);
    __syncthreads();
    if (tid == 0) {
        grid_arrive(a.bar);
        grid_wait(a.bar, bar_base + 2ull * ncta, a.err);
    }
    __syncthreads();
    stamp(a, 8);

    // ---- phase 3a: Q8-A of the hidden rows (all experts; 8 lanes per group) ----
    // all loads first (they are L2 round trips), then the arithmetic
    {
        constexpr uint32_t HQ_IT = (MAX_E * (F / 4) + NT - 1) / NT;
        float4 hreg[HQ_IT];
#pragma unroll
        for (uint32_t it = 0; it < HQ_IT; it++) {
            const uint32_t w4 = tid + it * NT;
            if (w4 < ne * (F / 4)) hreg[it] = __ldcg(reinterpret_cast<const float4 *>(a.h) + w4);
        }
#pragma unroll
        for (uint32_t it = 0; it < HQ_IT; it++) {
            const uint32_t w4 = tid + it * NT;
            if (w4 < ne * (F / 4)) {  // warp-uniform: ne * F / 4 is a multiple of 32
                float d;
                int bs;
                const uint32_t word = quant8_oct(hreg[it], &d, &bs);
                const uint32_t e = w4 / (F / 4), i = w4 - e * (F / 4);
                S.hq[e][i] = word;
                if ((lane & 7u) == 0) {
                    S.hd[e][i >> 3] = d;
                    S.hbs[e][i >> 3] = bs;
                }
            }
        }
    }
    __syncthreads();
    stamp(a, 9);

    // ---- phase 3b: down tiles; tile = 4 rows x 2 blocks; lane: block l/4 -> row l/8, half (l/4)&1 ----
    mbar_wait(&S.mbar[MB_DOWN], 0, a.err);
    stamp(a, 10);
    {
        const uint32_t col16 = 16u * (lane & 7u);  // first activation word of this lane's 64 columns
        const uint32_t g0 = 2u * (lane & 7u);
        for (uint32_t v = v0 + warp; v < v1; v += NW) {
            const uint32_t rq = v / ne, e = v - rq * ne;
            int hqr[16];
#pragma unroll
            for (int i = 0; i < 16; i += 4) {
                const uint4 t4 = *reinterpret_cast<const uint4 *>(&S.hq[e][col16 + i]);
                hqr[i] = (int)t4.x;
                hqr[i + 1] = (int)t4.y;
                hqr[i + 2] = (int)t4.z;
                hqr[i + 3] = (int)t4.w;
            }
            float r = q4b_tile_lane_dot(dstage + (size_t)(v - v0) * Q4B_TILE_BYTES, lane, tl, hqr,
                                        S.hd[e][g0], S.hd[e][g0 + 1], S.hbs[e][g0], S.hbs[e][g0 + 1]);
            r += __shfl_xor_sync(0xffffffffu, r, 1);
            r += __shfl_xor_sync(0xffffffffu, r, 2);
            r += __shfl_xor_sync(0xffffffffu, r, 4);
            if ((lane & 7u) == 0) S.part[v - v0][lane >> 3] = S.wts[e] * r;
        }
    }
    __syncthreads();
    stamp(a, 11);
    // combine over the experts in list order
    for (uint32_t t = tid; t < ((v1 - v0) / ne) * 4u; t += NT) {
        const uint32_t ql = t >> 2, row = t & 3u;
        float sum = 0.f;
        for (uint32_t e = 0; e < ne; e++) sum += S.part[ql * ne + e][row];
        const uint32_t r = (v0 / ne + ql) * 4u + row;
        a.y[r] = sum;
    }
    stamp(a, 12);
    // Host hand-off (the call with host buffers): the CTA that finishes last copies y into the
    // caller's pinned, mapped host buffer and then raises the flag the host is spinning on, so
    // the result needs neither a copy node nor a stream wake-up.  One CTA writes and fences at
    // system scope: having every CTA write its own rows and fence was measured slower (148
    // system-scope fences over the PCIe writes instead of one).  The count rides on the barrier
    // counter (a third arrival per CTA keeps it a multiple of the grid size).
    if (a.y_host) {
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const unsigned long long old = atomicAdd(a.bar, 1ull);
            S.last = old == bar_base + 3ull * ncta - 1ull ? 1u : 0u;
        }
        __syncthreads();
        if (S.last) {
            __threadfence();
            for (uint32_t i = tid; i < H / 4u; i += NT)
                reinterpret_cast<float4 *>(a.y_host)[i] = __ldcg(reinterpret_cast<const float4 *>(a.y) + i);
            __threadfence_system();
            __syncthreads();
            if (tid == 0) *a.flag_host = a.flag_val;   // every writer fenced at system scope above
            stamp(a, 15);   // in the last CTA only: when the flag was written
        }
    }
}

__global__ void __launch_bounds__(NT, 1) moe_decode_fused_k(const Args a) {
    fused_body(a, reinterpret_cast<const float4 *>(a.x));
}

// The host-buffer form: the 8 KB hidden row travels inside the launch's parameter block, so
// the call needs no separate host-to-device copy ahead of the kernel.
struct XRow {
    float4 v[H / 4];
};
__global__ void __launch_bounds__(NT, 1) moe_decode_fused_xp_k(const Args a, const __grid_constant__ XRow xr) {
    fused_body(a, xr.v);
}

}  // namespace fused

// Scratch of the fused kernel (allocated once, by init / scratch_warm).
static float *g_f_logit_part = nullptr;
static float *g_f_h = nullptr;
static unsigned long long *g_f_bar = nullptr;
static bool g_f_attr_set = false;
static unsigned long long *g_f_prof = nullptr;  // set by q4_cuda_fused_profile_enable(1)

static bool fused_scratch() {
    if (g_f_bar) return true;
    Q4B_CHECK(cudaMalloc(&g_f_logit_part, 1024 * 4 * sizeof(float)));
    Q4B_CHECK(cudaMalloc(&g_f_h, (size_t)fused::MAX_E * fused::F * sizeof(float)));
    Q4B_CHECK(cudaMalloc(&g_f_bar, sizeof(unsigned long long)));
    Q4B_CHECK(cudaMemset(g_f_bar, 0, sizeof(unsigned long long)));
    return true;
}

bool q4b_fused_warm() { return fused_scratch(); }

// After a bounded wait gave up the barrier counter is no longer a multiple of
// the grid size: start again from zero.
void q4b_fused_reset_barrier() {
    if (g_f_bar) cudaMemsetAsync(g_f_bar, 0, sizeof(unsigned long long), g_q4b.stream);
}

// Returns false when the fused kernel does not apply (caller takes the chain).
bool q4b_moe_decode_fused(const uint8_t *base, uint64_t stride, uint64_t og, uint64_t ou,
                          uint64_t od, int32_t shared_slot, const float *d_x,
                          const float *d_norm_w, float eps, const float *d_router,
                          uint32_t n_expert, uint32_t topk, uint32_t n_embd, uint32_t n_ff,
                          float *d_y, int32_t *d_ids, float *d_wts, float *y_host_dev,
                          uint32_t *flag_host_dev, uint32_t flag_val, const float *h_x_param) {
    using namespace fused;
    Q4bState &s = g_q4b;
    if (n_embd != H || n_ff != F || n_expert > NT || topk > 32) return false;
    if (!q4b_ptr_tiled(base) || (og % 16) || (ou % 16) || (od % 16) || (stride % 16)) return false;
    if (((uintptr_t)d_router % 16) || (!h_x_param && ((uintptr_t)d_x % 16)) ||
        (d_norm_w && ((uintptr_t)d_norm_w % 16)))
        return false;
    if (!fused_scratch()) return false;
    const uint32_t ncta = (uint32_t)s.n_sm;
    const uint32_t ne = topk + (shared_slot >= 0 ? 1u : 0u);
    const uint32_t max_units = (topk * F + ncta - 1) / ncta + 1;
    const uint32_t n_chunks = (max_units + UCHUNK - 1) / UCHUNK;
    const uint32_t max_sh = (F + ncta - 1) / ncta + 1;
    const uint32_t max_dt = ((H / 4 + ncta - 1) / ncta) * ne;
    const uint32_t max_rc = (n_expert * (H / RCHUNK) + ncta - 1) / ncta + 1;
    if (n_chunks > MAX_CHUNKS || n_chunks > NW - 2 || max_dt > MAX_DT || max_units > MAX_UNITS ||
        max_sh > MAX_SH || ne > MAX_E)
        return false;
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
    a.codes = s.codes_d;
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
    a.prof = g_f_prof;
    a.y_host = y_host_dev;
    a.flag_host = flag_host_dev;
    a.flag_val = flag_val;
    uint32_t stage_bytes = n_chunks * UCHUNK * 2u * Q4B_TILE_BYTES;
    if (stage_bytes < max_rc * RCHUNK * 4u) stage_bytes = max_rc * RCHUNK * 4u;
    const uint32_t small = (uint32_t)((sizeof(Small) + 127) & ~127u);
    a.off_stage = 65536u + small;
    a.off_down = a.off_stage + ((stage_bytes + 127u) & ~127u);
    a.off_sh = a.off_down + ((max_dt * Q4B_TILE_BYTES + 127u) & ~127u);
    const size_t smem = (size_t)a.off_sh + 2u * MAX_SH * Q4B_TILE_BYTES + 1024;
    if (smem > 227u * 1024u) return false;
    if (!g_f_attr_set) {
        Q4B_CHECK(cudaFuncSetAttribute(moe_decode_fused_k, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       227 * 1024));
        Q4B_CHECK(cudaFuncSetAttribute(moe_decode_fused_xp_k, cudaFuncAttributeMaxDynamicSharedMemorySize,
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
    cudaError_t le;
    if (h_x_param) {
        static XRow xr;   // filled and consumed inside this call: the launch copies its parameters
        memcpy(xr.v, h_x_param, sizeof(xr.v));
        le = cudaLaunchKernelEx(&cfg, moe_decode_fused_xp_k, a, xr);
    } else {
        le = cudaLaunchKernelEx(&cfg, moe_decode_fused_k, a);
    }
    if (le != cudaSuccess) {
        fprintf(stderr, "q4cuda: fused decode launch failed: %s\n", cudaGetErrorString(cudaGetLastError()));
        return false;
    }
    g_q4b_launches++;
    return true;
}

// In-kernel phase profile of the persistent decode kernel (diagnostics).
// enable(1) allocates the stamp buffer (not inside a capture); read copies the
// stamps of the last launch: out[cta * 16 + slot] in nanoseconds of the GPU's
// global timer; returns the number of CTAs.
extern "C" bool q4_cuda_fused_profile_enable(int on) {
    if (!g_q4b.ok) return false;
    if (on && !g_f_prof) {
        Q4B_CHECK(cudaMalloc(&g_f_prof, (size_t)g_q4b.n_sm * 16 * sizeof(unsigned long long)));
        Q4B_CHECK(cudaMemset(g_f_prof, 0, (size_t)g_q4b.n_sm * 16 * sizeof(unsigned long long)));
    } else if (!on && g_f_prof) {
        cudaStreamSynchronize(g_q4b.stream);
        cudaFree(g_f_prof);
        g_f_prof = nullptr;
    }
    return true;
}
extern "C" uint32_t q4_cuda_fused_profile_read(unsigned long long *out, uint32_t max_ctas) {
    if (!g_q4b.ok || !g_f_prof || !out) return 0;
    const uint32_t n = max_ctas < (uint32_t)g_q4b.n_sm ? max_ctas : (uint32_t)g_q4b.n_sm;
    if (cudaMemcpyAsync(out, g_f_prof, (size_t)n * 16 * sizeof(unsigned long long),
                        cudaMemcpyDeviceToHost, g_q4b.stream) != cudaSuccess ||
        cudaStreamSynchronize(g_q4b.stream) != cudaSuccess)
        return 0;
    return n;
}
