// A stack of MoE layers for one token as ONE persistent kernel (one CTA per SM); the
// output row of a layer is the input row of the next.  One layer is the special case.
//
// Per layer, in every CTA:
//   phase 0  the token's row (layer 0: the caller's x; later: the previous layer's y, taken
//            from the exchange words), RMSNorm, Q8-A quantisation -- every CTA the same
//   phase 1  router: dots of this CTA's rows of the router matrix (fetched one layer
//            ahead; one warp per quarter row), published as exchange words, four partial
//            sums per expert; the shared expert's gate/up rows (also fetched ahead),
//            SwiGLU, published
//   phase 2  all logits from the exchange words; the top-k by LOGIT order (softmax is
//            monotone), and at once the bulk copies of this CTA's share of the picked
//            experts' gate/up tiles, then of its down tiles; while those fly: softmax, the
//            check that the probability order gives the same picks (src/q4_quant.c:715-755
//            picks on probabilities, ties to the lower index), the renormalised weights;
//            gate/up dots, SwiGLU, hidden values published
//   phase 3  all hidden values from the exchange words, Q8-A per expert, down tiles x hq,
//            weighted sum over the experts in list order, y published (last layer: written)
//
// There is no grid barrier.  A value travels between CTAs as one 64-bit word
// {fp32 value, 32-bit epoch} written with a single store and polled with single loads:
// a word whose epoch is the current layer's is complete by construction, so producers
// need no fence and consumers no flag.  Every value a layer publishes is consumed by
// every CTA before that CTA publishes anything of the next stage, which is what makes
// one set of words per stage enough (see the hazard notes at the three publish sites).
// Epochs come from a device counter of launches, so a CUDA graph that replays the same
// launch still gets fresh epochs.  Every poll is bounded: a poll that runs out sets an
// error bit (q4_cuda_device_error), and the kernel carries on with whatever it read;
// expert ids are clamped, so all addresses stay valid.
//
// Weight bytes cross HBM -> shared memory exactly once, by 1-D bulk async copies (plain
// cp.async.bulk into this CTA only) that complete on mbarriers.
// Replaces the reference's per-layer launch chain (src/q4_moe.c:2077-2133; kernels
// wmoe_iq3_gu_q8 / wmoe_iq3_ya_q8, src/q4_rocm.cu:3912-4120).  Needs the tiled arena
// format (q4b_tile.cuh), n_embd == 2048, n_ff == 512, n_expert <= 512, topk <= 15.
// 512 threads per CTA: at 768 the 80-register limit spilled inside the tile loops.
#include "q4b_tile.cuh"

#include <atomic>
#include <type_traits>
#include <chrono>

#include "../../include/q4cuda.h"

extern std::atomic<uint64_t> g_q4b_launches;
bool q4b_ptr_tiled(const void *p);

namespace stk {

constexpr uint32_t NT = 512;          // threads per CTA
constexpr uint32_t NW = NT / 32;      // warps
constexpr uint32_t H = 2048;          // n_embd
constexpr uint32_t F = 512;           // n_ff
constexpr uint32_t MAX_E = 16;        // experts per token incl. shared (more: the launch chain runs)
constexpr uint32_t UCHUNK = 8;        // gate/up units per bulk-copy chunk
constexpr uint32_t MAX_CHUNKS = 6;
constexpr uint32_t MAX_UNITS = 48;    // routed (expert, hidden unit) pairs per CTA
constexpr uint32_t MAX_SH = 8;        // shared-expert units per CTA
constexpr uint32_t MAX_DT = 72;       // down tiles per CTA
constexpr uint32_t MAX_RROWS = 4;     // router rows per CTA
constexpr uint32_t MAX_LAYERS = 64;   // layers per launch (epochs are spaced by this)
constexpr uint32_t MBAR_LIMIT = 1000000u;   // polls before an mbarrier wait gives up (or a third of a second)
constexpr uint32_t POLL_LIMIT = 400000u;    // default polls before an exchange-word wait gives up

// mbarrier slots
constexpr uint32_t MB_ROUTER = 0, MB_SHARED = 1, MB_DOWN = 2, MB_CHUNK0 = 3;
constexpr uint32_t N_MBAR = MB_CHUNK0 + MAX_CHUNKS;

// error word bits (1 and 2 keep their meaning from the mbarrier / grid waits of the other kernels)
constexpr uint32_t ERR_MBAR = 1u, ERR_POLL = 4u;
// session: doorbell value that ends it; commands CTA 0 hands to the other CTAs; flag bits the host sees
constexpr uint32_t BELL_STOP = 0xffffffffu;
constexpr uint32_t CMD_GO = 1u, CMD_END = 2u;
constexpr uint32_t FLAG_ERR = 0x80000000u, FLAG_EXIT = 0x40000000u;

struct Layer {
    const uint8_t *base;      // slot 0 of this layer's experts
    const float *norm_w;      // may be NULL
    const float *router;      // [n_expert][H]
    const float *sgate;       // [H] or NULL: the shared expert's weight is sigmoid(sgate . xn) instead of 1
};

struct Args {
    Layer l0;                 // the layer when layers == NULL
    const Layer *layers;      // device array of n_layers descriptors, or NULL
    uint32_t n_layers;
    uint64_t stride, og, ou, od;
    int32_t shared_slot;
    const float *x;
    const uint32_t *codes;    // 512 byte-expanded codebook words (device memory)
    float eps;
    uint32_t n_expert, topk;
    float *y;
    int32_t *ids_out;         // [n_layers][topk] or NULL
    float *wts_out;
    unsigned long long *xw;   // exchange words: [H] a layer's output row
    unsigned long long *lw;   //                 [NT][4] partial logits (permuted, see logit_pos)
    unsigned long long *hw;   //                 [MAX_E * F] hidden values
    unsigned long long *ctr;  // [0] CTA starts (launch number = value / grid), [1] CTA finishes of host hand-offs
    uint32_t *err;
    unsigned long long *prof; // optional [gridDim.x][16] phase time stamps (ns) of layer prof_layer, or NULL
    uint32_t prof_layer;
    float *y_host;            // optional: host-mapped copy of y, written by the last CTA to finish
    volatile uint32_t *flag_host; // host-mapped word that receives flag_val (bit 31: error word was set)
    uint32_t flag_val;
    uint32_t poll_limit;
    // optional epilogue of the last layer (src/q4_rocm.cu:15990-16003, moe_final): besides y, the
    // hc residual streams res[c][.] += y * 2 sigmoid(inject[c] / hc)
    float *res;
    const float *inject;
    uint32_t hc;
    // session form (moe_decode_session_k): the kernel stays resident and serves one step per ring
    // of a doorbell in host memory; a step runs lps consecutive layers of the plan (cyclically)
    const float *x_host;          // host-mapped input row [H] of the step
    const uint32_t *bell_host;    // host-mapped doorbell: the number of the step to run, or BELL_STOP
    unsigned long long *cw;       // exchange word that carries a step's command from CTA 0 to the others
    uint32_t lps;                 // layers per step
    uint32_t li0;                 // the plan's layer the first step starts with
    uint32_t max_steps;           // the kernel returns after this many steps
    unsigned long long idle_ns;   // ... or when no ring comes for this long
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
// Bounded wait: gives up after MBAR_LIMIT polls or a third of a second and records it.
__device__ __forceinline__ void mbar_wait(uint64_t *bar, uint32_t parity, uint32_t *err) {
    unsigned long long t0 = 0;
    for (uint32_t i = 0; i < MBAR_LIMIT; i++) {
        if (mbar_try_wait(bar, parity)) return;
        __nanosleep(40);
        if ((i & 1023u) == 1023u) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
            if (t0 == 0) t0 = t;
            else if (t - t0 > 300000000ull) break;
        }
    }
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

// ---- exchange words ----
__device__ __forceinline__ void xw_store(unsigned long long *p, float v, uint32_t ep) {
    const unsigned long long w = ((unsigned long long)ep << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
// Four consecutive words (32-byte aligned); bounded.  The loop polls without pausing: a pause
// between polls (nanosleep) cost a microsecond per layer, and so did polling several groups of
// a thread together until all had come or letting one lane per warp watch for the rest -- what
// counts is how soon after the store the first successful load is issued.  (A single first
// look at several groups before their poll loops does pay: see the hidden rows.)
__device__ __forceinline__ float4 xw_poll4(const unsigned long long *p, uint32_t ep, uint32_t limit,
                                           uint32_t *err) {
    unsigned long long a = 0, b = 0, c = 0, d = 0;
    uint32_t i = 0;
    for (; i < limit; i++) {
        asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
        asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(c), "=l"(d) : "l"(p + 2) : "memory");
        if ((uint32_t)(a >> 32) == ep && (uint32_t)(b >> 32) == ep && (uint32_t)(c >> 32) == ep &&
            (uint32_t)(d >> 32) == ep)
            break;
    }
    if (i == limit) atomicOr(err, ERR_POLL);
    return make_float4(__uint_as_float((uint32_t)a), __uint_as_float((uint32_t)b),
                       __uint_as_float((uint32_t)c), __uint_as_float((uint32_t)d));
}

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// One word whose wait may be long (a session between two rings): bounded by time, not by polls.
// Returns the word's value, or CMD_END (with the error bit set) when the time ran out.
__device__ __forceinline__ uint32_t xw_poll_timed(const unsigned long long *p, uint32_t ep, unsigned long long ns,
                                                  uint32_t *err) {
    const unsigned long long t0 = global_ns();
    for (uint32_t i = 0;; i++) {
        unsigned long long w;
        asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
        if ((uint32_t)(w >> 32) == ep) return (uint32_t)w;
        if ((i & 1023u) == 1023u) {
            if (global_ns() - t0 > ns) break;
            if (i > (1u << 17)) __nanosleep(200);   // idle for a tenth of a second already: poll less often
        }
    }
    atomicOr(err, ERR_POLL);
    return CMD_END;
}

// Phase time stamp for the optional in-kernel profile.
__device__ __forceinline__ void stamp(const Args &a, bool on, uint32_t slot) {
    if (on && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        a.prof[blockIdx.x * 16u + slot] = t;
    }
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
    uint32_t cmd;    // session: this step's command
    float fac[64];   // epilogue: the streams' factors
    uint32_t ep0;    // epoch of layer 0 of this launch
    uint64_t mbar[N_MBAR];
    alignas(16) float xn[H];            // normalised x (router input)
    alignas(16) uint32_t xq[H / 4];     // Q8-A of xn, int8x4 words
    float xd[H / 32];
    int xbs[H / 32];
    int32_t ids[MAX_E];                 // the layer's experts in the order they are computed in
    float wts[MAX_E];
    float psel[32];                     // probabilities of the picks
    uint32_t kv[32];                    // keys of the picks
    float red[NW];
    double redd[NW];
    uint32_t wmax[NW];                  // selection: per-warp largest key, candidates per warp
    uint32_t wcnt[NW];
    alignas(16) uint32_t hq[MAX_E][F / 4];  // Q8-A of the hidden rows
    float hd[MAX_E][F / 32];
    int hbs[MAX_E][F / 32];
    float part[MAX_DT][4];              // phase-3 partial sums: [tile][row in tile]
    uint32_t ck[NW][32];                // selection: candidates (key, index); general path: per-warp lists
    uint32_t ci[NW][32];
};

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

// Order-preserving map of a float to an unsigned key (larger float = larger key; never 0
// for a number).
__device__ __forceinline__ uint32_t float_key(float f) {
    const uint32_t u = __float_as_uint(__fadd_rn(f, 0.f));   // -0 -> +0
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// Thread tid of the selection owns expert lane * nwe + warp (nwe = warps that hold
// experts): neighbouring experts sit in different warps, so a run of popular experts does
// not pile its candidates into one warp.  logit_pos is the inverse: where the logit of
// expert e is published so that thread tid reads word tid.
__device__ __forceinline__ uint32_t logit_pos(uint32_t e, uint32_t nwe) {
    return (e % nwe) * 32u + e / nwe;
}

// The topk largest keys of the block (0 = no entry; equal keys: lower expert index first)
// -> S.ids[r] (clamped to [0, n_expert)), S.kv[r], r < topk, in order.  `ex` is this
// thread's expert index.  Ends with __syncthreads().
// Fast path: a threshold (the topk-th largest of the per-warp maxima) leaves a few
// candidates, which one warp ranks all against all.  More than 32 candidates (many equal
// keys, or topk above the number of warps): every warp extracts its ordered top-k with
// warp reductions and warp 0 merges the lists.
__device__ __forceinline__ void select_topk(uint32_t key, uint32_t ex, uint32_t topk,
                                            uint32_t n_expert, Small &S, uint32_t tid) {
    const uint32_t lane = tid & 31u, warp = tid >> 5;
    const uint32_t full = 0xffffffffu;
    const uint32_t wm = __reduce_max_sync(full, key);
    if (lane == 0) S.wmax[warp] = wm;
    __syncthreads();
    const uint32_t mv = lane < NW ? S.wmax[lane] : 0u;
    uint32_t rank = 0;
#pragma unroll
    for (uint32_t j = 0; j < NW; j++) {
        const uint32_t o = __shfl_sync(full, mv, j);
        rank += (o > mv || (o == mv && j < lane)) ? 1u : 0u;
    }
    const uint32_t tb = __ballot_sync(full, lane < NW && rank == topk - 1u);
    const uint32_t tau = tb ? __shfl_sync(full, mv, __ffs(tb) - 1) : 0u;
    const bool cand = key != 0u && key >= tau;
    const uint32_t cm = __ballot_sync(full, cand);
    if (lane == 0) S.wcnt[warp] = __popc(cm);
    __syncthreads();
    const uint32_t cv = lane < NW ? S.wcnt[lane] : 0u;
    uint32_t inc = cv;
#pragma unroll
    for (uint32_t o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(full, inc, o);
        if (lane >= o) inc += t;
    }
    const uint32_t total = __shfl_sync(full, inc, 31);
    const uint32_t off = __shfl_sync(full, inc - cv, warp);
    if (total <= 32u && total >= topk) {
        if (cand) {
            const uint32_t pos = off + __popc(cm & ((1u << lane) - 1u));
            S.ck[0][pos] = key;
            S.ci[0][pos] = ex;
        }
        __syncthreads();
        if (warp == 0) {
            const uint32_t k = lane < total ? S.ck[0][lane] : 0u;
            const uint32_t ix = lane < total ? S.ci[0][lane] : 0xffffffffu;
            uint32_t r = 0;
#pragma unroll
            for (uint32_t j = 0; j < 32; j++) {
                const uint32_t ok = __shfl_sync(full, k, j), oi = __shfl_sync(full, ix, j);
                r += (ok > k || (ok == k && oi < ix)) ? 1u : 0u;
            }
            if (lane < total && r < topk) {
                S.ids[r] = (int32_t)min(ix, n_expert - 1u);
                S.kv[r] = k;
            }
        }
        __syncthreads();
        return;
    }
    // ---- general path ----
    uint32_t k2 = key, my_key = 0u, my_idx = 0xffffffffu;
    if (wm != 0u) {
        for (uint32_t r = 0; r < topk; r++) {
            const uint32_t kmax = __reduce_max_sync(full, k2);
            const uint32_t imin = __reduce_min_sync(full, (k2 == kmax && kmax != 0u) ? ex : 0xffffffffu);
            if (lane == r) {
                my_key = kmax;
                my_idx = imin;
            }
            if (ex == imin) k2 = 0u;
        }
    }
    S.ck[warp][lane] = my_key;
    S.ci[warp][lane] = my_idx;
    __syncthreads();
    if (warp == 0) {
        uint32_t pos = 0;
        uint32_t hk = lane < NW ? S.ck[lane][0] : 0u;
        uint32_t hi = lane < NW ? S.ci[lane][0] : 0xffffffffu;
        for (uint32_t t = 0; t < topk; t++) {
            const uint32_t kmax = __reduce_max_sync(full, hk);
            const uint32_t imin = __reduce_min_sync(full, hk == kmax ? hi : 0xffffffffu);
            if (hk == kmax && hi == imin) {  // this lane's list head was taken
                pos++;
                hk = pos < 32u ? S.ck[lane][pos] : 0u;
                hi = pos < 32u ? S.ci[lane][pos] : 0xffffffffu;
            }
            if (lane == t) {
                S.ids[t] = (int32_t)min(imin, n_expert - 1u);
                S.kv[t] = kmax;
            }
        }
    }
    __syncthreads();
}

// Bulk copies of this CTA's routed gate/up tiles: unit u = e * F + f; chunk k covers units
// [u0 + k*UCHUNK, ...), staged at stage + k * UCHUNK * 2 * 880 as gate tiles then up tiles.
// One warp per chunk issues (lane 0).
__device__ __forceinline__ void issue_gate_up(const Args &a, const Layer &L, Small &S, uint8_t *stage,
                                              uint32_t u0, uint32_t u1, uint32_t n_chunks,
                                              uint32_t warp, uint32_t lane) {
    if (warp < n_chunks && lane == 0) {
        const uint32_t k = warp;
        const uint32_t ua = u0 + k * UCHUNK, ub = min(ua + UCHUNK, u1);
        uint8_t *dst = stage + (size_t)k * UCHUNK * 2u * Q4B_TILE_BYTES;
        mbar_expect_tx(&S.mbar[MB_CHUNK0 + k], (ub - ua) * 2u * Q4B_TILE_BYTES);
        uint32_t u = ua;
        while (u < ub) {  // a chunk may straddle two experts: one copy per expert's run
            const uint32_t e = u / F, f = u - e * F;
            const uint32_t run = min(ub - u, F - f);
            const uint8_t *pk = L.base + (uint64_t)S.ids[e] * a.stride;
            bulk_g2s(dst + (size_t)(u - ua) * Q4B_TILE_BYTES, pk + a.og + (size_t)f * Q4B_TILE_BYTES,
                     run * Q4B_TILE_BYTES, &S.mbar[MB_CHUNK0 + k]);
            bulk_g2s(dst + (size_t)(UCHUNK + (u - ua)) * Q4B_TILE_BYTES,
                     pk + a.ou + (size_t)f * Q4B_TILE_BYTES, run * Q4B_TILE_BYTES,
                     &S.mbar[MB_CHUNK0 + k]);
            u += run;
        }
    }
}

// Bulk copies of this CTA's down tiles: its row quads of one expert lie back to back in the pack,
// so one copy per expert, staged expert by expert (tile (row quad rq, expert e) at slot
// e * nrq + rq - rq0).  Many small copies cost more to issue than they take to arrive.
__device__ __forceinline__ void issue_down(const Args &a, const Layer &L, Small &S, uint8_t *dstage,
                                           uint32_t v0, uint32_t v1, uint32_t ne, uint32_t tid) {
    if (tid >= (NW - 1) * 32 && v1 > v0) {
        const uint32_t e = tid - (NW - 1) * 32;
        const uint32_t rq0 = v0 / ne, nrq = (v1 - v0) / ne;
        if (e == 0) mbar_expect_tx(&S.mbar[MB_DOWN], (v1 - v0) * Q4B_TILE_BYTES);
        __syncwarp();
        if (e < ne)
            bulk_g2s(dstage + (size_t)e * nrq * Q4B_TILE_BYTES,
                     L.base + (uint64_t)S.ids[e] * a.stride + a.od + (size_t)rq0 * Q4B_TILE_BYTES,
                     nrq * Q4B_TILE_BYTES, &S.mbar[MB_DOWN]);
    }
}

// The kernel body; xrow is the token's hidden row as H/4 float4: device memory for the
// device-pointer call, the kernel's own parameter block for the host-buffer call.
template <bool SESSION, bool XPARAM = false>
__device__ __forceinline__ void stack_body(const Args &a, const float4 *xrow) {
    // used directly (no integer round trip), so that the compiler keeps these as
    // shared-space accesses; dynamic shared memory starts on the declared alignment
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *sm = smem_raw;
    uint32_t *tab = reinterpret_cast<uint32_t *>(sm);
    Small &S = *reinterpret_cast<Small *>(sm + 65536);
    uint8_t *stage = sm + a.off_stage;  // router rows, then routed gate/up tiles
    uint8_t *dstage = sm + a.off_down;  // down tiles
    uint8_t *sstage = sm + a.off_sh;    // shared-expert gate/up tiles
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t cta = blockIdx.x, ncta = gridDim.x;
    const bool has_sh = a.shared_slot >= 0;
    const uint32_t ne = a.topk + (has_sh ? 1u : 0u);
    const uint32_t nwe = (a.n_expert + 31u) / 32u;       // warps that hold experts in the selection
    const uint32_t ex = lane * nwe + warp;               // this thread's expert in the selection
    const bool ex_ok = warp < nwe && ex < a.n_expert;
    const uint32_t limit = a.poll_limit;

    // ---- work split (the same in every layer) ----
    const uint32_t r0 = (uint32_t)((uint64_t)cta * a.n_expert / ncta);        // router rows
    const uint32_t r1 = (uint32_t)((uint64_t)(cta + 1) * a.n_expert / ncta);
    const uint32_t n_units = a.topk * F;  // routed (expert, hidden unit) pairs
    const uint32_t u0 = (uint32_t)((uint64_t)cta * n_units / ncta);
    const uint32_t u1 = (uint32_t)((uint64_t)(cta + 1) * n_units / ncta);
    const uint32_t n_chunks = (u1 - u0 + UCHUNK - 1) / UCHUNK;
    const uint32_t s0 = has_sh ? (uint32_t)((uint64_t)cta * F / ncta) : 0u;  // shared-expert units
    const uint32_t s1 = has_sh ? (uint32_t)((uint64_t)(cta + 1) * F / ncta) : 0u;
    const bool sh_split = 2u * (s1 - s0) <= NW;   // few shared units: one tile per warp
    // down tiles = (row quad, expert) pairs, expert fastest; a CTA takes whole row quads, so every
    // output row is summed over the experts by one CTA, in list order, and written once
    const uint32_t v0 = (uint32_t)((uint64_t)cta * (H / 4) / ncta) * ne;
    const uint32_t v1 = (uint32_t)((uint64_t)(cta + 1) * (H / 4) / ncta) * ne;

    // loads with nothing before them in the dependency chain go first
    Layer cur = a.layers ? a.layers[SESSION ? a.li0 : 0u] : a.l0;
    float4 xv = make_float4(0.f, 0.f, 0.f, 0.f), wv = make_float4(1.f, 1.f, 1.f, 1.f);
    uint32_t code = 0;
    if (tid < H / 4) {
        if constexpr (XPARAM) {
            // The row sits in the parameter block (constant bank): a warp whose lanes ask for 32
            // different addresses is served one address at a time, each a miss of the constant
            // cache (measured: 6 us).  So the warp reads its 32 entries one by one, every lane
            // the same address, and lane i keeps entry i.
#pragma unroll 8
            for (uint32_t i = 0; i < 32; i++) {
                const float4 t = xrow[(tid & ~31u) + i];
                if ((tid & 31u) == i) xv = t;
            }
        } else if constexpr (!SESSION) {
            xv = xrow[tid];
        }
        if (cur.norm_w) wv = reinterpret_cast<const float4 *>(cur.norm_w)[tid];
        code = a.codes[tid];
    }
    if (tid == 0) {
        for (uint32_t i = 0; i < N_MBAR; i++) mbar_init(&S.mbar[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (a.res && tid >= 64 && tid - 64 < a.hc) S.fac[tid - 64] = hc_stream_factor(a.inject, 0, a.hc, tid - 64);
    if (tid < MAX_E) {   // entry topk of the expert list is the shared expert, in every layer
        S.ids[tid] = (has_sh && tid == a.topk) ? a.shared_slot : 0;
        S.wts[tid] = 1.0f;
    }
    __syncthreads();
    if (tid == 0 && r1 > r0) {  // router rows: contiguous in memory
        const uint32_t bytes = (r1 - r0) * H * 4u;
        mbar_expect_tx(&S.mbar[MB_ROUTER], bytes);
        bulk_g2s(stage, cur.router + (size_t)r0 * H, bytes, &S.mbar[MB_ROUTER]);
    }
    if (tid == 32 && s1 > s0) {   // shared expert: gate tiles then up tiles of units [s0, s1)
        const uint32_t bytes = (s1 - s0) * Q4B_TILE_BYTES;
        const uint8_t *pk = cur.base + (uint64_t)a.shared_slot * a.stride;
        mbar_expect_tx(&S.mbar[MB_SHARED], 2u * bytes);
        bulk_g2s(sstage, pk + a.og + (size_t)s0 * Q4B_TILE_BYTES, bytes, &S.mbar[MB_SHARED]);
        bulk_g2s(sstage + (size_t)MAX_SH * Q4B_TILE_BYTES, pk + a.ou + (size_t)s0 * Q4B_TILE_BYTES,
                 bytes, &S.mbar[MB_SHARED]);
    }
    if (tid == 64) {
        // launch number: every CTA of every launch adds one, launches on the library's stream
        // do not overlap, so old / grid is the same in all CTAs of a launch
        const unsigned long long old = atomicAdd(a.ctr, 1ull);
        S.ep0 = (uint32_t)(((old / ncta) * MAX_LAYERS) % 0xffffffffull) + 1u;   // never 0
    }
    // code table: entry i replicated once per lane: thread t < 512 holds entry t, a warp
    // broadcasts its 32 entries one by one
    if (tid < 512) {
#pragma unroll 8
        for (uint32_t i = 0; i < 32; i++) {
            const uint32_t v = __shfl_sync(0xffffffffu, code, i);
            tab[(warp * 32u + i) * 32u + lane] = v;
        }
    }
    const uint32_t *tl = tab + lane;
    uint32_t par = 0;        // parity of the once-per-layer mbarriers
    uint32_t par_chunk = 0;  // parity of the mbarriers armed once per selection: gate/up chunks, down tiles

    uint32_t li = SESSION ? a.li0 : 0u;   // index of `cur` among the plan's layers
    uint32_t step = 0;   // session: steps served so far
    if constexpr (SESSION) __syncthreads();   // S.ep0
    for (;;) {           // one pass; a session: one pass per ring of the doorbell
    uint32_t epb = 0;    // this pass's first layer epoch, relative to S.ep0
    if constexpr (SESSION) {
        // A step owns MAX_LAYERS epochs: the first for its input row and command, the rest for its layers.
        epb = step * MAX_LAYERS + 1u;
        uint32_t ep_in = S.ep0 + step * MAX_LAYERS;
        if (ep_in < S.ep0) ep_in += 1u;
        if (cta == 0) {
            // CTA 0 watches the doorbell (reads of host memory: a microsecond or two each), fetches
            // the row from host memory and hands row and command to the other CTAs as exchange words.
            // One watcher: eight of them (to see a ring sooner) made a step 15 us slower.
            if (tid == 0) {
                uint32_t cmd = CMD_END;
                const unsigned long long t0 = global_ns();
                for (;;) {
                    uint32_t b;
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(b) : "l"(a.bell_host) : "memory");
                    if (b == step + 1u) {
                        cmd = CMD_GO;
                        break;
                    }
                    if (b == BELL_STOP || global_ns() - t0 > a.idle_ns) break;
                }
                S.cmd = cmd;
            }
            __syncthreads();
            if (tid < H / 4) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (S.cmd == CMD_GO)
                    asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                                 : "l"(reinterpret_cast<const float4 *>(a.x_host) + tid)
                                 : "memory");
                // read by every CTA right below; written again only after the host has seen this
                // step's result, i.e. after every CTA finished the step
                xw_store(a.xw + 4u * tid, v.x, ep_in);
                xw_store(a.xw + 4u * tid + 1, v.y, ep_in);
                xw_store(a.xw + 4u * tid + 2, v.z, ep_in);
                xw_store(a.xw + 4u * tid + 3, v.w, ep_in);
                xv = v;
            }
            if (tid == 0) {
                xw_store(a.cw, __uint_as_float(S.cmd), ep_in);
                // leaving without having been told to: the host must not wait for a result
                if (S.cmd != CMD_GO) *a.flag_host = FLAG_EXIT;
            }
        } else {
            // One thread per CTA watches one command word, then the CTA reads the row.  Letting all
            // threads watch their own words of the row instead (one hop less) measured 0.8 us slower
            // per step: 75,000 pollers delay the very stores they wait for.
            if (tid == 0) S.cmd = xw_poll_timed(a.cw, ep_in, a.idle_ns + 1000000000ull, a.err);
            __syncthreads();
            if (S.cmd == CMD_GO && tid < H / 4) xv = xw_poll4(a.xw + 4u * tid, ep_in, limit, a.err);
        }
        if (S.cmd != CMD_GO) break;
    }
    const uint32_t n_run = SESSION ? a.lps : a.n_layers;
    for (uint32_t l = 0; l < n_run; l++) {
        const bool prof = a.prof && li == a.prof_layer;
        const bool out = l + 1 == n_run;      // the pass's last layer: its y leaves the kernel
        const bool more = SESSION || !out;    // some layer follows (a session: the next step's first)
        const uint32_t nli = li + 1 < a.n_layers ? li + 1 : 0u;
        Layer nxt = cur;
        if (more && a.layers) nxt = a.layers[nli];
        stamp(a, prof, 0);
        // ---- phase 0: RMSNorm, Q8-A ----
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
                if (cur.norm_w) {
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
        stamp(a, prof, 1);
        uint32_t ep = S.ep0 + epb + l;      // this layer's epoch (skips 0 on wrap-around)
        if (ep < S.ep0) ep += 1u;

        // ---- phase 1: router rows x xn, one warp per quarter row ----
        if (r1 > r0) mbar_wait(&S.mbar[MB_ROUTER], par, a.err);
        stamp(a, prof, 2);
#pragma unroll 1
        for (uint32_t c = warp; c < 4u * (r1 - r0); c += NW) {
            const uint32_t rl = c >> 2, part = c & 3u;
            const float4 *w4 = reinterpret_cast<const float4 *>(stage + ((size_t)rl * H + part * (H / 4)) * 4u);
            const float4 *x4 = reinterpret_cast<const float4 *>(S.xn + part * (H / 4));
            float acc = 0.f;
#pragma unroll
            for (uint32_t i = 0; i < H / 4 / 128; i++) {
                const float4 rw = w4[lane + 32 * i], rx = x4[lane + 32 * i];
                acc += rw.x * rx.x + rw.y * rx.y + rw.z * rx.z + rw.w * rx.w;
            }
            acc = q4b_warp_sum(acc);
            // logits (four partial sums per expert): written here, read by every CTA in phase 2 of
            // this layer; a CTA reaches this line for the next layer only after all CTAs published
            // this layer's y, i.e. after they all finished reading these words
            if (lane == 0) xw_store(a.lw + 4u * logit_pos(r0 + rl, nwe) + part, acc, ep);
        }
        // the shared expert's gate (src/q4_moe.c:1404-1435, sgate): its weight in this layer's sum.
        // On a warp that has a router task only; read in phase 3, block barriers lie between.
        if (has_sh && warp == 4) {
            float g = 1.0f;
            if (cur.sgate) {
                const float4 *g4 = reinterpret_cast<const float4 *>(cur.sgate);
                const float4 *x4 = reinterpret_cast<const float4 *>(S.xn);
                float acc = 0.f;
#pragma unroll 4
                for (uint32_t i = lane; i < H / 4; i += 32) {
                    const float4 gw = __ldg(g4 + i), gx = x4[i];
                    acc += gw.x * gx.x + gw.y * gx.y + gw.z * gx.z + gw.w * gx.w;
                }
                acc = q4b_warp_sum(acc);
                g = 1.f / (1.f + expf(-acc));
            }
            if (lane == 0) S.wts[a.topk] = g;
        }
        stamp(a, prof, 3);

        // activations of this lane's 64 columns (lane l of a gate/up tile owns columns 64 l ..)
        int q[16];
#pragma unroll
        for (int i = 0; i < 16; i++) q[i] = (int)S.xq[16u * lane + i];
        const float dx0 = S.xd[2u * lane], dx1 = S.xd[2u * lane + 1];
        const int bs0 = S.xbs[2u * lane], bs1 = S.xbs[2u * lane + 1];

        // ---- the shared expert's gate/up rows (its tiles were fetched a layer ahead) ----
        if (s1 > s0) {
            mbar_wait(&S.mbar[MB_SHARED], par, a.err);
            // One warp per hidden unit: its gate tile and its up tile back to back (two independent
            // instruction streams), both sums, SwiGLU, and the value goes out at once.  On the
            // last warps: the first ones hold the router rows, the two run side by side.
            // Hidden values: written here and after the routed dots, read by every CTA in phase 3
            // of this layer; a CTA reaches these lines for the next layer only after all CTAs
            // published this layer's y, i.e. after they all finished reading these words.
            if (sh_split) {
                // few units: gate tile and up tile on different warps, the two sums meet after the barrier
                const uint32_t wv = NW - 1u - warp;
                if (wv < 2u * (s1 - s0)) {
                    float x = q4b_tile_lane_dot(sstage + (size_t)((wv & 1u) * MAX_SH + (wv >> 1)) * Q4B_TILE_BYTES, lane,
                                                tl, q, dx0, dx1, bs0, bs1);
#pragma unroll
                    for (int o = 16; o; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
                    if (lane == 0) S.red[wv] = x;   // free until this layer's softmax sum
                }
            } else {
                for (uint32_t ul = NW - 1u - warp; ul < s1 - s0; ul += NW) {
                    const uint8_t *tile = sstage + (size_t)ul * Q4B_TILE_BYTES;
                    float g = q4b_tile_lane_dot(tile, lane, tl, q, dx0, dx1, bs0, bs1);
                    float u = q4b_tile_lane_dot(tile + (size_t)MAX_SH * Q4B_TILE_BYTES, lane, tl, q, dx0, dx1, bs0,
                                                bs1);
#pragma unroll
                    for (int o = 16; o; o >>= 1) {
                        g += __shfl_xor_sync(0xffffffffu, g, o);
                        u += __shfl_xor_sync(0xffffffffu, u, o);
                    }
                    if (lane == 0) xw_store(a.hw + a.topk * F + s0 + ul, q4b_swiglu(g, u), ep);
                }
            }
        }
        __syncthreads();   // every warp is done with the router rows and the shared tiles
        if (sh_split && tid < s1 - s0)
            xw_store(a.hw + a.topk * F + s0 + tid, q4b_swiglu(S.red[2u * tid], S.red[2u * tid + 1u]), ep);
        if (tid == 32 && more && s1 > s0) {   // next layer's shared-expert tiles
            const uint32_t bytes = (s1 - s0) * Q4B_TILE_BYTES;
            const uint8_t *pk = nxt.base + (uint64_t)a.shared_slot * a.stride;
            mbar_expect_tx(&S.mbar[MB_SHARED], 2u * bytes);
            bulk_g2s(sstage, pk + a.og + (size_t)s0 * Q4B_TILE_BYTES, bytes, &S.mbar[MB_SHARED]);
            bulk_g2s(sstage + (size_t)MAX_SH * Q4B_TILE_BYTES, pk + a.ou + (size_t)s0 * Q4B_TILE_BYTES,
                     bytes, &S.mbar[MB_SHARED]);
        }
        stamp(a, prof, 4);

        // ---- phase 2a: the logits, top-k by logit order ----
        float lg = 0.f;
        uint32_t key = 0u;
        if (ex_ok) {
            const float4 pp = xw_poll4(a.lw + 4u * tid, ep, limit, a.err);
            lg = (pp.x + pp.y) + (pp.z + pp.w);
            key = float_key(lg);
        }
        stamp(a, prof, 5);
        select_topk(key, ex, a.topk, a.n_expert, S, tid);
        stamp(a, prof, 6);
        // ---- phase 2b: fetch this CTA's routed gate/up tiles ----
        issue_gate_up(a, cur, S, stage, u0, u1, n_chunks, warp, lane);
        // ---- softmax, weights, and the check of the pick order (the copies are in flight) ----
        {
            const float m = key_float(S.kv[0]);
            const float e = ex_ok ? expf(lg - m) : 0.f;
            const float s = block_reduce_sum(e, S.red);
            // the down tiles, behind the gate/up tiles in the copy queues (a block barrier lies
            // between the two issues); they are needed in phase 3
            issue_down(a, cur, S, dstage, v0, v1, ne, tid);
            const float inv = s > 0.f ? __fdiv_rn(1.0f, s) : 0.f;
            const float p = __fmul_rn(e, inv);
            bool first = true;
            for (;;) {
                int myr = -1;
                if (ex_ok)
                    for (uint32_t r = 0; r < a.topk; r++)
                        if ((uint32_t)S.ids[r] == ex) myr = (int)r;
                if (myr >= 0) S.psel[myr] = p;
                __syncthreads();
                // the reference picks on probabilities: an expert that was not picked but whose
                // probability is not below the last pick's (two logits that round to one
                // probability) may be the reference's pick.  Rare: pick again, on probabilities.
                const int bad = first && ex_ok && myr < 0 && p >= S.psel[a.topk - 1u];
                if (!__syncthreads_or(bad)) break;
                first = false;
                if (warp < n_chunks) mbar_wait(&S.mbar[MB_CHUNK0 + warp], par_chunk, a.err);
                if (warp == NW - 1) mbar_wait(&S.mbar[MB_DOWN], par_chunk, a.err);
                par_chunk ^= 1u;
                select_topk(ex_ok ? __float_as_uint(p) + 1u : 0u, ex, a.topk, a.n_expert, S, tid);
                issue_gate_up(a, cur, S, stage, u0, u1, n_chunks, warp, lane);
                __syncthreads();
                issue_down(a, cur, S, dstage, v0, v1, ne, tid);
            }
            if (warp == 0) {
                const float pr = lane < a.topk ? S.psel[lane] : 0.f;
                float wsum = 0.f;
                for (uint32_t r = 0; r < a.topk; r++) wsum = __fadd_rn(wsum, __shfl_sync(0xffffffffu, pr, r));
                const float w = wsum > 0.f ? __fmul_rn(pr, __fdiv_rn(1.0f, wsum)) : pr;
                const uint32_t id = lane < a.topk ? (uint32_t)S.ids[lane] : 0xffffffffu;
                if (lane < a.topk) S.wts[lane] = w;
                if (cta == 0 && (a.ids_out || a.wts_out)) {
                    // reported in the reference's order: probability, then index
                    uint32_t rr = 0;
                    for (uint32_t j = 0; j < a.topk; j++) {
                        const float pj = __shfl_sync(0xffffffffu, pr, j);
                        const uint32_t ij = __shfl_sync(0xffffffffu, id, j);
                        rr += (pj > pr || (pj == pr && ij < id)) ? 1u : 0u;
                    }
                    if (lane < a.topk) {
                        if (a.ids_out) a.ids_out[l * a.topk + rr] = (int32_t)id;
                        if (a.wts_out) a.wts_out[l * a.topk + rr] = w;
                    }
                }
            }
        }
        stamp(a, prof, 7);
        // ---- phase 2c: routed hidden units (gate and up tile of a unit by one warp), SwiGLU ----
        // The units beyond the last full round of NW: when they are few, their gate tiles and up tiles
        // go to different warps (one more tile for 2 n_tail warps instead of one more unit-long round
        // with n_tail warps at work) and meet after the block barrier below.
        const uint32_t n_u = u1 - u0;
        const uint32_t n_tail = (n_u >= NW && 2u * (n_u % NW) <= NW) ? n_u % NW : 0u;
        const uint32_t n_pair = n_u - n_tail;
        auto gu_tile = [&](uint32_t ul, uint32_t up) {
            const uint32_t k = ul / UCHUNK, j = ul - k * UCHUNK;
            return stage + ((size_t)k * UCHUNK * 2u + (up ? UCHUNK : 0u) + j) * Q4B_TILE_BYTES;
        };
#pragma unroll 1
        for (uint32_t ul = warp; ul < n_pair; ul += NW) {
            mbar_wait(&S.mbar[MB_CHUNK0 + ul / UCHUNK], par_chunk, a.err);
            float g = q4b_tile_lane_dot(gu_tile(ul, 0), lane, tl, q, dx0, dx1, bs0, bs1);
            float u = q4b_tile_lane_dot(gu_tile(ul, 1), lane, tl, q, dx0, dx1, bs0, bs1);
#pragma unroll
            for (int o = 16; o; o >>= 1) {
                g += __shfl_xor_sync(0xffffffffu, g, o);
                u += __shfl_xor_sync(0xffffffffu, u, o);
            }
            if (lane == 0) xw_store(a.hw + u0 + ul, q4b_swiglu(g, u), ep);
        }
        if (warp < 2u * n_tail) {
            const uint32_t ul = n_pair + (warp >> 1);
            mbar_wait(&S.mbar[MB_CHUNK0 + ul / UCHUNK], par_chunk, a.err);
            float x = q4b_tile_lane_dot(gu_tile(ul, warp & 1u), lane, tl, q, dx0, dx1, bs0, bs1);
#pragma unroll
            for (int o = 16; o; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
            if (lane == 0) S.red[warp] = x;   // free between the softmax sums of two layers
        }
        __syncthreads();   // every warp is done with the gate/up tiles
        if (tid < n_tail)
            xw_store(a.hw + u0 + n_pair + tid, q4b_swiglu(S.red[2u * tid], S.red[2u * tid + 1u]), ep);
        if (tid == 0 && more && r1 > r0) {   // next layer's router rows
            const uint32_t bytes = (r1 - r0) * H * 4u;
            mbar_expect_tx(&S.mbar[MB_ROUTER], bytes);
            bulk_g2s(stage, nxt.router + (size_t)r0 * H, bytes, &S.mbar[MB_ROUTER]);
        }
        if (more && tid < H / 4)    // next layer's norm weights: needed right after its row arrives
            wv = nxt.norm_w ? __ldg(reinterpret_cast<const float4 *>(nxt.norm_w) + tid)
                            : make_float4(1.f, 1.f, 1.f, 1.f);
        stamp(a, prof, 8);

        // ---- phase 3a: the hidden rows (all experts), Q8-A; 8 lanes per group ----
        {
            constexpr uint32_t HQ_IT = (MAX_E * (F / 4) + NT - 1) / NT;
            // First look at all of a thread's groups with the loads in flight together; the poll loop then
            // only takes the groups that had not arrived.
            unsigned long long hw_[HQ_IT][4];
#pragma unroll
            for (uint32_t it = 0; it < HQ_IT; it++) {
                const uint32_t w4 = tid + it * NT;
                if (w4 < ne * (F / 4)) {
                    const unsigned long long *p = a.hw + 4u * w4;
                    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];"
                                 : "=l"(hw_[it][0]), "=l"(hw_[it][1]) : "l"(p) : "memory");
                    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];"
                                 : "=l"(hw_[it][2]), "=l"(hw_[it][3]) : "l"(p + 2) : "memory");
                }
            }
#pragma unroll
            for (uint32_t it = 0; it < HQ_IT; it++) {
                const uint32_t w4 = tid + it * NT;
                if (w4 < ne * (F / 4)) {  // warp-uniform: ne * F / 4 is a multiple of 32
                    float4 hv;
                    if ((uint32_t)(hw_[it][0] >> 32) == ep && (uint32_t)(hw_[it][1] >> 32) == ep &&
                        (uint32_t)(hw_[it][2] >> 32) == ep && (uint32_t)(hw_[it][3] >> 32) == ep)
                        hv = make_float4(__uint_as_float((uint32_t)hw_[it][0]), __uint_as_float((uint32_t)hw_[it][1]),
                                         __uint_as_float((uint32_t)hw_[it][2]), __uint_as_float((uint32_t)hw_[it][3]));
                    else
                        hv = xw_poll4(a.hw + 4u * w4, ep, limit, a.err);
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
            }
        }
        __syncthreads();
        stamp(a, prof, 9);

        // ---- phase 3b: down tiles; tile = 4 rows x 2 blocks; lane: block l/4 -> row l/8, half (l/4)&1 ----
        mbar_wait(&S.mbar[MB_DOWN], par_chunk, a.err);
        stamp(a, prof, 10);
        {
            const uint32_t col16 = 16u * (lane & 7u);  // first activation word of this lane's 64 columns
            const uint32_t g0 = 2u * (lane & 7u);
            // A warp task: up to DK row quads of one expert.  The expert's activation words are
            // loaded once for the task, and the DK tile dots are independent instruction streams for
            // the scheduler to interleave (a lone tile dot is a chain of dependent shared-memory
            // lookups).  DK = 3 or 4: with 148 CTAs a CTA holds 3 or 4 row quads.
            const uint32_t nrq = (v1 - v0) / ne;
            auto down_tasks = [&](auto dk_tag) {
                constexpr uint32_t DK = decltype(dk_tag)::value;
                const uint32_t ngr = (nrq + DK - 1u) / DK;   // tasks per expert
#pragma unroll 1
                for (uint32_t task = warp; task < ne * ngr; task += NW) {
                    const uint32_t gq = task / ne, e = task - gq * ne;
                    const uint32_t q0 = gq * DK;
                    int hqr[16];
#pragma unroll
                    for (int c = 0; c < 16; c += 4) {
                        const uint4 t4 = *reinterpret_cast<const uint4 *>(&S.hq[e][col16 + c]);
                        hqr[c] = (int)t4.x;
                        hqr[c + 1] = (int)t4.y;
                        hqr[c + 2] = (int)t4.z;
                        hqr[c + 3] = (int)t4.w;
                    }
                    const float hd0 = S.hd[e][g0], hd1 = S.hd[e][g0 + 1];
                    const int hb0 = S.hbs[e][g0], hb1 = S.hbs[e][g0 + 1];
                    float r[DK];
#pragma unroll
                    for (uint32_t i = 0; i < DK; i++) {
                        const uint32_t rql = min(q0 + i, nrq - 1u);   // past the end: the last tile again, not stored
                        r[i] = q4b_tile_lane_dot(dstage + (size_t)(e * nrq + rql) * Q4B_TILE_BYTES, lane, tl, hqr,
                                                 hd0, hd1, hb0, hb1);
                    }
#pragma unroll
                    for (int o = 1; o < 8; o <<= 1) {
#pragma unroll
                        for (uint32_t i = 0; i < DK; i++) r[i] += __shfl_xor_sync(0xffffffffu, r[i], o);
                    }
                    if ((lane & 7u) == 0) {
                        const float w = S.wts[e];
#pragma unroll
                        for (uint32_t i = 0; i < DK; i++)
                            if (q0 + i < nrq) S.part[(q0 + i) * ne + e][lane >> 3] = w * r[i];
                    }
                }
            };
            if (nrq % 4u == 0u)
                down_tasks(std::integral_constant<uint32_t, 4>{});
            else
                down_tasks(std::integral_constant<uint32_t, 3>{});
        }
        __syncthreads();
        stamp(a, prof, 11);
        // combine over the experts in list order
        for (uint32_t t = tid; t < ((v1 - v0) / ne) * 4u; t += NT) {
            const uint32_t ql = t >> 2, row = t & 3u;
            float sum = 0.f;
            for (uint32_t e = 0; e < ne; e++) sum += S.part[ql * ne + e][row];
            const uint32_t r = (v0 / ne + ql) * 4u + row;
            // the layer's output row: written here, read by every CTA at the top of the next
            // layer; a CTA reaches this line for the next layer only after all CTAs published
            // that layer's hidden values, i.e. after they all read these words
            if (!out) {
                xw_store(a.xw + r, sum, ep);
            } else {
                a.y[r] = sum;
                if (a.y_host) a.y_host[r] = sum;   // straight into the caller's mapped host row (see the hand-off)
                if (a.res)
                    for (uint32_t c = 0; c < a.hc; c++)
                        a.res[(size_t)c * H + r] = __fmaf_rn(sum, S.fac[c], a.res[(size_t)c * H + r]);
            }
        }
        stamp(a, prof, 12);
        if (!out && tid < H / 4) xv = xw_poll4(a.xw + 4u * tid, ep, limit, a.err);
        if (more) {
            cur = nxt;
            li = nli;
            par ^= 1u;
        }
        par_chunk ^= 1u;
    }
    // Host hand-off (the call with host buffers): every CTA has written its rows of y straight into
    // the caller's pinned, mapped host row (posted writes, as soon as the rows were summed), fences at
    // GPU scope and counts itself; the CTA that finishes last fences once at system scope -- the
    // fence is cumulative over what it has observed through the counter -- and raises the flag the
    // host is spinning on.  No copy node, no stream wake-up, one system-scope fence (148 of them, one
    // per CTA, measured slower; so did a copy of the whole row by the last CTA: one more L2 round trip).
    if (a.y_host) {
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const unsigned long long old = atomicAdd(a.ctr + 1, 1ull);
            S.last = (old % ncta) == ncta - 1ull ? 1u : 0u;
        }
        __syncthreads();
        if (S.last) {
            if (tid == 0) {
                __threadfence_system();
                uint32_t ew;
                asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(ew) : "l"(a.err) : "memory");
                *a.flag_host = (a.flag_val + step) | (ew ? FLAG_ERR : 0u);   // every writer fenced at system scope above
            }
            stamp(a, a.prof != nullptr, 15);   // in the last CTA only: when the flag was written
        }
    }
    if constexpr (!SESSION) break;
    step++;
    if (step >= a.max_steps) break;
    }
    if constexpr (SESSION) {
        // the epochs this launch used: later launches start beyond them (every CTA adds the same)
        if (tid == 64) atomicAdd(a.ctr, (unsigned long long)(step + 1u));
    }
}

__global__ void __launch_bounds__(NT, 1) moe_decode_stack_k(const Args a) {
    stack_body<false>(a, reinterpret_cast<const float4 *>(a.x));
}
__global__ void __launch_bounds__(NT, 1) moe_decode_session_k(const Args a) {
    stack_body<true>(a, nullptr);
}

// The host-buffer form: the 8 KB hidden row travels inside the launch's parameter block, so
// the call needs no separate host-to-device copy ahead of the kernel.
struct XRow {
    float4 v[H / 4];
};
__global__ void __launch_bounds__(NT, 1) moe_decode_stack_xp_k(const Args a, const __grid_constant__ XRow xr) {
    stack_body<false, true>(a, xr.v);
}

}  // namespace stk

// Scratch of the kernel (allocated once, by init / scratch_warm).
static unsigned long long *g_s_words = nullptr;   // xw | lw | hw
static unsigned long long *g_s_ctr = nullptr;
static bool g_s_attr_set = false;
static unsigned long long *g_s_prof = nullptr;  // set by q4_cuda_fused_profile_enable(1)
static uint32_t g_s_prof_layer = 0;
static uint32_t g_s_poll_limit = stk::POLL_LIMIT;
static struct Q4bSession *g_s_session = nullptr;   // the live session, if any (its kernel owns the GPU)

static bool stack_scratch() {
    if (g_s_ctr) return true;
    const size_t words = (size_t)stk::H + 4u * stk::NT + (size_t)stk::MAX_E * stk::F + 4u;   // xw | lw | hw | cw
    Q4B_CHECK(cudaMalloc(&g_s_words, words * sizeof(unsigned long long)));
    Q4B_CHECK(cudaMemset(g_s_words, 0, words * sizeof(unsigned long long)));
    Q4B_CHECK(cudaMalloc(&g_s_ctr, 2 * sizeof(unsigned long long)));
    Q4B_CHECK(cudaMemset(g_s_ctr, 0, 2 * sizeof(unsigned long long)));
    return true;
}

bool q4b_fused_warm() { return stack_scratch(); }
static void session_end_of(const struct Q4bStackPlan *p);
void q4b_fused_shutdown() {
    session_end_of(nullptr);
    cudaFree(g_s_words);
    cudaFree(g_s_ctr);
    if (g_s_prof) cudaFree(g_s_prof);
    g_s_words = g_s_ctr = g_s_prof = nullptr;
}

// Does the persistent kernel take this shape?  (No: the caller runs the launch chain.)
static bool stack_shape_ok(const uint8_t *base, uint64_t stride, uint64_t og, uint64_t ou, uint64_t od,
                           int32_t shared_slot, uint32_t n_expert, uint32_t topk, uint32_t n_embd,
                           uint32_t n_ff, stk::Args *a, size_t *smem_out) {
    using namespace stk;
    Q4bState &s = g_q4b;
    if (n_embd != H || n_ff != F || n_expert > NT || n_expert == 0 || topk == 0 || topk > 32 ||
        topk > n_expert)
        return false;
    if (!q4b_ptr_tiled(base) || (og % 16) || (ou % 16) || (od % 16) || (stride % 16)) return false;
    const uint32_t ncta = (uint32_t)s.n_sm;
    const uint32_t ne = topk + (shared_slot >= 0 ? 1u : 0u);
    const uint32_t max_units = (topk * F + ncta - 1) / ncta + 1;
    const uint32_t n_chunks = (max_units + UCHUNK - 1) / UCHUNK;
    const uint32_t max_sh = (F + ncta - 1) / ncta + 1;
    const uint32_t max_dt = ((H / 4 + ncta - 1) / ncta) * ne;
    const uint32_t max_rr = (n_expert + ncta - 1) / ncta;
    if (n_chunks > MAX_CHUNKS || n_chunks > NW - 2 || max_dt > MAX_DT || max_units > MAX_UNITS ||
        max_sh > MAX_SH || ne > MAX_E || max_rr > MAX_RROWS)
        return false;
    uint32_t stage_bytes = n_chunks * UCHUNK * 2u * Q4B_TILE_BYTES;
    if (stage_bytes < max_rr * H * 4u) stage_bytes = max_rr * H * 4u;
    const uint32_t small = (uint32_t)((sizeof(Small) + 127) & ~127u);
    a->off_stage = 65536u + small;
    a->off_down = a->off_stage + ((stage_bytes + 127u) & ~127u);
    a->off_sh = a->off_down + ((max_dt * Q4B_TILE_BYTES + 127u) & ~127u);
    const size_t smem = (size_t)a->off_sh + 2u * MAX_SH * Q4B_TILE_BYTES + 1024;
    if (smem > 227u * 1024u) return false;
    *smem_out = smem;
    return true;
}

static void session_args(const struct Q4bSession *ses, stk::Args *a);
static void plan_args(const struct Q4bStackPlan *pl, stk::Args *a);

// Launches the kernel over n_layers layers (layers == NULL: the one layer l0).  Returns false,
// with nothing enqueued, when the kernel does not apply.
static bool stack_launch(const stk::Layer &l0, const stk::Layer *d_layers, uint32_t n_layers,
                         uint64_t stride, uint64_t og, uint64_t ou, uint64_t od, int32_t shared_slot,
                         const float *d_x, float eps, uint32_t n_expert, uint32_t topk, uint32_t n_embd,
                         uint32_t n_ff, float *d_y, int32_t *d_ids, float *d_wts, float *y_host_dev,
                         uint32_t *flag_host_dev, uint32_t flag_val, const float *h_x_param,
                         const struct Q4bSession *ses = nullptr, const struct Q4bStackPlan *pl = nullptr) {
    using namespace stk;
    Q4bState &s = g_q4b;
    Args a;
    size_t smem = 0;
    if (n_layers == 0 || n_layers > MAX_LAYERS || (n_layers > 1 && !d_layers)) return false;
    if (g_s_session && !ses) return false;   // a session's kernel is resident: nothing else can run until it ends
    if (!stack_shape_ok(l0.base, stride, og, ou, od, shared_slot, n_expert, topk, n_embd, n_ff, &a, &smem))
        return false;
    if (((uintptr_t)l0.router % 16) || (!h_x_param && ((uintptr_t)d_x % 16)) ||
        (l0.norm_w && ((uintptr_t)l0.norm_w % 16)) || ((uintptr_t)d_y % 16) || ((uintptr_t)l0.sgate % 16))
        return false;
    if (!stack_scratch()) return false;
    a.l0 = l0;
    a.layers = d_layers;
    a.n_layers = n_layers;
    a.stride = stride;
    a.og = og;
    a.ou = ou;
    a.od = od;
    a.shared_slot = shared_slot;
    a.x = d_x;
    a.codes = s.codes_d;
    a.eps = eps;
    a.n_expert = n_expert;
    a.topk = topk;
    a.y = d_y;
    a.ids_out = d_ids;
    a.wts_out = d_wts;
    a.xw = g_s_words;
    a.lw = g_s_words + H;
    a.hw = g_s_words + H + 4u * NT;
    a.ctr = g_s_ctr;
    a.err = s.err_d;
    a.prof = g_s_prof;
    a.prof_layer = g_s_prof_layer < n_layers ? g_s_prof_layer : n_layers - 1;
    a.y_host = y_host_dev;
    a.flag_host = flag_host_dev;
    a.flag_val = flag_val;
    a.poll_limit = g_s_poll_limit;
    a.res = nullptr;
    a.inject = nullptr;
    a.hc = 0;
    if (pl) plan_args(pl, &a);
    a.x_host = nullptr;
    a.bell_host = nullptr;
    a.cw = g_s_words + H + 4u * NT + (size_t)MAX_E * F;
    a.lps = n_layers;
    a.li0 = 0;
    a.max_steps = 1;
    a.idle_ns = 0;
    if (!g_s_attr_set) {
        Q4B_CHECK(cudaFuncSetAttribute(moe_decode_stack_k, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       227 * 1024));
        Q4B_CHECK(cudaFuncSetAttribute(moe_decode_stack_xp_k, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       227 * 1024));
        Q4B_CHECK(cudaFuncSetAttribute(moe_decode_session_k, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       227 * 1024));
        g_s_attr_set = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)s.n_sm);
    cfg.blockDim = dim3(NT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s.stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident at once: they wait for one another's words
    at[0].val.cooperative = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    cudaError_t le;
    if (ses) {
        session_args(ses, &a);
        le = cudaLaunchKernelEx(&cfg, moe_decode_session_k, a);
    } else if (h_x_param) {
        XRow xr;   // the launch copies its parameters
        memcpy(xr.v, h_x_param, sizeof(xr.v));
        le = cudaLaunchKernelEx(&cfg, moe_decode_stack_xp_k, a, xr);
    } else {
        le = cudaLaunchKernelEx(&cfg, moe_decode_stack_k, a);
    }
    if (le != cudaSuccess) {
        fprintf(stderr, "q4cuda: persistent decode launch failed: %s\n", cudaGetErrorString(cudaGetLastError()));
        return false;
    }
    g_q4b_launches++;
    return true;
}

// One layer (q4_cuda_moe_decode and the host-buffer call).  Returns false when the kernel
// does not apply (caller takes the chain).
bool q4b_moe_decode_fused(const uint8_t *base, uint64_t stride, uint64_t og, uint64_t ou,
                          uint64_t od, int32_t shared_slot, const float *d_x,
                          const float *d_norm_w, float eps, const float *d_router,
                          uint32_t n_expert, uint32_t topk, uint32_t n_embd, uint32_t n_ff,
                          float *d_y, int32_t *d_ids, float *d_wts, float *y_host_dev,
                          uint32_t *flag_host_dev, uint32_t flag_val, const float *h_x_param) {
    const stk::Layer l0 = {base, d_norm_w, d_router, nullptr};
    return stack_launch(l0, nullptr, 1, stride, og, ou, od, shared_slot, d_x, eps, n_expert, topk, n_embd,
                        n_ff, d_y, d_ids, d_wts, y_host_dev, flag_host_dev, flag_val, h_x_param);
}

// ---- a stack of layers bound once ----
struct Q4bStackPlan {
    stk::Layer *d_layers;
    stk::Layer first;
    uint32_t n_layers;
    uint64_t stride, og, ou, od;
    int32_t shared_slot;
    float eps;
    uint32_t n_expert, topk, n_embd, n_ff;
    float *y_alias;        // device alias of the host result buffer last used with _host
    const void *y_alias_of;
    float *res;            // optional epilogue (q4_cuda_decode_stack_set_final)
    const float *inject;
    uint32_t hc;
};
static void plan_args(const Q4bStackPlan *pl, stk::Args *a) {
    a->res = pl->res;
    a->inject = pl->inject;
    a->hc = pl->hc;
}
static Q4bStackPlan *g_s_plans[64] = {};   // live plans (their cached aliases die with host_free)

extern "C" void *q4_cuda_decode_stack_plan(const q4_cuda_stack_layer_t *layers, uint32_t n_layers,
                                           uint64_t stride, uint64_t og, uint64_t ou, uint64_t od,
                                           int32_t shared_slot, float eps, uint32_t n_expert, uint32_t topk,
                                           uint32_t n_embd, uint32_t n_ff) {
    if (!g_q4b.ok || !layers || n_layers == 0 || n_layers > stk::MAX_LAYERS) return nullptr;
    stk::Args tmp;
    size_t smem = 0;
    for (uint32_t l = 0; l < n_layers; l++) {
        if (!layers[l].base || !layers[l].d_router || ((uintptr_t)layers[l].d_router % 16) ||
            ((uintptr_t)layers[l].d_norm_w % 16))
            return nullptr;
        if (!stack_shape_ok(layers[l].base, stride, og, ou, od, shared_slot, n_expert, topk, n_embd, n_ff,
                            &tmp, &smem))
            return nullptr;
    }
    int slot = -1;
    for (int i = 0; i < 64; i++)
        if (!g_s_plans[i]) {
            slot = i;
            break;
        }
    if (slot < 0) return nullptr;
    stk::Layer host[stk::MAX_LAYERS];
    for (uint32_t l = 0; l < n_layers; l++)
        host[l] = stk::Layer{layers[l].base, layers[l].d_norm_w, layers[l].d_router, nullptr};
    Q4bStackPlan *p = new Q4bStackPlan{};
    if (cudaMalloc(&p->d_layers, n_layers * sizeof(stk::Layer)) != cudaSuccess ||
        cudaMemcpy(p->d_layers, host, n_layers * sizeof(stk::Layer), cudaMemcpyHostToDevice) != cudaSuccess) {
        cudaGetLastError();
        if (p->d_layers) cudaFree(p->d_layers);
        delete p;
        return nullptr;
    }
    p->first = host[0];
    p->n_layers = n_layers;
    p->stride = stride;
    p->og = og;
    p->ou = ou;
    p->od = od;
    p->shared_slot = shared_slot;
    p->eps = eps;
    p->n_expert = n_expert;
    p->topk = topk;
    p->n_embd = n_embd;
    p->n_ff = n_ff;
    g_s_plans[slot] = p;
    return p;
}
static void session_end_of(const Q4bStackPlan *p);   // ends the live session if it runs on p (NULL: any)
extern "C" void q4_cuda_decode_stack_free(void *plan) {
    Q4bStackPlan *p = (Q4bStackPlan *)plan;
    if (!p) return;
    session_end_of(p);
    for (int i = 0; i < 64; i++)
        if (g_s_plans[i] == p) g_s_plans[i] = nullptr;
    if (g_q4b.ok) {
        cudaStreamSynchronize(g_q4b.stream);
        cudaFree(p->d_layers);
    }
    delete p;
}
extern "C" uint32_t q4_cuda_decode_stack_layers(void *plan) {
    return plan ? ((Q4bStackPlan *)plan)->n_layers : 0u;
}
extern "C" bool q4_cuda_decode_stack_dev(void *plan, const float *d_x, float *d_y, int32_t *d_ids,
                                         float *d_wts) {
    Q4bStackPlan *p = (Q4bStackPlan *)plan;
    if (!g_q4b.ok || !p || !d_x || !d_y) return false;
    return stack_launch(p->first, p->d_layers, p->n_layers, p->stride, p->og, p->ou, p->od, p->shared_slot,
                        d_x, p->eps, p->n_expert, p->topk, p->n_embd, p->n_ff, d_y, d_ids, d_wts, nullptr,
                        nullptr, 0, nullptr, nullptr, p);
}
// The shared expert's gate vector of one layer of the plan ([n_embd] floats on the device, 16-byte
// aligned; NULL: weight 1).  Waits for the stream: the layer table is rewritten in place.
extern "C" bool q4_cuda_decode_stack_set_sgate(void *plan, uint32_t layer, const float *d_sgate) {
    Q4bStackPlan *p = (Q4bStackPlan *)plan;
    if (!g_q4b.ok || !p || layer >= p->n_layers || ((uintptr_t)d_sgate % 16) || p->shared_slot < 0) return false;
    if (g_s_session) return false;
    Q4B_CHECK(cudaStreamSynchronize(g_q4b.stream));
    Q4B_CHECK(cudaMemcpy(reinterpret_cast<uint8_t *>(p->d_layers + layer) + offsetof(stk::Layer, sgate), &d_sgate,
                         sizeof d_sgate, cudaMemcpyHostToDevice));
    if (layer == 0) p->first.sgate = d_sgate;
    return true;
}
// Epilogue of the plan's last layer: besides y, d_res[c][i] += y[i] * 2 sigmoid(d_inject[c] / hc) for
// the hc residual streams (what q4_hip_moe_final does with y after the layer); d_res == NULL: off.
extern "C" bool q4_cuda_decode_stack_set_final(void *plan, float *d_res, const float *d_inject, uint32_t hc) {
    Q4bStackPlan *p = (Q4bStackPlan *)plan;
    if (!p || (d_res && (!d_inject || hc == 0 || hc > 64))) return false;
    p->res = d_res;
    p->inject = d_res ? d_inject : nullptr;
    p->hc = d_res ? hc : 0;
    return true;
}

// Device alias of a mapped, page-locked host buffer (NULL when it is anything else).
float *q4b_host_alias(const void *h) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, h) == cudaSuccess && at.type == cudaMemoryTypeHost && at.devicePointer &&
        ((uintptr_t)at.devicePointer % 16u) == 0)
        return (float *)at.devicePointer;
    cudaGetLastError();
    return nullptr;
}
// Forget cached aliases of a host buffer that is going away (q4_hip_host_free_coh,
// q4_hip_host_unregister, shutdown call this).
void q4b_stack_forget_host(const void *h) {
    for (int i = 0; i < 64; i++)
        if (g_s_plans[i] && (!h || g_s_plans[i]->y_alias_of == h)) {
            g_s_plans[i]->y_alias_of = nullptr;
            g_s_plans[i]->y_alias = nullptr;
        }
}

// Waits for the hand-off flag of launch `epoch`.  false: the kernel reported a device error,
// or the flag never came (then the stream's own error is printed).
bool q4b_wait_flag(uint32_t epoch) {
    Q4bState &s = g_q4b;
    volatile uint32_t *f = s.flag_h;
    for (uint64_t spins = 0; (*f & 0x7fffffffu) != epoch; spins++) {
        if (spins > 200000000ull) {        // far beyond any launch: let the stream say why
            Q4B_CHECK(cudaStreamSynchronize(s.stream));
            break;
        }
#if defined(__x86_64__)
        __builtin_ia32_pause();
#endif
    }
    std::atomic_thread_fence(std::memory_order_acquire);
    return *f == epoch;
}
uint32_t q4b_next_flag_epoch() {
    Q4bState &s = g_q4b;
    s.flag_epoch = (s.flag_epoch + 1u) & 0x7fffffffu;
    if (!s.flag_epoch) s.flag_epoch = 1u;
    return s.flag_epoch;
}

extern "C" bool q4_cuda_decode_stack_host(void *plan, const float *h_x, float *h_y) {
    Q4bStackPlan *p = (Q4bStackPlan *)plan;
    Q4bState &s = g_q4b;
    if (!s.ok || !p || !h_x || !h_y) return false;
    float *d_x = s.xn + (size_t)(Q4B_MAX_TOK - 1) * Q4B_XQ_MAXLEN;
    float *d_y = s.xn + (size_t)(Q4B_MAX_TOK - 2) * Q4B_XQ_MAXLEN;
    if (s.flag_h) {
        if (p->y_alias_of != h_y) {   // the attribute query costs about a microsecond: once per buffer
            p->y_alias = q4b_host_alias(h_y);
            p->y_alias_of = p->y_alias ? h_y : nullptr;
        }
        if (p->y_alias) {
            const uint32_t epoch = q4b_next_flag_epoch();
            if (stack_launch(p->first, p->d_layers, p->n_layers, p->stride, p->og, p->ou, p->od, p->shared_slot,
                             d_x, p->eps, p->n_expert, p->topk, p->n_embd, p->n_ff, d_y, nullptr, nullptr,
                             p->y_alias, s.flag_d, epoch, h_x, nullptr, p))
                return q4b_wait_flag(epoch);
        }
    }
    Q4B_CHECK(cudaMemcpyAsync(d_x, h_x, (size_t)p->n_embd * 4, cudaMemcpyHostToDevice, s.stream));
    if (!q4_cuda_decode_stack_dev(plan, d_x, d_y, nullptr, nullptr)) return false;
    Q4B_CHECK(cudaMemcpyAsync(h_y, d_y, (size_t)p->n_embd * 4, cudaMemcpyDeviceToHost, s.stream));
    Q4B_CHECK(cudaStreamSynchronize(s.stream));
    return true;
}

// ---- sessions: the kernel stays resident, a step costs no launch ----
// A decode loop that calls one MoE layer per launch pays the launch (5 us of host time, about
// as much again on the device) and the drain of the previous kernel on every call.  A session
// launches the stack kernel once; it then waits on a doorbell word in pinned host memory.  A
// step: the host writes the token's row into the session's pinned row buffer and rings; CTA 0
// reads bell and row over the bus and hands the row to the other CTAs through the exchange
// words; the step's layers run as in any stack launch (the next step's router rows and shared
// expert tiles were fetched while the kernel waited); the last CTA writes y and the step number
// into pinned host memory, where the host is spinning.  While a session is live its kernel
// holds every SM: other work queued on the device waits, and the library's other decode calls
// answer false.  The kernel leaves by itself when told (end), after max_steps steps, or when no
// ring came for idle_ms; the next step call then starts it again.
struct Q4bSession {
    Q4bStackPlan *plan;
    uint32_t lps, max_steps, idle_ms;
    uint32_t rung;          // steps rung since the kernel was launched
    uint32_t pos;           // the plan's layer the next step starts with
    bool launched;
    float *x_h, *y_h;       // pinned, mapped
    uint32_t *bell_h, *flag_h;
    float *x_d, *y_hd;      // their device aliases
    uint32_t *bell_d, *flag_d;
    float *y_d;             // device row the CTAs write their parts of y into
};

static void session_args(const Q4bSession *ses, stk::Args *a) {
    a->x = nullptr;
    a->x_host = ses->x_d;
    a->bell_host = ses->bell_d;
    a->lps = ses->lps;
    a->li0 = ses->pos;
    a->max_steps = ses->max_steps;
    a->idle_ns = (unsigned long long)ses->idle_ms * 1000000ull;
    a->flag_val = 1u;       // step n (from 1) reports n
}

static bool session_launch(Q4bSession *ses) {
    Q4bStackPlan *p = ses->plan;
    *ses->bell_h = 0;
    *ses->flag_h = 0;
    std::atomic_thread_fence(std::memory_order_seq_cst);
    ses->rung = 0;
    ses->launched = stack_launch(p->first, p->d_layers, p->n_layers, p->stride, p->og, p->ou, p->od,
                                 p->shared_slot, nullptr, p->eps, p->n_expert, p->topk, p->n_embd, p->n_ff,
                                 ses->y_d, nullptr, nullptr, ses->y_hd, ses->flag_d, 1u, nullptr, ses);
    return ses->launched;
}

extern "C" void *q4_cuda_decode_session_begin(void *plan, uint32_t layers_per_step, uint32_t max_steps,
                                              uint32_t idle_ms) {
    Q4bStackPlan *p = (Q4bStackPlan *)plan;
    if (!g_q4b.ok || !p || g_s_session) return nullptr;
    if (layers_per_step == 0) layers_per_step = p->n_layers;
    if (layers_per_step > p->n_layers || layers_per_step > stk::MAX_LAYERS - 2u) return nullptr;
    if (p->n_layers > 1 && !p->d_layers) return nullptr;
    Q4bSession *ses = new Q4bSession{};
    ses->plan = p;
    ses->lps = layers_per_step;
    ses->max_steps = max_steps == 0 || max_steps > (1u << 20) ? (1u << 20) : max_steps;
    ses->idle_ms = idle_ms == 0 ? 2000u : (idle_ms > 10000u ? 10000u : idle_ms);
    void *host = nullptr;
    const size_t row = (size_t)stk::H * sizeof(float);
    if (cudaHostAlloc(&host, 2 * row + 256, cudaHostAllocMapped) != cudaSuccess ||
        cudaMalloc(&ses->y_d, row) != cudaSuccess) {
        cudaGetLastError();
        if (host) cudaFreeHost(host);
        delete ses;
        return nullptr;
    }
    ses->x_h = (float *)host;
    ses->y_h = ses->x_h + stk::H;
    ses->bell_h = (uint32_t *)(ses->y_h + stk::H);
    ses->flag_h = ses->bell_h + 32;    // its own cache line
    void *dev = nullptr;
    if (cudaHostGetDevicePointer(&dev, host, 0) != cudaSuccess) {
        cudaGetLastError();
        cudaFreeHost(host);
        cudaFree(ses->y_d);
        delete ses;
        return nullptr;
    }
    ses->x_d = (float *)dev;
    ses->y_hd = ses->x_d + stk::H;
    ses->bell_d = (uint32_t *)(ses->y_hd + stk::H);
    ses->flag_d = ses->bell_d + 32;
    if (!session_launch(ses)) {
        cudaFreeHost(host);
        cudaFree(ses->y_d);
        delete ses;
        return nullptr;
    }
    g_s_session = ses;
    return ses;
}

// Waits until the kernel has left (it does so by itself: stop bell, step limit or idle time).
static bool session_drain(Q4bSession *ses) {
    if (!ses->launched) return true;
    ses->launched = false;
    return cudaStreamSynchronize(g_q4b.stream) == cudaSuccess;
}

extern "C" bool q4_cuda_decode_session_step(void *session, const float *h_x, float *h_y) {
    Q4bSession *ses = (Q4bSession *)session;
    if (!g_q4b.ok || !ses || ses != g_s_session || !h_x || !h_y) return false;
    volatile uint32_t *flag = ses->flag_h;
    for (int attempt = 0; attempt < 2; attempt++) {
        if (!ses->launched || ses->rung >= ses->max_steps || (*flag & stk::FLAG_EXIT)) {
            if (!session_drain(ses) || !session_launch(ses)) return false;
        }
        memcpy(ses->x_h, h_x, (size_t)stk::H * sizeof(float));
        const uint32_t n = ++ses->rung;
        __atomic_store_n(ses->bell_h, n, __ATOMIC_RELEASE);
        uint32_t f = 0;
        bool done = false;
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(ses->idle_ms + 3000u);
        for (uint64_t spins = 0;; spins++) {
            f = *flag;
            if ((f & stk::FLAG_EXIT) || (f & 0x3fffffffu) == n) {
                done = true;
                break;
            }
            if ((spins & 0xffffu) == 0xffffu && std::chrono::steady_clock::now() > deadline) break;
#if defined(__x86_64__)
            __builtin_ia32_pause();
#endif
        }
        std::atomic_thread_fence(std::memory_order_acquire);
        if (!done) {                      // far beyond any step: stop the kernel and let the stream say why
            __atomic_store_n(ses->bell_h, stk::BELL_STOP, __ATOMIC_RELEASE);
            session_drain(ses);
            return false;
        }
        if (f & stk::FLAG_EXIT) continue;   // the kernel had just left on its idle limit: start it again, once
        memcpy(h_y, ses->y_h, (size_t)stk::H * sizeof(float));
        ses->pos = (ses->pos + ses->lps) % ses->plan->n_layers;
        return !(f & stk::FLAG_ERR);
    }
    return false;
}

static void session_end_of(const Q4bStackPlan *p) {
    if (g_s_session && (!p || g_s_session->plan == p)) q4_cuda_decode_session_end(g_s_session);
}
extern "C" bool q4_cuda_decode_session_end(void *session) {
    Q4bSession *ses = (Q4bSession *)session;
    if (!ses || ses != g_s_session) return false;
    __atomic_store_n(ses->bell_h, stk::BELL_STOP, __ATOMIC_RELEASE);
    const bool ok = session_drain(ses);
    g_s_session = nullptr;
    cudaFreeHost(ses->x_h);
    cudaFree(ses->y_d);
    delete ses;
    return ok;
}

// In-kernel phase profile of the persistent decode kernel (diagnostics).
// enable(1) allocates the stamp buffer (not inside a capture); read copies the
// stamps of the last launch: out[cta * 16 + slot] in nanoseconds of the GPU's
// global timer; returns the number of CTAs.
extern "C" bool q4_cuda_fused_profile_enable(int on) {
    if (!g_q4b.ok) return false;
    if (on && !g_s_prof) {
        Q4B_CHECK(cudaMalloc(&g_s_prof, (size_t)g_q4b.n_sm * 16 * sizeof(unsigned long long)));
        Q4B_CHECK(cudaMemset(g_s_prof, 0, (size_t)g_q4b.n_sm * 16 * sizeof(unsigned long long)));
    } else if (!on && g_s_prof) {
        cudaStreamSynchronize(g_q4b.stream);
        cudaFree(g_s_prof);
        g_s_prof = nullptr;
    }
    return true;
}
extern "C" void q4_cuda_fused_profile_layer(uint32_t layer) { g_s_prof_layer = layer; }
extern "C" uint32_t q4_cuda_fused_profile_read(unsigned long long *out, uint32_t max_ctas) {
    if (!g_q4b.ok || !g_s_prof || !out) return 0;
    const uint32_t n = max_ctas < (uint32_t)g_q4b.n_sm ? max_ctas : (uint32_t)g_q4b.n_sm;
    if (cudaMemcpyAsync(out, g_s_prof, (size_t)n * 16 * sizeof(unsigned long long),
                        cudaMemcpyDeviceToHost, g_q4b.stream) != cudaSuccess ||
        cudaStreamSynchronize(g_q4b.stream) != cudaSuccess)
        return 0;
    return n;
}
// How many polls a wait for another CTA's word may take before it gives up (0 = the
// default).  For tests of the give-up path.
extern "C" void q4_cuda_decode_wait_limit(uint32_t polls) {
    g_s_poll_limit = polls ? polls : stk::POLL_LIMIT;
}
