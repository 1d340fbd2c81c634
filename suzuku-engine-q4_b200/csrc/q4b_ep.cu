// Expert parallelism over NCCL: libq4cuda_ep.so, one process per GPU.
//
// The reference is single-device (src/q4_rocm.cu:545-550), so this has no counterpart
// there; it shards the same path the way the path shards naturally: experts are
// independent packs (src/q4_expert.c:962-982) and the per-token combine is a plain
// weighted sum (src/q4_rocm.cu:15739-15751).
//
// Rank r of G holds experts [r*E/G, (r+1)*E/G) in slots 0..E/G-1 of its arena and a
// copy of the shared expert in slot E/G; the router and norm weights are replicated;
// each rank owns T_local tokens.  One layer on every rank:
//   1. RMSNorm, router GEMV, softmax/top-k for its own tokens
//   2. dispatch: normalised rows + picks of all ranks are gathered everywhere.  With
//      top-10 of 512 over <= 8 ranks a token visits 1-(1-1/G)^10 = 74..100 % of the
//      ranks, so the all-to-all degenerates to an all-gather; sending fp32 rows keeps
//      the quantisation (Q8-A, per row) on the receiving side bit-identical to 1 GPU
//   3. every rank runs its own experts on the rows that picked them (grouped product,
//      each tile decoded once), plus the shared expert for the tokens it owns, and
//      reduces per token: partial[t] = sum of its picks here, in pick order
//   4. combine: all-to-all of the partial rows to the tokens' owners, summed there in
//      rank order (reproducible)
// Everything runs on the library's stream; the only synchronising calls are the NCCL
// communicator set-up and the explicit barrier helper.
#include <cuda_runtime.h>
#include <nccl.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/q4cuda.h"
#include "../../include/q4cuda_ep.h"

namespace {

ncclComm_t g_comm = nullptr;
int g_rank = 0, g_world = 1;
float *g_scalar = nullptr;  // one float for barrier / max

#define EP_NCCL(call)                                                                   \
    do {                                                                                \
        ncclResult_t r_ = (call);                                                       \
        if (r_ != ncclSuccess) {                                                        \
            fprintf(stderr, "q4cuda_ep: %s failed: %s\n", #call, ncclGetErrorString(r_)); \
            return false;                                                               \
        }                                                                               \
    } while (0)

inline uint64_t al(uint64_t v) { return (v + 255u) & ~(uint64_t)255u; }

// y[t] = sum over ranks s = 0..G-1 of recv[s][t], in that order.
__global__ void ep_sum_k(const float *__restrict__ recv, float *__restrict__ y, uint32_t n,
                         uint32_t world) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float acc = 0.f;
    for (uint32_t s = 0; s < world; s++) acc += recv[(uint64_t)s * n + i];
    y[i] = acc;
}

// ---- the layer's all-reduce over peer memory (one kernel, no library call) ----
// Every rank exports one buffer (two copies of up to AR_MAX_ELEMS floats, then ready words) through
// CUDA IPC; the others map it.  The kernel on rank r: (1) copies its partial rows into its exported
// buffer (copy p = epoch & 1), fences at GPU scope (the rows stay in its own memory) and counts; the
// CTA that counts last stores the epoch into word [p][r] of EVERY rank's ready words (release stores
// at system scope to peer memory, one thread per rank); (2) waits,
// bounded in time, until its own ready words [p][0..G) all show the epoch; (3) every thread sums its
// elements over the ranks' buffers in rank order (plain loads from peer memory over NVLink), so all
// ranks end with the same bits; (4) the CTA that finishes last publishes the epoch for the next
// launch.  Two copies suffice: a rank can overwrite copy p only two launches later, and it gets
// there only after every peer has signalled the launch in between, which a peer does after it has
// finished reading copy p.  No multicast, no TMA: plain ld/st on mapped peer memory.
constexpr uint32_t AR_MAX_ELEMS = 64u * 4096u;
constexpr uint32_t AR_MAX_RANKS = 8;
constexpr uint32_t AR_CTAS = 64, AR_THREADS = 512;
constexpr uint32_t AR_ERR = 0x1000u;   // bit of the device error word: a peer's rows did not come in time
constexpr size_t AR_BUF_BYTES = 2ull * AR_MAX_ELEMS * sizeof(float);
// after the two row copies: 256 bytes of ready words (all-reduce [2][8], gather [2][8]), then the
// gather area [2][AR_MAX_RANKS][GATHER_SLOT] that the peers write their picks into
constexpr uint32_t GATHER_SLOT = 4096;
constexpr size_t AR_GATHER_OFF = AR_BUF_BYTES + 256;
constexpr size_t AR_MEM_BYTES = AR_GATHER_OFF + 2ull * AR_MAX_RANKS * GATHER_SLOT;
struct ArArgs {
    const float *src;
    float *dst;
    uint32_t n4;                       // float4 elements
    uint32_t world, rank;
    float *bufs[AR_MAX_RANKS];         // every rank's exported buffer (own: local pointer)
    uint32_t *ready[AR_MAX_RANKS];     // every rank's ready words [2][AR_MAX_RANKS]
    uint32_t *ctl;                     // local: [0] epoch of the last finished launch, [1] copies done, [2] CTAs done, [3] error
    unsigned long long wait_ns;
};
__global__ void __launch_bounds__(AR_THREADS) ep_allreduce_k(const __grid_constant__ ArArgs a) {
    __shared__ uint32_t s_epoch, s_last;
    const uint32_t tid = threadIdx.x;
    if (tid == 0) {
        uint32_t e;
        asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(e) : "l"(a.ctl) : "memory");
        s_epoch = e + 1u;
    }
    __syncthreads();
    const uint32_t epoch = s_epoch, p = epoch & 1u;
    const uint32_t gtid = blockIdx.x * AR_THREADS + tid, gsz = gridDim.x * AR_THREADS;
    float4 *mine = reinterpret_cast<float4 *>(a.bufs[a.rank]) + (size_t)p * (AR_MAX_ELEMS / 4u);
    const float4 *src4 = reinterpret_cast<const float4 *>(a.src);
    for (uint32_t i = gtid; i < a.n4; i += gsz) mine[i] = src4[i];
    __syncthreads();
    // The rows live in this GPU's memory: a fence at GPU scope and a count per CTA; the CTA that counts
    // last tells every rank (this one too), one thread per rank so that the system-scope release stores
    // go out side by side (one thread storing them in turn spent a fence per rank).
    if (tid == 0) {
        __threadfence();
        const uint32_t old = atomicAdd(a.ctl + 1, 1u);
        s_last = old % gridDim.x == gridDim.x - 1u ? 1u : 0u;
        if (s_last) __threadfence();
    }
    __syncthreads();
    if (s_last && tid < a.world)
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.ready[tid] + p * AR_MAX_RANKS + a.rank), "r"(epoch)
                     : "memory");
    if (tid < a.world) {
        const uint32_t *w = a.ready[a.rank] + p * AR_MAX_RANKS + tid;
        unsigned long long t0;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
        for (uint32_t i = 0;; i++) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(w) : "memory");
            if (v == epoch) break;
            if ((i & 255u) == 255u) {
                unsigned long long t;
                asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
                if (t - t0 > a.wait_ns) {
                    atomicOr(a.ctl + 3, AR_ERR);
                    break;
                }
            }
        }
    }
    __syncthreads();
    float4 *dst4 = reinterpret_cast<float4 *>(a.dst);
    for (uint32_t i = gtid; i < a.n4; i += gsz) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t r = 0; r < a.world; r++) {
            const float4 *b = reinterpret_cast<const float4 *>(a.bufs[r]) + (size_t)p * (AR_MAX_ELEMS / 4u) + i;
            float4 v;
            asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                         : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                         : "l"(b)
                         : "memory");
            acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
        }
        dst4[i] = acc;
    }
    __syncthreads();
    if (tid == 0) {
        const uint32_t old = atomicAdd(a.ctl + 2, 1u);
        if (old % gridDim.x == gridDim.x - 1u)
            asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(a.ctl), "r"(epoch) : "memory");
    }
}

// The picks of every rank's own tokens, gathered on every rank (a few hundred bytes per rank): each
// rank pushes its block into slot [copy][rank] of every rank's gather area and stores the epoch into
// that rank's gather-ready word; then waits (bounded) for all ranks' words and copies the slots out.
// One CTA.  Epochs and the two copies work as in the all-reduce (their own counter, ctl[4]).
struct GatherArgs {
    const int32_t *ids_l;
    const float *wts_l;
    int32_t *ids;
    float *wts;
    uint32_t n;                        // entries per rank (tokens x picks)
    uint32_t world, rank;
    uint8_t *mem[AR_MAX_RANKS];        // every rank's exported memory
    uint32_t *ctl;
    unsigned long long wait_ns;
};
__global__ void __launch_bounds__(256) ep_gather_picks_k(const __grid_constant__ GatherArgs a) {
    __shared__ uint32_t s_epoch;
    const uint32_t tid = threadIdx.x;
    if (tid == 0) {
        uint32_t e;
        asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(e) : "l"(a.ctl + 4) : "memory");
        s_epoch = e + 1u;
    }
    __syncthreads();
    const uint32_t epoch = s_epoch, p = epoch & 1u;
    const size_t slot = AR_GATHER_OFF + ((size_t)p * AR_MAX_RANKS + a.rank) * GATHER_SLOT;
    for (uint32_t r = 0; r < a.world; r++) {
        uint32_t *dst = reinterpret_cast<uint32_t *>(a.mem[r] + slot);
        for (uint32_t i = tid; i < a.n; i += 256) {
            dst[i] = (uint32_t)a.ids_l[i];
            dst[a.n + i] = __float_as_uint(a.wts_l[i]);
        }
    }
    __syncthreads();
    if (tid < a.world)   // one thread per rank: the release stores (each orders the CTA's pushes before it) go out side by side
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(reinterpret_cast<uint32_t *>(a.mem[tid] + AR_BUF_BYTES) +
                                                              2u * AR_MAX_RANKS + p * AR_MAX_RANKS + a.rank),
                     "r"(epoch)
                     : "memory");
    if (tid < a.world) {
        const uint32_t *w = reinterpret_cast<const uint32_t *>(a.mem[a.rank] + AR_BUF_BYTES) + 2u * AR_MAX_RANKS +
                            p * AR_MAX_RANKS + tid;
        unsigned long long t0;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
        for (uint32_t i = 0;; i++) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(w) : "memory");
            if (v == epoch) break;
            if ((i & 255u) == 255u) {
                unsigned long long t;
                asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
                if (t - t0 > a.wait_ns) {
                    atomicOr(a.ctl + 3, AR_ERR);
                    break;
                }
            }
        }
    }
    __syncthreads();
    for (uint32_t r = 0; r < a.world; r++) {
        const uint32_t *src =
            reinterpret_cast<const uint32_t *>(a.mem[a.rank] + AR_GATHER_OFF + ((size_t)p * AR_MAX_RANKS + r) * GATHER_SLOT);
        for (uint32_t i = tid; i < a.n; i += 256) {
            uint32_t vi, vw;
            asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(vi) : "l"(src + i) : "memory");
            asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(vw) : "l"(src + a.n + i) : "memory");
            a.ids[(size_t)r * a.n + i] = (int32_t)vi;
            a.wts[(size_t)r * a.n + i] = __uint_as_float(vw);
        }
    }
    __syncthreads();
    if (tid == 0) asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(a.ctl + 4), "r"(epoch) : "memory");
}

struct ArState {
    bool ok;
    uint8_t *mem;                      // exported: [2][AR_MAX_ELEMS] floats | ready words
    uint32_t *ctl;                     // local control words
    float *bufs[AR_MAX_RANKS];
    uint32_t *ready[AR_MAX_RANKS];
    void *opened[AR_MAX_RANKS];
} g_ar = {};

struct EpWs {
    float *xn_l, *logits, *wts_l, *xn, *wts, *rw, *gu, *pd, *partial, *recv;
    int32_t *ids_l, *ids, *atok, *rsrc, *bounds;
    void *xq, *hq;
    uint64_t bytes;
};

EpWs carve(uint8_t *p, uint32_t world, uint32_t t_local, uint32_t topk, uint32_t n_expert,
           uint32_t n_embd, uint32_t n_ff) {
    EpWs w;
    uint64_t off = 0;
    const uint64_t T = (uint64_t)world * t_local, k1 = topk + 1u, rows = T * k1;
    auto take = [&](uint64_t n) {
        uint8_t *r = p ? p + off : nullptr;
        off += al(n);
        return r;
    };
    w.xn_l = (float *)take((uint64_t)t_local * n_embd * 4);
    w.logits = (float *)take((uint64_t)t_local * n_expert * 4);
    w.ids_l = (int32_t *)take((uint64_t)t_local * topk * 4);
    w.wts_l = (float *)take((uint64_t)t_local * topk * 4);
    w.xn = (float *)take(T * n_embd * 4);
    w.ids = (int32_t *)take(T * topk * 4);
    w.wts = (float *)take(T * topk * 4);
    w.atok = (int32_t *)take(rows * 4);
    w.rsrc = (int32_t *)take(rows * 4);
    w.rw = (float *)take(rows * 4);
    w.bounds = (int32_t *)take(1025 * 4);
    w.xq = take(q4_mmq_q8_bytes(rows, n_embd));
    w.gu = (float *)take(rows * 2 * n_ff * 4);
    w.hq = take(q4_mmq_q8_bytes(rows, n_ff));
    w.pd = (float *)take(rows * n_embd * 4);
    w.partial = (float *)take(T * n_embd * 4);
    w.recv = (float *)take(T * n_embd * 4);
    w.bytes = off;
    return w;
}

int g_ar_mode = 2;   // 0: ncclAllReduce, 1: the peer-memory kernel, 2 (default): the kernel where it was set up
// The kernel's cost is a handful of NVLink round trips (copy out, signal, wait, read) whatever the number
// of ranks.  Measured inside the 48-layer job of 64 tokens it is 10 us per layer faster than
// ncclAllReduce at 2 ranks and 9 us at 8 (512 KB per layer: latency, not bandwidth); with one thread
// storing the ranks' ready flags in turn it had been 2-4 us slower.
int g_split_routing = 0;   // q4_cuda_ep_split_routing
bool ar_use_kernel() { return g_ar.ok && g_ar_mode != 0; }

void ar_teardown() {
    for (uint32_t r = 0; r < AR_MAX_RANKS; r++)
        if (g_ar.opened[r]) cudaIpcCloseMemHandle(g_ar.opened[r]);
    if (g_ar.mem) cudaFree(g_ar.mem);
    if (g_ar.ctl) cudaFree(g_ar.ctl);
    g_ar = ArState{};
}

// Maps every rank's exported buffer.  All ranks end with the same answer (a minimum over the ranks):
// either every rank uses the peer kernel or none does.
bool ar_setup() {
    cudaStream_t st = (cudaStream_t)q4_hip_stream();
    int ok = 1;
    cudaIpcMemHandle_t mine;
    memset(&mine, 0, sizeof mine);
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    if (g_world > (int)AR_MAX_RANKS || g_world < 2 || cudaMalloc(&g_ar.mem, AR_MEM_BYTES) != cudaSuccess ||
        cudaMemset(g_ar.mem, 0, AR_MEM_BYTES) != cudaSuccess || cudaMalloc(&g_ar.ctl, 64) != cudaSuccess ||
        cudaMemset(g_ar.ctl, 0, 64) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess ||
        cudaIpcGetMemHandle(&mine, g_ar.mem) != cudaSuccess) {
        cudaGetLastError();
        ok = 0;
    }
    // the handles of all ranks, gathered through the communicator
    uint8_t *d_all = (uint8_t *)q4_hip_malloc(64u * (size_t)g_world + 256);
    cudaIpcMemHandle_t all[AR_MAX_RANKS];
    memset(all, 0, sizeof all);
    if (!d_all) return false;
    bool gathered = g_world <= (int)AR_MAX_RANKS &&
                    cudaMemcpy(d_all + 64 * g_rank, &mine, 64, cudaMemcpyHostToDevice) == cudaSuccess &&
                    ncclAllGather(d_all + 64 * g_rank, d_all, 64, ncclUint8, g_comm, st) == ncclSuccess &&
                    cudaStreamSynchronize(st) == cudaSuccess &&
                    cudaMemcpy(all, d_all, 64u * (size_t)g_world, cudaMemcpyDeviceToHost) == cudaSuccess;
    if (!gathered) ok = 0;
    // every rank learns whether every rank got this far before anyone opens a handle
    float v = (float)ok;
    if (cudaMemcpy(g_scalar, &v, 4, cudaMemcpyHostToDevice) != cudaSuccess ||
        ncclAllReduce(g_scalar, g_scalar, 1, ncclFloat, ncclMin, g_comm, st) != ncclSuccess ||
        cudaStreamSynchronize(st) != cudaSuccess || cudaMemcpy(&v, g_scalar, 4, cudaMemcpyDeviceToHost) != cudaSuccess)
        v = 0.f;
    if (v >= 1.f) {
        for (int r = 0; r < g_world && ok; r++) {
            void *ptr = g_ar.mem;
            if (r != g_rank) {
                if (cudaIpcOpenMemHandle(&ptr, all[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                    cudaGetLastError();
                    ok = 0;
                    break;
                }
                g_ar.opened[r] = ptr;
            }
            g_ar.bufs[r] = (float *)ptr;
            g_ar.ready[r] = (uint32_t *)((uint8_t *)ptr + AR_BUF_BYTES);
        }
        v = (float)ok;
        if (cudaMemcpy(g_scalar, &v, 4, cudaMemcpyHostToDevice) != cudaSuccess ||
            ncclAllReduce(g_scalar, g_scalar, 1, ncclFloat, ncclMin, g_comm, st) != ncclSuccess ||
            cudaStreamSynchronize(st) != cudaSuccess ||
            cudaMemcpy(&v, g_scalar, 4, cudaMemcpyDeviceToHost) != cudaSuccess)
            v = 0.f;
    }
    q4_hip_free(d_all);
    if (v < 1.f) {
        ar_teardown();
        return false;
    }
    g_ar.ok = true;
    return true;
}

bool gather_launch(const int32_t *ids_l, const float *wts_l, int32_t *ids, float *wts, uint32_t n, cudaStream_t st) {
    GatherArgs a;
    a.ids_l = ids_l;
    a.wts_l = wts_l;
    a.ids = ids;
    a.wts = wts;
    a.n = n;
    a.world = (uint32_t)g_world;
    a.rank = (uint32_t)g_rank;
    for (uint32_t r = 0; r < AR_MAX_RANKS; r++) a.mem[r] = (uint8_t *)g_ar.bufs[r];
    a.ctl = g_ar.ctl;
    a.wait_ns = 2000000000ull;
    ep_gather_picks_k<<<1, 256, 0, st>>>(a);
    return cudaGetLastError() == cudaSuccess;
}

bool ar_launch(const float *src, float *dst, size_t n, cudaStream_t st) {
    ArArgs a;
    a.src = src;
    a.dst = dst;
    a.n4 = (uint32_t)(n / 4u);
    a.world = (uint32_t)g_world;
    a.rank = (uint32_t)g_rank;
    for (uint32_t r = 0; r < AR_MAX_RANKS; r++) {
        a.bufs[r] = g_ar.bufs[r];
        a.ready[r] = g_ar.ready[r];
    }
    a.ctl = g_ar.ctl;
    a.wait_ns = 2000000000ull;
    ep_allreduce_k<<<AR_CTAS, AR_THREADS, 0, st>>>(a);
    return cudaGetLastError() == cudaSuccess;
}

}  // namespace

// ---- communicator ----
extern "C" bool q4_cuda_ep_unique_id(uint8_t *out128) {
    if (!out128) return false;
    ncclUniqueId id;
    EP_NCCL(ncclGetUniqueId(&id));
    static_assert(sizeof(ncclUniqueId) == 128, "id size");
    memcpy(out128, &id, 128);
    return true;
}

// The device must already be current and q4_hip_init() done on it.
extern "C" bool q4_cuda_ep_init(const uint8_t *id128, int rank, int world) {
    if (!id128 || world < 1 || rank < 0 || rank >= world || g_comm || !q4_hip_ok()) return false;
    ncclUniqueId id;
    memcpy(&id, id128, 128);
    EP_NCCL(ncclCommInitRank(&g_comm, world, id, rank));
    g_rank = rank;
    g_world = world;
    g_scalar = (float *)q4_hip_malloc(256);
    if (!g_scalar) return false;
    if (world > 1) (void)ar_setup();   // without it q4_cuda_ep_layer_ar keeps ncclAllReduce
    return true;
}
// Which all-reduce q4_cuda_ep_layer_ar uses: 1 or 2 (default) the library's own kernel over mapped peer
// memory where every rank could map every other rank's buffer (else ncclAllReduce), 0 ncclAllReduce.
// Returns 1 when the kernel is in effect.  Every rank must make the same call.
extern "C" int q4_cuda_ep_allreduce_mode(int mode) {
    if (mode >= 0 && mode <= 2) g_ar_mode = mode;
    return ar_use_kernel() ? 1 : 0;
}
// 1: with the peer buffers mapped, a rank routes only its own tokens and the picks are gathered through
// peer memory; 0 (default): every rank routes all tokens.  Every rank must make the same call.
extern "C" void q4_cuda_ep_split_routing(int on) { g_split_routing = on ? 1 : 0; }
// Error word of the peer all-reduce (0x1000: a peer's rows did not arrive within two seconds).  Synchronises.
extern "C" uint32_t q4_cuda_ep_error(void) {
    uint32_t e = 0;
    if (!g_ar.ok) return 0;
    q4_hip_sync();
    if (cudaMemcpy(&e, g_ar.ctl + 3, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return 0xffffffffu;
    return e;
}

extern "C" void q4_cuda_ep_shutdown(void) {
    if (!g_comm) return;
    q4_hip_sync();
    ar_teardown();
    ncclCommDestroy(g_comm);
    g_comm = nullptr;
    q4_hip_free(g_scalar);
    g_scalar = nullptr;
    g_world = 1;
    g_rank = 0;
}

extern "C" int q4_cuda_ep_rank(void) { return g_rank; }
extern "C" int q4_cuda_ep_world(void) { return g_world; }

// max over ranks of one host float (also a barrier): synchronises.
extern "C" bool q4_cuda_ep_allreduce_max(float *h_value) {
    if (!g_comm || !h_value) return false;
    cudaStream_t st = (cudaStream_t)q4_hip_stream();
    if (!q4_hip_h2d(g_scalar, h_value, 4)) return false;
    EP_NCCL(ncclAllReduce(g_scalar, g_scalar, 1, ncclFloat, ncclMax, g_comm, st));
    return q4_hip_d2h(h_value, g_scalar, 4);
}

extern "C" uint64_t q4_cuda_ep_layer_ws_bytes(uint32_t world, uint32_t t_local, uint32_t topk,
                                              uint32_t n_expert, uint32_t n_embd, uint32_t n_ff) {
    return carve(nullptr, world, t_local, topk, n_expert, n_embd, n_ff).bytes;
}

// One MoE layer for this rank's t_local tokens (steps 1-4 of the header comment).
// base/stride/og/ou/od address THIS rank's arena (local slot j = expert rank*E/G + j,
// shared expert in slot E/G when has_shared); d_router is the full [n_expert][n_embd]
// matrix; d_x / d_y hold t_local rows.  Every rank must call it with the same shapes.
extern "C" bool q4_cuda_ep_layer(const uint8_t *base, uint64_t stride, uint64_t og, uint64_t ou,
                                 uint64_t od, int has_shared, const float *d_x,
                                 const float *d_norm_w, float eps, const float *d_router,
                                 uint32_t n_expert, uint32_t topk, uint32_t n_embd, uint32_t n_ff,
                                 uint32_t t_local, float *d_y, void *d_ws, uint64_t ws_bytes) {
    if (!g_comm || !base || !d_x || !d_router || !d_y || !d_ws || t_local == 0) return false;
    const uint32_t G = (uint32_t)g_world;
    if (n_expert % G) return false;
    const uint32_t e_local = n_expert / G, n_e = e_local + 1u;
    if (n_e > 512u || topk == 0 || topk >= 64u) return false;
    const EpWs w = carve((uint8_t *)d_ws, G, t_local, topk, n_expert, n_embd, n_ff);
    if (ws_bytes < w.bytes) return false;
    cudaStream_t st = (cudaStream_t)q4_hip_stream();
    const uint32_t T = G * t_local, k1 = topk + 1u;
    const uint64_t rows = (uint64_t)T * k1;
    const uint64_t gate_bytes = (uint64_t)n_ff * (n_embd / 256u) * 110u;
    if (ou != og + gate_bytes) return false;
    // 1. own tokens: norm, router, top-k
    if (!q4_hip_grouped_rms_n(d_x, d_norm_w, w.xn_l, n_embd, 1, eps, t_local)) return false;
    if (!q4_hip_gemv_dd_n(Q4_T_F32, (const uint8_t *)d_router, n_expert, n_embd, w.xn_l, w.logits,
                          1.0f, t_local))
        return false;
    if (!q4_hip_route_pf(w.logits, w.ids_l, w.wts_l, t_local, n_expert, topk)) return false;
    // 2. dispatch
    EP_NCCL(ncclGroupStart());
    EP_NCCL(ncclAllGather(w.xn_l, w.xn, (size_t)t_local * n_embd, ncclFloat, g_comm, st));
    EP_NCCL(ncclAllGather(w.ids_l, w.ids, (size_t)t_local * topk, ncclInt32, g_comm, st));
    EP_NCCL(ncclAllGather(w.wts_l, w.wts, (size_t)t_local * topk, ncclFloat, g_comm, st));
    EP_NCCL(ncclGroupEnd());
    // 3. local experts on the rows that picked them
    if (!q4_cuda_assign_local(w.ids, w.wts, w.atok, w.rsrc, w.rw, w.bounds, T, topk,
                              (uint32_t)g_rank * e_local, e_local, has_shared, (uint32_t)g_rank * t_local,
                              t_local))
        return false;
    if (!q4_mmq_quantize(w.xn, w.atok, w.xq, Q4_T_IQ3_S, n_embd, rows)) return false;
    // rows of the largest entry one expects: the shared expert's (own tokens), or a routed
    // expert's share of all picks with a wide margin; only a hint for the kernel choice
    const uint32_t share = 4u * (T * topk / n_expert + 1u);
    const uint32_t max_hint = t_local > share ? t_local : share;
    if (!q4_mmq_mul_id(base + og, Q4_T_IQ3_S, 2ull * n_ff, n_embd, stride, n_e, w.xq, w.bounds,
                       max_hint, rows, w.gu, 2ull * n_ff))
        return false;
    if (!q4_cuda_mmq_swiglu_quantize(w.gu, w.hq, rows, n_ff)) return false;
    if (!q4_mmq_mul_id(base + od, Q4_T_IQ3_S, n_embd, n_ff, stride, n_e, w.hq, w.bounds,
                       max_hint, rows, w.pd, n_embd))
        return false;
    if (!q4_cuda_expert_reduce_set(w.partial, w.pd, w.rsrc, w.rw, T, k1, n_embd)) return false;
    // 4. combine
    const size_t blk = (size_t)t_local * n_embd;
    EP_NCCL(ncclGroupStart());
    for (uint32_t p = 0; p < G; p++) {
        EP_NCCL(ncclSend(w.partial + p * blk, blk, ncclFloat, (int)p, g_comm, st));
        EP_NCCL(ncclRecv(w.recv + p * blk, blk, ncclFloat, (int)p, g_comm, st));
    }
    EP_NCCL(ncclGroupEnd());
    ep_sum_k<<<(unsigned)((blk + 255) / 256), 256, 0, st>>>(w.recv, d_y, (uint32_t)blk, G);
    return cudaGetLastError() == cudaSuccess;
}

// The same layer in its one-collective form.  Every rank holds ALL T = world * t_local token
// rows (d_x and d_y have T rows, identical on every rank): each rank norms and routes all
// tokens itself (the router is replicated; at decode batch sizes that costs less than an
// exchange), runs its own experts on the rows that picked them plus the shared expert for the
// tokens [rank * t_local, (rank + 1) * t_local), and ONE all-reduce sums the per-rank partial
// rows into d_y on every rank -- which is the next layer's input, already in place.  One
// collective and nine launches per layer instead of two exchanges and twelve launches; at 64
// tokens the all-reduce moves 512 KB.  Results equal the single-GPU ones up to the order of the
// fp32 sum over ranks.
extern "C" bool q4_cuda_ep_layer_ar(const uint8_t *base, uint64_t stride, uint64_t og, uint64_t ou,
                                    uint64_t od, int has_shared, const float *d_x,
                                    const float *d_norm_w, float eps, const float *d_router,
                                    uint32_t n_expert, uint32_t topk, uint32_t n_embd, uint32_t n_ff,
                                    uint32_t t_local, float *d_y, void *d_ws, uint64_t ws_bytes) {
    if (!g_comm || !base || !d_x || !d_router || !d_y || !d_ws || t_local == 0) return false;
    const uint32_t G = (uint32_t)g_world;
    if (n_expert % G) return false;
    const uint32_t e_local = n_expert / G, n_e = e_local + 1u;
    if (n_e > 512u || topk == 0 || topk >= 64u) return false;
    const EpWs w = carve((uint8_t *)d_ws, G, t_local, topk, n_expert, n_embd, n_ff);
    if (ws_bytes < w.bytes) return false;
    cudaStream_t st = (cudaStream_t)q4_hip_stream();
    const uint32_t T = G * t_local, k1 = topk + 1u;
    const uint64_t rows = (uint64_t)T * k1;
    if (ou != og + (uint64_t)n_ff * (n_embd / 256u) * 110u) return false;
    // all tokens: norm, router, top-k (w.recv doubles as the T x n_expert logits: T * n_embd floats
    // hold them as long as n_expert <= n_embd)
    if (n_expert > n_embd) return false;
    // Routing.  Default: every rank routes all T tokens itself, norm + router product + top-k in one
    // launch where the shape allows (the same values as the three launches).  With the peer buffers
    // mapped and the split switched on, a rank routes only its own tokens and the ranks' picks are
    // gathered through peer memory (a few hundred bytes each).
    const bool want_split = g_split_routing && g_ar.ok && t_local <= 8u && (size_t)t_local * topk * 8u <= GATHER_SLOT;
    if (want_split) {
        if (!q4_hip_grouped_rms_n(d_x, d_norm_w, w.xn, n_embd, 1, eps, T)) return false;
        if (!q4_cuda_route_small(d_x + (size_t)g_rank * t_local * n_embd, d_norm_w, eps, d_router, n_expert, topk,
                                 n_embd, t_local, w.xn_l, w.logits, w.ids_l, w.wts_l))
            return false;
        if (!gather_launch(w.ids_l, w.wts_l, w.ids, w.wts, t_local * topk, st)) return false;
    } else if (!q4_cuda_route_small(d_x, d_norm_w, eps, d_router, n_expert, topk, n_embd, T, w.xn, w.recv, w.ids,
                                    w.wts)) {
        if (!q4_hip_grouped_rms_n(d_x, d_norm_w, w.xn, n_embd, 1, eps, T)) return false;
        if (!q4_hip_gemv_dd_n(Q4_T_F32, (const uint8_t *)d_router, n_expert, n_embd, w.xn, w.recv, 1.0f, T))
            return false;
        if (!q4_hip_route_pf(w.recv, w.ids, w.wts, T, n_expert, topk)) return false;
    }
    // local experts on the rows that picked them, the shared expert for this rank's tokens
    if (!q4_cuda_assign_local(w.ids, w.wts, w.atok, w.rsrc, w.rw, w.bounds, T, topk,
                              (uint32_t)g_rank * e_local, e_local, has_shared, (uint32_t)g_rank * t_local,
                              t_local))
        return false;
    if (!q4_mmq_quantize(w.xn, w.atok, w.xq, Q4_T_IQ3_S, n_embd, rows)) return false;
    const uint32_t share = 4u * (T * topk / n_expert + 1u);
    const uint32_t max_hint = t_local > share ? t_local : share;
    if (!q4_mmq_mul_id(base + og, Q4_T_IQ3_S, 2ull * n_ff, n_embd, stride, n_e, w.xq, w.bounds,
                       max_hint, rows, w.gu, 2ull * n_ff))
        return false;
    if (!q4_cuda_mmq_swiglu_quantize(w.gu, w.hq, rows, n_ff)) return false;
    if (!q4_mmq_mul_id(base + od, Q4_T_IQ3_S, n_embd, n_ff, stride, n_e, w.hq, w.bounds,
                       max_hint, rows, w.pd, n_embd))
        return false;
    if (!q4_cuda_expert_reduce_set(w.partial, w.pd, w.rsrc, w.rw, T, k1, n_embd)) return false;
    const size_t n = (size_t)T * n_embd;
    if (ar_use_kernel() && n <= AR_MAX_ELEMS && (n % 4u) == 0 && (((uintptr_t)w.partial | (uintptr_t)d_y) & 15u) == 0)
        return ar_launch(w.partial, d_y, n, st);
    EP_NCCL(ncclAllReduce(w.partial, d_y, n, ncclFloat, ncclSum, g_comm, st));
    return true;
}

// What the collectives of one layer cost by themselves, with the layer's payload sizes and
// nothing else on the stream: out[0] = the two exchanges of q4_cuda_ep_layer (gather of rows
// and picks, all-to-all of partial rows), out[1] = the one all-reduce of q4_cuda_ep_layer_ar;
// microseconds per layer, mean of `iters` back-to-back rounds.  Synchronises.
extern "C" bool q4_cuda_ep_exchange_floor_us(uint32_t t_local, uint32_t n_embd, uint32_t topk, uint32_t n_expert,
                                             uint32_t n_ff, void *d_ws, uint64_t ws_bytes, uint32_t iters,
                                             float *out2) {
    if (!g_comm || !d_ws || !out2 || iters == 0 || t_local == 0) return false;
    const uint32_t G = (uint32_t)g_world;
    const EpWs w = carve((uint8_t *)d_ws, G, t_local, topk, n_expert, n_embd, n_ff);
    if (ws_bytes < w.bytes) return false;
    cudaStream_t st = (cudaStream_t)q4_hip_stream();
    const uint32_t T = G * t_local;
    const size_t blk = (size_t)t_local * n_embd;
    cudaEvent_t e0, e1;
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return false;
    for (int form = 0; form < 2; form++) {
        for (uint32_t it = 0; it < iters + 3u; it++) {
            if (it == 3u) cudaEventRecord(e0, st);
            if (form == 0) {
                EP_NCCL(ncclGroupStart());
                EP_NCCL(ncclAllGather(w.xn_l, w.xn, (size_t)t_local * n_embd, ncclFloat, g_comm, st));
                EP_NCCL(ncclAllGather(w.ids_l, w.ids, (size_t)t_local * topk, ncclInt32, g_comm, st));
                EP_NCCL(ncclAllGather(w.wts_l, w.wts, (size_t)t_local * topk, ncclFloat, g_comm, st));
                EP_NCCL(ncclGroupEnd());
                EP_NCCL(ncclGroupStart());
                for (uint32_t p = 0; p < G; p++) {
                    EP_NCCL(ncclSend(w.partial + p * blk, blk, ncclFloat, (int)p, g_comm, st));
                    EP_NCCL(ncclRecv(w.recv + p * blk, blk, ncclFloat, (int)p, g_comm, st));
                }
                EP_NCCL(ncclGroupEnd());
            } else {   // the all-reduce q4_cuda_ep_layer_ar would use
                const size_t n = (size_t)T * n_embd;
                if (ar_use_kernel() && n <= AR_MAX_ELEMS && (n % 4u) == 0) {
                    if (!ar_launch(w.partial, w.recv, n, st)) return false;
                } else {
                    EP_NCCL(ncclAllReduce(w.partial, w.recv, n, ncclFloat, ncclSum, g_comm, st));
                }
            }
        }
        cudaEventRecord(e1, st);
        if (cudaEventSynchronize(e1) != cudaSuccess) return false;
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        out2[form] = 1e3f * ms / (float)iters;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return true;
}
