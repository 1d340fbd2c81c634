// Routed experts for one token with NO allocation anywhere on the call path.
//
// Who needs this: a host that cannot call cudaMalloc when the experts run.  The
// engine's planner hands every free byte of device memory to its expert slots
// and KV pages at start-up, so a later cudaMalloc simply fails; a serving loop
// inside a stream capture may not allocate at all; and a caller with a hard
// latency budget cannot afford the device-wide synchronisation an allocation
// implies.  The other entry points of this library keep their quantised
// activations in buffers that q4_hip_init() obtained with cudaMalloc.  This
// one keeps them in a fixed array that is part of the loaded library image, so
// it needs neither q4_hip_init() nor any allocator: the caller passes inputs,
// outputs and a stream, nothing else.
//
// The price is a fixed maximum size (Q4B_NA_* below, about 40 KB that every GPU
// which loads the library holds until the process exits) and one shared array:
// every call writes it, so two calls that overlap on the GPU (two streams, two
// host threads) race and must be serialised by the caller.  Nothing in the array
// has to start at zero: each call overwrites every word it later reads.
#include "q4b_tile.cuh"

#include <atomic>

#include "../../include/q4cuda.h"

extern std::atomic<uint64_t> g_q4b_launches;
bool q4b_ptr_tiled(const void *p);

#define Q4B_NA_MAX_EXPERTS 16u   // experts per call
#define Q4B_NA_MAX_IN 4096u      // widest input row (n_embd)
#define Q4B_NA_MAX_FF 2048u      // widest hidden row (n_ff)
#define Q4B_NA_MAX_DEV 64

namespace {

// Layout of the scratch: quantised x, then the quantised hidden row of each expert.
struct NoAllocScratch {
    int8_t xq[Q4B_NA_MAX_IN];
    float xd[Q4B_NA_MAX_IN / 32];
    int32_t xbs[Q4B_NA_MAX_IN / 32];
    int8_t hq[Q4B_NA_MAX_EXPERTS][Q4B_NA_MAX_FF];
    float hd[Q4B_NA_MAX_EXPERTS][Q4B_NA_MAX_FF / 32];
    int32_t hbs[Q4B_NA_MAX_EXPERTS][Q4B_NA_MAX_FF / 32];
};

// The scratch itself: device memory that exists as soon as the library is loaded.
// In host code this name is only a handle for the runtime, not a device address.
static __device__ __align__(256) unsigned char g_na_scratch[sizeof(NoAllocScratch)];

// Per device: the array's real device address (from cudaGetSymbolAddress) and whether
// the codebook constant has been filled on that device.
NoAllocScratch *g_na_ptr[Q4B_NA_MAX_DEV] = {};

// Once per device, with that device current.  No allocation: a symbol lookup and a
// 1 KB copy into constant memory.
NoAllocScratch *na_setup() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= Q4B_NA_MAX_DEV) {
        fprintf(stderr, "q4cuda: no-alloc exec: no current CUDA device\n");
        return nullptr;
    }
    if (g_na_ptr[dev]) return g_na_ptr[dev];
    void *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_na_scratch);
    if (e != cudaSuccess || !p) {
        fprintf(stderr, "q4cuda: no-alloc exec: cudaGetSymbolAddress failed: %s\n",
                cudaGetErrorString(e));
        return nullptr;
    }
    e = cudaMemcpyToSymbol(c_iq3s_codes, q4b_iq3s_codes, sizeof(q4b_iq3s_codes));
    if (e != cudaSuccess) {
        fprintf(stderr, "q4cuda: no-alloc exec: codebook upload failed: %s\n", cudaGetErrorString(e));
        return nullptr;
    }
    // The upload comes from pageable memory: the call may return before the copy has landed, and
    // it is ordered on the legacy default stream only, not against the caller's stream.  Wait
    // for it once (a synchronisation, not an allocation).
    e = cudaStreamSynchronize(0);
    if (e != cudaSuccess) {
        fprintf(stderr, "q4cuda: no-alloc exec: codebook upload did not complete: %s\n", cudaGetErrorString(e));
        return nullptr;
    }
    g_na_ptr[dev] = (NoAllocScratch *)p;
    return g_na_ptr[dev];
}

}  // namespace

extern "C" bool q4_cuda_moe_exec_noalloc(const uint8_t *base, uint64_t stride,
                                         const int32_t *d_slots, const float *d_wts, uint32_t n,
                                         uint64_t og, uint64_t ou, uint64_t od, const float *d_x,
                                         float *d_h, float *d_y, uint32_t n_ff, uint32_t in_dim,
                                         uint32_t n_embd, void *stream) {
    if (!base || !d_slots || !d_wts || !d_x || !d_h || !d_y || n == 0 || n_embd == 0) return false;
    if (n > Q4B_NA_MAX_EXPERTS || in_dim > Q4B_NA_MAX_IN || n_ff > Q4B_NA_MAX_FF) {
        fprintf(stderr,
                "q4cuda: no-alloc exec: n=%u in_dim=%u n_ff=%u exceeds the fixed scratch "
                "(at most %u experts, in_dim %u, n_ff %u)\n",
                n, in_dim, n_ff, Q4B_NA_MAX_EXPERTS, Q4B_NA_MAX_IN, Q4B_NA_MAX_FF);
        return false;
    }
    if (in_dim == 0 || n_ff == 0 || (in_dim % Q4B_QK) || (n_ff % Q4B_QK)) {
        fprintf(stderr, "q4cuda: no-alloc exec: in_dim and n_ff must be multiples of 256\n");
        return false;
    }
    const bool tiled = q4b_ptr_tiled(base);
    if (tiled && ((stride % Q4B_TILE_BYTES) || (og % Q4B_TILE_BYTES) || (ou % Q4B_TILE_BYTES) ||
                  (od % Q4B_TILE_BYTES))) {
        fprintf(stderr, "q4cuda: no-alloc exec: in a tiled arena the three matrices must start on 880-byte tiles\n");
        return false;
    }
    NoAllocScratch *s = na_setup();
    if (!s) return false;
    cudaStream_t st = (cudaStream_t)stream;
    // x -> Q8-A
    {
        const uint32_t gps = in_dim >> 5;
        quant8_k<<<(gps + 7) / 8, 256, 0, st>>>(d_x, 0, gps, gps, s->xq, s->xd, s->xbs, 0, 0, nullptr);
        g_q4b_launches++;
        if (!q4b_launch_ok("noalloc quant8 x")) return false;
    }
    // gate/up + SwiGLU
    {
        const size_t sm = 2048 + in_dim + 8 * (in_dim >> 5);
        const dim3 grid((n_ff + 7) / 8, n);
        if (tiled)
            moe_gu_k<true><<<grid, 256, sm, st>>>(base + og, base + ou, stride, d_slots, nullptr, s->xq,
                                                  s->xd, s->xbs, in_dim, n_ff, d_h);
        else
            moe_gu_k<false><<<grid, 256, sm, st>>>(base + og, base + ou, stride, d_slots, nullptr, s->xq,
                                                   s->xd, s->xbs, in_dim, n_ff, d_h);
        g_q4b_launches++;
        if (!q4b_launch_ok("noalloc moe_gu")) return false;
    }
    // h -> Q8-A, one slice per expert
    {
        const uint32_t gps = n_ff >> 5;
        const uint64_t ngr = (uint64_t)gps * n;
        quant8_k<<<(unsigned)((ngr + 7) / 8), 256, 0, st>>>(d_h, n_ff, gps, ngr, &s->hq[0][0],
                                                           &s->hd[0][0], &s->hbs[0][0], Q4B_NA_MAX_FF,
                                                           Q4B_NA_MAX_FF / 32, nullptr);
        g_q4b_launches++;
        if (!q4b_launch_ok("noalloc quant8 h")) return false;
    }
    // down + weighted combine: y += ...
    if (tiled)
        moe_ya_k<true><<<(n_embd + 7) / 8, 256, 0, st>>>(base + od, stride, d_slots, d_wts, n, nullptr,
                                                        &s->hq[0][0], &s->hd[0][0], &s->hbs[0][0],
                                                        Q4B_NA_MAX_FF, Q4B_NA_MAX_FF / 32, n_ff, n_embd,
                                                        d_y);
    else
        moe_ya_k<false><<<(n_embd + 7) / 8, 256, 0, st>>>(base + od, stride, d_slots, d_wts, n, nullptr,
                                                         &s->hq[0][0], &s->hd[0][0], &s->hbs[0][0],
                                                         Q4B_NA_MAX_FF, Q4B_NA_MAX_FF / 32, n_ff,
                                                         n_embd, d_y);
    g_q4b_launches++;
    return q4b_launch_ok("noalloc moe_ya");
}
