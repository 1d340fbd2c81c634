// Lifecycle, memory, expert arenas, graphs and timers of the q4cuda library.
// Counterpart of the reference device layer's plumbing (src/q4_rocm.cu:507-560,
// 661-801 for streams and arenas); the arithmetic lives in the other files.
#include "q4b_tile.cuh"

#include <atomic>
#include <string.h>

#include "../../include/q4cuda.h"

#define Q4B_IQ3S_CODES_DECL static const
#include "iq2s_codes.h"
#include "iq3s_codes.h"
#include "iq3xxs_codes.h"

Q4bState g_q4b = {};
bool q4b_fused_warm();   // q4b_stack.cu: scratch of the persistent decode kernel
void q4b_fused_shutdown();
void q4b_stack_forget_host(const void *h);
static void timer_marks_shutdown();
bool q4b_window_warm();  // q4b_grouped.cu: scratch of the verify-window path
bool q4b_elem_warm();    // q4b_elem.cu: lists of the per-token exec, rows of the 2..8-row GEMV
void q4b_elem_shutdown();
bool q4b_mmvq_warm();    // q4b_mmvq.cu: quantised rows of the dense 8-bit product
bool q4b_route_small_warm();   // q4b_decode.cu: counters of the one-launch routing
void q4b_route_small_shutdown();
void q4b_mmvq_shutdown();
bool q4b_wbuf_tiled(const void *p);
bool q4b_mmq_tc_warm();  // q4b_grouped.cu: tensor-core grouped product (optional)
std::atomic<uint64_t> g_q4b_launches{0};

namespace {

struct Arena {
    uint8_t *base;
    uint32_t n_slots;
    uint64_t stride;
    uint64_t bytes;
    bool tiled;  // slots hold the tiled IQ3_S format (q4b_tile.cuh)
};
Arena g_arena[4] = {};

// Environment knob, read once: Q4B_TILED=0 keeps arenas in the engine's byte
// layout (the fused kernels then do not apply and the launch chain runs).
int g_tiled_default = -1;
bool tiled_default() {
    if (g_tiled_default < 0) {
        const char *e = getenv("Q4B_TILED");
        g_tiled_default = !(e && e[0] == '0');
    }
    return g_tiled_default != 0;
}

// In-place regrouping of runs of eight 110-byte super-blocks into tiles
// (forward) or back (inverse).  One warp per tile via shared memory.
template <bool FORWARD>
__global__ void tile_permute_k(uint8_t *data, uint64_t n_tiles) {
    __shared__ __align__(16) uint8_t buf[8][Q4B_TILE_BYTES];
    const uint32_t w = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint64_t t = (uint64_t)blockIdx.x * 8u + w;
    if (t >= n_tiles) return;
    uint8_t *p = data + t * Q4B_TILE_BYTES;
    uint8_t *b = buf[w];
    for (uint32_t i = lane; i < Q4B_TILE_BYTES / 16; i += 32)
        reinterpret_cast<uint4 *>(b)[i] = reinterpret_cast<const uint4 *>(p)[i];
    __syncwarp();
    // engine layout of block k: 110k + {0: d, 2: qs[64], 66: qh[8], 74: signs[32], 106: scales[4]}
    for (uint32_t i = lane; i < Q4B_TILE_BYTES; i += 32) {
        const uint32_t k = i / 110u, o = i - k * 110u;
        uint32_t to;
        if (o < 2)
            to = Q4B_TILE_OFF_D + 2 * k + o;
        else if (o < 66)
            to = Q4B_TILE_OFF_QS + 64 * k + (o - 2);
        else if (o < 74)
            to = Q4B_TILE_OFF_QH + 8 * k + (o - 66);
        else if (o < 106)
            to = Q4B_TILE_OFF_SG + 32 * k + (o - 74);
        else
            to = Q4B_TILE_OFF_SC + 4 * k + (o - 106);
        if (o >= 74 && o < 106) continue;  // sign words: handled below, as words
        if (FORWARD)
            p[to] = b[i];
        else
            p[i] = b[to];
    }
    for (uint32_t g = lane; g < 64; g += 32) {  // 64 sign words per tile
        const uint32_t k = g >> 3, ib = g & 7u;
        const uint32_t eng = 110u * k + 74u + 4u * ib, til = Q4B_TILE_OFF_SG + 32u * k + 4u * ib;
        if (FORWARD) {
            const uint32_t w32 = b[eng] | (b[eng + 1] << 8) | (b[eng + 2] << 16) | ((uint32_t)b[eng + 3] << 24);
            *reinterpret_cast<uint32_t *>(p + til) = q4b_sign_permute(w32);
        } else {
            const uint32_t w32 = q4b_sign_unpermute(*reinterpret_cast<const uint32_t *>(b + til));
            p[eng] = (uint8_t)w32;
            p[eng + 1] = (uint8_t)(w32 >> 8);
            p[eng + 2] = (uint8_t)(w32 >> 16);
            p[eng + 3] = (uint8_t)(w32 >> 24);
        }
    }
}

bool launch_tile_permute(uint8_t *data, uint64_t bytes, bool forward, cudaStream_t st) {
    const uint64_t n_tiles = bytes / Q4B_TILE_BYTES;
    if (n_tiles == 0) return true;
    const unsigned nb = (unsigned)((n_tiles + 7) / 8);
    if (forward)
        tile_permute_k<true><<<nb, 256, 0, st>>>(data, n_tiles);
    else
        tile_permute_k<false><<<nb, 256, 0, st>>>(data, n_tiles);
    g_q4b_launches++;
    return q4b_launch_ok("tile_permute");
}

cudaEvent_t g_ev0, g_ev1;
bool g_capturing = false;

bool alloc_scratch() {
    Q4bState &s = g_q4b;
    if (s.xq) return true;
    const size_t nq = (size_t)Q4B_XQ_SLICES * Q4B_XQ_MAXLEN;
    Q4B_CHECK(cudaMalloc(&s.xq, nq));
    Q4B_CHECK(cudaMalloc(&s.xd, nq / 32 * sizeof(float)));
    Q4B_CHECK(cudaMalloc(&s.xbs, nq / 32 * sizeof(int32_t)));
    Q4B_CHECK(cudaMalloc(&s.xn, (size_t)Q4B_MAX_TOK * Q4B_XQ_MAXLEN * sizeof(float)));
    Q4B_CHECK(cudaMalloc(&s.logits, (size_t)Q4B_MAX_TOK * 1024 * sizeof(float)));
    Q4B_CHECK(cudaMalloc(&s.r_ids, (size_t)Q4B_MAX_TOK * 64 * sizeof(int32_t)));
    Q4B_CHECK(cudaMalloc(&s.r_wts, (size_t)Q4B_MAX_TOK * 64 * sizeof(float)));
    Q4B_CHECK(cudaMalloc(&s.r_cnt, (size_t)Q4B_MAX_TOK * sizeof(int32_t)));
    Q4B_CHECK(cudaMalloc(&s.hbuf, nq * sizeof(float)));
    q4b_mmq_tc_warm();  // without it the grouped product stays on the CUDA cores
    return q4b_fused_warm() && q4b_window_warm() && q4b_elem_warm() && q4b_mmvq_warm() && q4b_route_small_warm();
}

}  // namespace

extern "C" bool q4_hip_init(void) {
    Q4bState &s = g_q4b;
    if (s.ok) return true;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
        fprintf(stderr, "q4cuda: no CUDA device; this library has no CPU path\n");
        return false;
    }
    int dev = 0;
    Q4B_CHECK(cudaGetDevice(&dev));
    cudaDeviceProp p;
    Q4B_CHECK(cudaGetDeviceProperties(&p, dev));
    if (p.major != 10) {
        fprintf(stderr, "q4cuda: device %d is sm_%d%d; the kernels are built for sm_100a only\n",
                dev, p.major, p.minor);
        return false;
    }
    s.device = dev;
    s.n_sm = p.multiProcessorCount;
    Q4B_CHECK(cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking));
    Q4B_CHECK(cudaStreamCreateWithFlags(&s.copy_stream, cudaStreamNonBlocking));
    Q4B_CHECK(cudaStreamCreateWithFlags(&s.aux_stream, cudaStreamNonBlocking));
    Q4B_CHECK(cudaEventCreateWithFlags(&s.ev_fork, cudaEventDisableTiming));
    Q4B_CHECK(cudaEventCreateWithFlags(&s.ev_join, cudaEventDisableTiming));
    Q4B_CHECK(cudaMemcpyToSymbol(c_iq3s_codes, q4b_iq3s_codes, sizeof(q4b_iq3s_codes)));
    Q4B_CHECK(cudaHostAlloc(&s.es_h, 64 * sizeof(int32_t), cudaHostAllocMapped));
    Q4B_CHECK(cudaHostAlloc(&s.ew_h, 64 * sizeof(float), cudaHostAllocMapped));
    Q4B_CHECK(cudaHostAlloc(&s.en_h, sizeof(int32_t), cudaHostAllocMapped));
    Q4B_CHECK(cudaHostGetDevicePointer(&s.es_d, s.es_h, 0));
    Q4B_CHECK(cudaHostGetDevicePointer(&s.ew_d, s.ew_h, 0));
    Q4B_CHECK(cudaHostGetDevicePointer(&s.en_d, s.en_h, 0));
    Q4B_CHECK(cudaHostAlloc(&s.topk_ids_h, 64 * sizeof(int32_t), cudaHostAllocDefault));
    Q4B_CHECK(cudaHostAlloc(&s.topk_wts_h, 64 * sizeof(float), cudaHostAllocDefault));
    Q4B_CHECK(cudaMalloc(&s.topk_ids_d, 64 * sizeof(int32_t)));
    Q4B_CHECK(cudaMalloc(&s.topk_wts_d, 64 * sizeof(float)));
    Q4B_CHECK(cudaMalloc(&s.err_d, sizeof(uint32_t)));
    Q4B_CHECK(cudaMemset(s.err_d, 0, sizeof(uint32_t)));
    s.flag_h = s.flag_d = nullptr;
    s.flag_epoch = 0;
    if (cudaHostAlloc((void **)&s.flag_h, 64, cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess &&
        cudaHostGetDevicePointer((void **)&s.flag_d, s.flag_h, 0) == cudaSuccess) {
        *s.flag_h = 0;
    } else {   // no mapped host memory: the host-buffer call keeps its copy + sync form
        cudaGetLastError();
        if (s.flag_h) cudaFreeHost(s.flag_h);
        s.flag_h = s.flag_d = nullptr;
    }
    Q4B_CHECK(cudaHostAlloc(&s.err_h, sizeof(uint32_t), cudaHostAllocDefault));
    {
        uint32_t codes[512];
        for (int i = 0; i < 512; i++) {
            const uint32_t c = q4b_iq3s_codes[i];
            codes[i] = (c & 7u) | ((c & 0x38u) << 5) | ((c & 0x1c0u) << 10) | ((c & 0xe00u) << 15);
        }
        Q4B_CHECK(cudaMalloc(&s.codes_d, sizeof(codes)));
        Q4B_CHECK(cudaMemcpy(s.codes_d, codes, sizeof(codes), cudaMemcpyHostToDevice));
    }
    {   // the two small codebooks, expanded from their packed level numbers to magnitude bytes
        static const uint8_t l3[8] = {4, 12, 20, 28, 36, 44, 52, 62}, l2[4] = {8, 25, 43, 0};
        static uint32_t g3[256];
        static uint32_t g2[2048];
        for (int i = 0; i < 256; i++) {
            g3[i] = 0;
            for (int j = 0; j < 4; j++) g3[i] |= (uint32_t)l3[(q4b_iq3xxs_codes[i] >> (3 * j)) & 7] << (8 * j);
        }
        for (int i = 0; i < 1024; i++)
            for (int h = 0; h < 2; h++) {
                g2[2 * i + h] = 0;
                for (int j = 0; j < 4; j++)
                    g2[2 * i + h] |= (uint32_t)l2[(q4b_iq2s_codes[i] >> (2 * (4 * h + j))) & 3] << (8 * j);
            }
        Q4B_CHECK(cudaMalloc(&s.grid3xxs_d, sizeof g3));
        Q4B_CHECK(cudaMemcpy(s.grid3xxs_d, g3, sizeof g3, cudaMemcpyHostToDevice));
        Q4B_CHECK(cudaMalloc(&s.grid2s_d, sizeof g2));
        Q4B_CHECK(cudaMemcpy(s.grid2s_d, g2, sizeof g2, cudaMemcpyHostToDevice));
    }
    Q4B_CHECK(cudaEventCreate(&g_ev0));
    Q4B_CHECK(cudaEventCreate(&g_ev1));
    if (!alloc_scratch()) return false;
    s.ok = true;
    return true;
}

extern "C" void q4_hip_moe_scratch_warm(void) {
    if (g_q4b.ok) alloc_scratch();
}

extern "C" void q4_hip_shutdown(void) {
    Q4bState &s = g_q4b;
    if (!s.ok) return;
    cudaDeviceSynchronize();
    for (int a = 0; a < 4; a++) {
        if (g_arena[a].base) cudaFree(g_arena[a].base);
        g_arena[a] = Arena{};
    }
    q4b_elem_shutdown();
    q4b_mmvq_shutdown();
    q4b_route_small_shutdown();
    q4b_fused_shutdown();
    q4b_stack_forget_host(nullptr);
    cudaFree(s.xq);
    cudaFree(s.xd);
    cudaFree(s.xbs);
    cudaFree(s.xn);
    cudaFree(s.logits);
    cudaFree(s.r_ids);
    cudaFree(s.r_wts);
    cudaFree(s.r_cnt);
    cudaFree(s.hbuf);
    cudaFreeHost(s.es_h);
    cudaFreeHost(s.ew_h);
    cudaFreeHost(s.en_h);
    cudaFreeHost(s.topk_ids_h);
    cudaFreeHost(s.topk_wts_h);
    cudaFree(s.topk_ids_d);
    cudaFree(s.topk_wts_d);
    cudaFree(s.err_d);
    if (s.flag_h) cudaFreeHost(s.flag_h);
    s.flag_h = s.flag_d = nullptr;
    cudaFree(s.codes_d);
    cudaFree(s.grid3xxs_d);
    cudaFree(s.grid2s_d);
    s.grid3xxs_d = nullptr;
    s.grid2s_d = nullptr;
    cudaFreeHost(s.err_h);
    cudaEventDestroy(g_ev0);
    cudaEventDestroy(g_ev1);
    timer_marks_shutdown();
    cudaStreamDestroy(s.stream);
    cudaStreamDestroy(s.copy_stream);
    cudaStreamDestroy(s.aux_stream);
    cudaEventDestroy(s.ev_fork);
    cudaEventDestroy(s.ev_join);
    s = Q4bState{};
}

extern "C" bool q4_hip_ok(void) { return g_q4b.ok; }
extern "C" void *q4_hip_stream(void) { return (void *)g_q4b.stream; }
extern "C" void q4_hip_sync(void) {
    if (g_q4b.ok) cudaDeviceSynchronize();
}
extern "C" bool q4_hip_stream_sync(void) {
    return g_q4b.ok && cudaStreamSynchronize(g_q4b.stream) == cudaSuccess;
}

extern "C" void *q4_hip_malloc(size_t n) {
    if (!g_q4b.ok || n == 0) return nullptr;
    void *p = nullptr;
    if (cudaMalloc(&p, n) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return p;
}
extern "C" void q4_hip_free(void *p) {
    if (g_q4b.ok && p) cudaFree(p);
}
extern "C" bool q4_hip_h2d(void *d, const void *h, size_t n) {
    if (!g_q4b.ok || !d || !h) return false;
    Q4B_CHECK(cudaMemcpyAsync(d, h, n, cudaMemcpyHostToDevice, g_q4b.stream));
    Q4B_CHECK(cudaStreamSynchronize(g_q4b.stream));
    return true;
}
extern "C" bool q4_hip_d2h(void *h, const void *d, size_t n) {
    if (!g_q4b.ok || !d || !h) return false;
    Q4B_CHECK(cudaMemcpyAsync(h, d, n, cudaMemcpyDeviceToHost, g_q4b.stream));
    Q4B_CHECK(cudaStreamSynchronize(g_q4b.stream));
    return true;
}
extern "C" bool q4_hip_h2d_async(void *d, const void *h, uint64_t n) {
    if (!g_q4b.ok || !d || !h) return false;
    Q4B_CHECK(cudaMemcpyAsync(d, h, n, cudaMemcpyHostToDevice, g_q4b.stream));
    return true;
}
extern "C" bool q4_hip_d2h_async(void *h, const void *d, uint64_t n) {
    if (!g_q4b.ok || !d || !h) return false;
    Q4B_CHECK(cudaMemcpyAsync(h, d, n, cudaMemcpyDeviceToHost, g_q4b.stream));
    return true;
}
extern "C" bool q4_hip_copy_async(float *d, const float *s, uint64_t n) {
    if (!g_q4b.ok || !d || !s) return false;
    Q4B_CHECK(cudaMemcpyAsync(d, s, n * sizeof(float), cudaMemcpyDeviceToDevice, g_q4b.stream));
    return true;
}
extern "C" uint64_t q4_hip_vram_free(void) {
    if (!g_q4b.ok) return 0;
    size_t f = 0, t = 0;
    if (cudaMemGetInfo(&f, &t) != cudaSuccess) return 0;
    return f;
}

__global__ static void fill_k(float *d, float v, uint64_t n) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t step = (uint64_t)gridDim.x * blockDim.x;
    for (; i < n; i += step) d[i] = v;
}
extern "C" bool q4_hip_fill(float *d, float v, uint64_t n) {
    if (!g_q4b.ok || !d || n == 0) return false;
    uint64_t nb = (n + 255) / 256;
    if (nb > 4096) nb = 4096;
    fill_k<<<(unsigned)nb, 256, 0, g_q4b.stream>>>(d, v, n);
    g_q4b_launches++;
    return q4b_launch_ok("fill");
}

// ---- arenas ----
extern "C" bool q4_hip_experts_alloc_a(int arena, uint32_t n_slots, uint64_t slot_bytes) {
    if (!g_q4b.ok || arena < 0 || arena >= 4 || n_slots == 0 || slot_bytes == 0) return false;
    Arena &a = g_arena[arena];
    if (a.base) return false;
    // 256 bytes of zeroed slack after the last slot: kernels that fetch whole
    // 16-byte chunks may read a few bytes past the end of the last pack.
    const uint64_t bytes = (uint64_t)n_slots * slot_bytes + 256;
    if (cudaMalloc(&a.base, bytes) != cudaSuccess) {
        cudaGetLastError();
        a.base = nullptr;
        return false;
    }
    cudaMemsetAsync(a.base + bytes - 256, 0, 256, g_q4b.stream);
    a.n_slots = n_slots;
    a.stride = slot_bytes;
    a.bytes = bytes;
    // Tiled only where the slot can hold nothing but an all-IQ3_S pack: gate, up and down of
    // widths that are multiples of 256 make 330 * n_ff * n_embd / 256 = a multiple of 84480
    // bytes.  A multiple of 880 alone is not enough: a pack with an IQ4_NL down projection can
    // have such a size, and tiling its bytes on upload would scramble it (such a pack stays in
    // the engine's byte order; the exec calls refuse a non-IQ3_S part on a tiled arena before
    // anything is enqueued).
    a.tiled = tiled_default() && (slot_bytes % (g_tiled_default == 2 ? Q4B_TILE_BYTES : 84480u)) == 0;
    return true;
}
extern "C" void q4_hip_experts_free_a(int arena) {
    if (!g_q4b.ok || arena < 0 || arena >= 4) return;
    if (g_arena[arena].base) {
        cudaDeviceSynchronize();
        cudaFree(g_arena[arena].base);
    }
    g_arena[arena] = Arena{};
}
extern "C" uint32_t q4_hip_experts_n_a(int arena) {
    return (arena >= 0 && arena < 4) ? g_arena[arena].n_slots : 0;
}
extern "C" bool q4_hip_experts_put_async_a(int arena, uint32_t slot, const uint8_t *host,
                                           uint64_t n) {
    if (!g_q4b.ok || arena < 0 || arena >= 4 || !host) return false;
    Arena &a = g_arena[arena];
    if (!a.base || slot >= a.n_slots || n > a.stride) return false;
    if (a.tiled && (n % Q4B_TILE_BYTES)) return false;
    Q4B_CHECK(cudaMemcpyAsync(a.base + (uint64_t)slot * a.stride, host, n, cudaMemcpyHostToDevice,
                              g_q4b.copy_stream));
    if (a.tiled && !launch_tile_permute(a.base + (uint64_t)slot * a.stride, n, true, g_q4b.copy_stream))
        return false;
    return true;
}
extern "C" bool q4_hip_experts_put_a(int arena, uint32_t slot, const uint8_t *host, uint64_t n) {
    if (!q4_hip_experts_put_async_a(arena, slot, host, n)) return false;
    Q4B_CHECK(cudaStreamSynchronize(g_q4b.copy_stream));
    return true;
}
extern "C" const uint8_t *q4_hip_experts_dev_a(int arena, uint32_t slot) {
    if (arena < 0 || arena >= 4 || !g_arena[arena].base || slot >= g_arena[arena].n_slots)
        return nullptr;
    return g_arena[arena].base + (uint64_t)slot * g_arena[arena].stride;
}
extern "C" const uint8_t *q4_hip_experts_base_a(int arena) {
    return (arena >= 0 && arena < 4) ? g_arena[arena].base : nullptr;
}
extern "C" uint64_t q4_hip_experts_stride_a(int arena) {
    return (arena >= 0 && arena < 4) ? g_arena[arena].stride : 0;
}
extern "C" bool q4_hip_experts_alloc(uint32_t n, uint64_t b) { return q4_hip_experts_alloc_a(0, n, b); }
extern "C" void q4_hip_experts_free(void) { q4_hip_experts_free_a(0); }
extern "C" uint32_t q4_hip_experts_n(void) { return q4_hip_experts_n_a(0); }
extern "C" bool q4_hip_experts_put(uint32_t slot, const uint8_t *h, uint64_t n) {
    return q4_hip_experts_put_a(0, slot, h, n);
}
extern "C" bool q4_hip_experts_put_async(uint32_t slot, const uint8_t *h, uint64_t n) {
    return q4_hip_experts_put_async_a(0, slot, h, n);
}
extern "C" const uint8_t *q4_hip_experts_dev(uint32_t slot) { return q4_hip_experts_dev_a(0, slot); }
extern "C" void q4_hip_copy_wait(void) {
    if (g_q4b.ok) cudaStreamSynchronize(g_q4b.copy_stream);
}

// ---- graphs ----
extern "C" int q4_hip_graph_begin(void) {
    if (!g_q4b.ok || g_capturing) return 0;
    if (cudaStreamBeginCapture(g_q4b.stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    g_capturing = true;
    return 1;
}
extern "C" void *q4_hip_graph_end(void) {
    if (!g_q4b.ok || !g_capturing) return nullptr;
    g_capturing = false;
    cudaGraph_t g = nullptr;
    if (cudaStreamEndCapture(g_q4b.stream, &g) != cudaSuccess || !g) {
        cudaGetLastError();
        return nullptr;
    }
    cudaGraphExec_t ex = nullptr;
    cudaError_t e = cudaGraphInstantiate(&ex, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return (void *)ex;
}
extern "C" uint32_t q4_hip_graph_nodes(void *exec) {
    (void)exec;
    return 0;  // the reference reports node counts for diagnostics only
}
extern "C" bool q4_hip_graph_launch(void *exec) {
    if (!g_q4b.ok || !exec) return false;
    Q4B_CHECK(cudaGraphLaunch((cudaGraphExec_t)exec, g_q4b.stream));
    return true;
}
extern "C" void q4_hip_graph_free(void *exec) {
    if (exec) cudaGraphExecDestroy((cudaGraphExec_t)exec);
}

// ---- timers / counters ----
extern "C" bool q4_cuda_timer_begin(void) {
    if (!g_q4b.ok) return false;
    Q4B_CHECK(cudaEventRecord(g_ev0, g_q4b.stream));
    return true;
}
extern "C" bool q4_cuda_timer_end(void) {
    if (!g_q4b.ok) return false;
    Q4B_CHECK(cudaEventRecord(g_ev1, g_q4b.stream));
    return true;
}
extern "C" float q4_cuda_timer_ms(void) {
    if (!g_q4b.ok) return -1.f;
    if (cudaEventSynchronize(g_ev1) != cudaSuccess) return -1.f;
    float ms = -1.f;
    if (cudaEventElapsedTime(&ms, g_ev0, g_ev1) != cudaSuccess) return -1.f;
    return ms;
}
// A row of marks on the compute stream (events created on first use, kept until shutdown): a
// benchmark that repeats a timed region marks its boundaries and reads the intervals afterwards.
static cudaEvent_t g_marks[Q4B_MAX_MARKS];
static uint32_t g_marks_made = 0;
extern "C" bool q4_cuda_timer_mark(uint32_t i) {
    if (!g_q4b.ok || i >= Q4B_MAX_MARKS) return false;
    while (g_marks_made <= i) {
        Q4B_CHECK(cudaEventCreate(&g_marks[g_marks_made]));
        g_marks_made++;
    }
    Q4B_CHECK(cudaEventRecord(g_marks[i], g_q4b.stream));
    return true;
}
extern "C" float q4_cuda_timer_between_ms(uint32_t i, uint32_t j) {
    if (!g_q4b.ok || i >= g_marks_made || j >= g_marks_made) return -1.f;
    if (cudaEventSynchronize(g_marks[j]) != cudaSuccess) return -1.f;
    float ms = -1.f;
    if (cudaEventElapsedTime(&ms, g_marks[i], g_marks[j]) != cudaSuccess) return -1.f;
    return ms;
}
static void timer_marks_shutdown() {
    for (uint32_t i = 0; i < g_marks_made; i++) cudaEventDestroy(g_marks[i]);
    g_marks_made = 0;
}
extern "C" uint64_t q4_cuda_launch_count(void) { return g_q4b_launches.load(); }
extern "C" uint32_t q4_cuda_device_error(void) {
    if (!g_q4b.ok) return 0xffffffffu;
    if (cudaMemcpyAsync(g_q4b.err_h, g_q4b.err_d, 4, cudaMemcpyDeviceToHost, g_q4b.stream) !=
            cudaSuccess ||
        cudaStreamSynchronize(g_q4b.stream) != cudaSuccess)
        return 0xffffffffu;
    const uint32_t v = *g_q4b.err_h;
    if (v) cudaMemsetAsync(g_q4b.err_d, 0, 4, g_q4b.stream);
    return v;
}

// ---- pinned host memory (reference: q4_hip_host_alloc_coh, src/q4.h:1251-1252) ----
extern "C" void *q4_hip_host_alloc_coh(size_t n) {
    if (!g_q4b.ok || n == 0) return nullptr;
    void *p = nullptr;
    // mapped as well as pinned: kernels may write results straight into it
    if (cudaHostAlloc(&p, n, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return p;
}
extern "C" void q4_hip_host_free_coh(void *p) {
    if (g_q4b.ok && p) {
        q4b_stack_forget_host(p);   // a decode plan may hold this buffer's device alias
        cudaFreeHost(p);
    }
}

// ---- tiled arenas ----
bool q4b_ptr_tiled(const void *p) {
    const uint8_t *q = (const uint8_t *)p;
    for (int a = 0; a < 4; a++)
        if (g_arena[a].base && g_arena[a].tiled && q >= g_arena[a].base &&
            q < g_arena[a].base + g_arena[a].bytes)
            return true;
    return q4b_wbuf_tiled(p);   // a gathered copy of a tiled arena keeps its byte order
}
extern "C" void q4_cuda_set_tiled_default(int on) { g_tiled_default = on == 2 ? 2 : (on ? 1 : 0); }
extern "C" int q4_cuda_experts_tiled_a(int arena) {
    return (arena >= 0 && arena < 4 && g_arena[arena].base && g_arena[arena].tiled) ? 1 : 0;
}
extern "C" bool q4_cuda_experts_retile_a(int arena, uint32_t first_slot, uint32_t n_slots) {
    if (!g_q4b.ok || arena < 0 || arena >= 4) return false;
    Arena &a = g_arena[arena];
    if (!a.base || !a.tiled || (uint64_t)first_slot + n_slots > a.n_slots || n_slots == 0) return false;
    return launch_tile_permute(a.base + (uint64_t)first_slot * a.stride, (uint64_t)n_slots * a.stride,
                               true, g_q4b.stream);
}
extern "C" bool q4_cuda_experts_get_a(int arena, uint32_t slot, uint8_t *host, uint64_t n) {
    if (!g_q4b.ok || arena < 0 || arena >= 4 || !host) return false;
    Arena &a = g_arena[arena];
    if (!a.base || slot >= a.n_slots || n > a.stride || n == 0) return false;
    uint8_t *src = a.base + (uint64_t)slot * a.stride;
    if (!a.tiled) {
        Q4B_CHECK(cudaMemcpyAsync(host, src, n, cudaMemcpyDeviceToHost, g_q4b.stream));
        Q4B_CHECK(cudaStreamSynchronize(g_q4b.stream));
        return true;
    }
    if (n % Q4B_TILE_BYTES) return false;
    uint8_t *tmp = nullptr;
    if (cudaMalloc(&tmp, n) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    bool ok = cudaMemcpyAsync(tmp, src, n, cudaMemcpyDeviceToDevice, g_q4b.stream) == cudaSuccess &&
              launch_tile_permute(tmp, n, false, g_q4b.stream) &&
              cudaMemcpyAsync(host, tmp, n, cudaMemcpyDeviceToHost, g_q4b.stream) == cudaSuccess &&
              cudaStreamSynchronize(g_q4b.stream) == cudaSuccess;
    cudaFree(tmp);
    return ok;
}
