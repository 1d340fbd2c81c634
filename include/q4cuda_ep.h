/* q4cuda_ep: expert-parallel MoE layer over NCCL (libq4cuda_ep.so), one process per GPU.
 *
 * No counterpart in the reference, which is single-device (src/q4_rocm.cu:545-550).  The
 * path shards by expert: packs are independent units (src/q4_expert.c:962-982) and the
 * combine is a weighted sum per token (src/q4_rocm.cu:15739-15751).  Rank r of G keeps
 * experts [r*E/G, (r+1)*E/G) in slots 0..E/G-1 of its own arena and a copy of the shared
 * expert in slot E/G; router and norm weights are replicated; tokens are split evenly.
 * Per layer: gather of the normalised rows and picks (the dispatch), local experts on the
 * rows that picked them, all-to-all of per-token partial sums (the combine), summed at
 * the owner in rank order.  Results equal the single-GPU ones up to fp32 summation order.
 *
 * Requires libq4cuda.so initialised (q4_hip_init) on the device this process uses.
 */
#ifndef Q4CUDA_EP_H
#define Q4CUDA_EP_H

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Rank 0 makes the 128-byte NCCL id and hands it to the others by any host channel. */
bool q4_cuda_ep_unique_id(uint8_t *out128);
bool q4_cuda_ep_init(const uint8_t *id128, int rank, int world);
void q4_cuda_ep_shutdown(void);
int q4_cuda_ep_rank(void);
int q4_cuda_ep_world(void);
/* Max over ranks of one host float; synchronises (doubles as a barrier). */
bool q4_cuda_ep_allreduce_max(float *h_value);

/* One MoE layer for this rank's t_local tokens.  base/stride/og/ou/od address THIS
 * rank's arena (gate and up contiguous); d_router is the full [n_expert][n_embd] fp32
 * matrix; d_x and d_y hold t_local rows of n_embd floats (d_y overwritten); d_ws is
 * caller-owned scratch of q4_cuda_ep_layer_ws_bytes(...) bytes.  n_expert must divide
 * by the world size and n_expert/world + 1 <= 512.  Every rank calls it with the same
 * shapes; everything is enqueued on the compute stream of libq4cuda. */
uint64_t q4_cuda_ep_layer_ws_bytes(uint32_t world, uint32_t t_local, uint32_t topk,
                                   uint32_t n_expert, uint32_t n_embd, uint32_t n_ff);
bool q4_cuda_ep_layer(const uint8_t *base, uint64_t stride, uint64_t og, uint64_t ou, uint64_t od,
                      int has_shared, const float *d_x, const float *d_norm_w, float eps,
                      const float *d_router, uint32_t n_expert, uint32_t topk, uint32_t n_embd,
                      uint32_t n_ff, uint32_t t_local, float *d_y, void *d_ws, uint64_t ws_bytes);

/* The one-collective form of the same layer: d_x and d_y hold ALL world * t_local token rows,
 * identical on every rank; each rank norms and routes every token itself, runs its own experts
 * (and the shared expert for tokens [rank * t_local, (rank + 1) * t_local)), and one all-reduce
 * leaves the summed rows in d_y on every rank.  Same arguments otherwise; n_expert <= n_embd. */
bool q4_cuda_ep_layer_ar(const uint8_t *base, uint64_t stride, uint64_t og, uint64_t ou, uint64_t od,
                         int has_shared, const float *d_x, const float *d_norm_w, float eps,
                         const float *d_router, uint32_t n_expert, uint32_t topk, uint32_t n_embd,
                         uint32_t n_ff, uint32_t t_local, float *d_y, void *d_ws, uint64_t ws_bytes);
/* The all-reduce of q4_cuda_ep_layer_ar: 1 or 2 (default) = the library's own kernel over peer memory
 * (every rank exports one buffer through CUDA IPC at q4_cuda_ep_init; a rank's kernel copies its partial
 * rows there, signals every rank with release stores, waits -- bounded -- for the others' signals and sums
 * the ranks' rows in rank order with plain loads over NVLink), used when every rank could map every other
 * rank's buffer, ncclAllReduce otherwise; 0 = ncclAllReduce.  Measured inside the 48-layer job the kernel
 * is 9-10 us per layer faster.  Returns 1 when the kernel is in effect; every rank must make the same
 * call.  q4_cuda_ep_error: 0, or 0x1000 after a wait ran out (synchronises). */
int q4_cuda_ep_allreduce_mode(int mode);
/* Routing of q4_cuda_ep_layer_ar when the peer buffers are mapped: 1 = a rank routes only its own tokens
 * (norm, router product, top-k in one launch) and the ranks' picks are gathered through peer memory;
 * 0 (default) = every rank routes all tokens itself.  Every rank must make the same call. */
void q4_cuda_ep_split_routing(int on);
uint32_t q4_cuda_ep_error(void);
/* Cost of one layer's collectives alone, microseconds (mean of iters rounds with the layer's
 * payload sizes): out2[0] the two exchanges of q4_cuda_ep_layer, out2[1] the all-reduce of
 * q4_cuda_ep_layer_ar.  Synchronises; d_ws as for the layer calls. */
bool q4_cuda_ep_exchange_floor_us(uint32_t t_local, uint32_t n_embd, uint32_t topk, uint32_t n_expert,
                                  uint32_t n_ff, void *d_ws, uint64_t ws_bytes, uint32_t iters, float *out2);

#ifdef __cplusplus
}
#endif
#endif
