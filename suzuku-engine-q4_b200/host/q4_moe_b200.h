/* Host side of the MoE feed-forward path in C, above the device C ABI (include/q4cuda.h),
 * in the shape of the reference engine's all-GPU layer routines (src/q4_moe.c:2052-2133
 * q4_moe_layer_dev, src/q4_moe.c:3002-3935 q4_moe_layer_dev_n).
 *
 * The reference reaches its weights through q4_gguf / q4_store / q4_expert_cache (file
 * parsing, residency, offload), none of which is part of this path on a B200, where every
 * expert is resident: a layer is described here by the few facts those routines read out
 * of them -- the arena that holds the packs (slot e = routed expert e, one more slot = the
 * shared expert), the offsets of gate/up/down inside a pack, the router and norm tensors.
 */
#ifndef Q4_MOE_B200_H
#define Q4_MOE_B200_H

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct q4b_moe_layer {
    int arena;              /* library arena that holds this layer's packs (0..3) */
    uint32_t first_slot;    /* slot of routed expert 0; expert e is first_slot + e */
    int32_t shared_slot;    /* absolute slot of the shared expert, or -1 */
    uint32_t n_embd, n_ff, n_expert, topk;
    uint64_t og, ou, od;    /* byte offsets of gate | up | down inside a pack */
    const float *d_router;  /* device, fp32 [n_expert][n_embd] */
    const float *d_norm_w;  /* device, fp32 [n_embd], or NULL */
    float eps;
} q4b_moe_layer;

/* Pack geometry for IQ3_S experts (src/q4_expert.c:962-982): gate rows | up rows | down rows. */
uint64_t q4b_iq3s_row_bytes(uint32_t ncols);
uint64_t q4b_expert_pack_bytes(uint32_t n_embd, uint32_t n_ff);
void q4b_moe_layer_offsets(q4b_moe_layer *L);

/* Upload n_expert routed packs (+ the shared pack, may be NULL) into an arena; slot = expert id,
 * the reference's all-resident placement devtab[e] = e (src/q4_moe.c:1919-1934). */
bool q4b_moe_layer_load(q4b_moe_layer *L, int arena, const uint8_t *packs, const uint8_t *shared,
                        uint32_t n_expert, uint32_t n_embd, uint32_t n_ff);

/* The same from the tensors as a model file stores them: ffn_gate_exps / ffn_up_exps /
 * ffn_down_exps hold all experts' matrices of one kind back to back (expert e at e * slice);
 * the pack of expert e is its gate, up and down slices in that order
 * (src/q4_expert.c:962-993).  sh_* are the shared expert's three matrices (all NULL = none).
 * Packs are assembled in page-locked staging memory and queued on the copy stream. */
bool q4b_moe_layer_load_stacked(q4b_moe_layer *L, int arena, const uint8_t *gate_exps,
                                const uint8_t *up_exps, const uint8_t *down_exps,
                                const uint8_t *sh_gate, const uint8_t *sh_up, const uint8_t *sh_down,
                                uint32_t n_expert, uint32_t n_embd, uint32_t n_ff);

/* The same from a GGUF model file (host/q4_gguf_experts.h): the layer's stacked expert tensors
 * are sliced into packs expert by expert (src/q4_expert.c:962-993) and uploaded, the shared
 * expert's tensors (if the layer has them) into the slot after the last routed expert.  The
 * shapes come from the tensors.  Takes any pack the file holds; the arena is tiled only when
 * the pack is all IQ3_S.  `gguf` is a q4b_gguf the caller opened. */
bool q4b_moe_layer_load_gguf(q4b_moe_layer *L, int arena, const void *gguf, int32_t layer);

/* Scratch floats q4_moe_layer_dev needs at d_ws (src/q4_moe.c:2062-2065 sizes it the same way). */
uint64_t q4_moe_layer_dev_ws_floats(const q4b_moe_layer *L);

/* One token, the reference's fine-grained call sequence: RMSNorm, router GEMV, zero y,
 * softmax/top-k (ids come back to the host), routed + shared experts through q4_hip_moe_exec.
 * d_x is the pre-norm hidden row; d_y receives the layer's output. */
bool q4_moe_layer_dev(const q4b_moe_layer *L, const float *d_x, float *d_y, float *d_ws);

/* The same layer through the single fused call. */
bool q4_moe_layer_dev_fused(const q4b_moe_layer *L, const float *d_x, float *d_y, int32_t *d_ids,
                            float *d_wts);

/* n_tok tokens (prefill chunk, verify window, batched decode); d_ws of
 * q4_cuda_moe_layer_n_ws_bytes() bytes. */
bool q4_moe_layer_dev_n(const q4b_moe_layer *L, const float *d_x, float *d_y, uint32_t n_tok,
                        void *d_ws, uint64_t ws_bytes);

#ifdef __cplusplus
}
#endif
#endif
