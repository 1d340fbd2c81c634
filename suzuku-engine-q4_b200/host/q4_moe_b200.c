/* See q4_moe_b200.h.  Plain C over include/q4cuda.h; no CUDA headers, no other dependency. */
#include "q4_moe_b200.h"

#include <stddef.h>
#include <string.h>

#include "../../include/q4cuda.h"
#include "q4_gguf_experts.h"

uint64_t q4b_iq3s_row_bytes(uint32_t ncols) { return (uint64_t)(ncols / 256u) * 110u; }

uint64_t q4b_expert_pack_bytes(uint32_t n_embd, uint32_t n_ff) {
    return 2ull * n_ff * q4b_iq3s_row_bytes(n_embd) + (uint64_t)n_embd * q4b_iq3s_row_bytes(n_ff);
}

void q4b_moe_layer_offsets(q4b_moe_layer *L) {
    L->og = 0;
    L->ou = (uint64_t)L->n_ff * q4b_iq3s_row_bytes(L->n_embd);
    L->od = 2ull * L->n_ff * q4b_iq3s_row_bytes(L->n_embd);
}

bool q4b_moe_layer_load(q4b_moe_layer *L, int arena, const uint8_t *packs, const uint8_t *shared,
                        uint32_t n_expert, uint32_t n_embd, uint32_t n_ff) {
    if (!L || !packs || n_expert == 0 || (n_embd % 256u) || (n_ff % 256u)) return false;
    const uint64_t pb = q4b_expert_pack_bytes(n_embd, n_ff);
    if (!q4_hip_experts_alloc_a(arena, n_expert + (shared ? 1u : 0u), pb)) return false;
    for (uint32_t e = 0; e < n_expert; e++)
        if (!q4_hip_experts_put_async_a(arena, e, packs + (uint64_t)e * pb, pb)) return false;
    if (shared && !q4_hip_experts_put_async_a(arena, n_expert, shared, pb)) return false;
    q4_hip_copy_wait();
    L->arena = arena;
    L->first_slot = 0;
    L->shared_slot = shared ? (int32_t)n_expert : -1;
    L->n_embd = n_embd;
    L->n_ff = n_ff;
    L->n_expert = n_expert;
    q4b_moe_layer_offsets(L);
    return true;
}

bool q4b_moe_layer_load_stacked(q4b_moe_layer *L, int arena, const uint8_t *gate_exps,
                                const uint8_t *up_exps, const uint8_t *down_exps,
                                const uint8_t *sh_gate, const uint8_t *sh_up, const uint8_t *sh_down,
                                uint32_t n_expert, uint32_t n_embd, uint32_t n_ff) {
    if (!L || !gate_exps || !up_exps || !down_exps || n_expert == 0 || (n_embd % 256u) || (n_ff % 256u))
        return false;
    const bool sh = sh_gate && sh_up && sh_down;
    if (!sh && (sh_gate || sh_up || sh_down)) return false;
    const uint64_t sg = (uint64_t)n_ff * q4b_iq3s_row_bytes(n_embd), su = sg;
    const uint64_t sd = (uint64_t)n_embd * q4b_iq3s_row_bytes(n_ff), pb = sg + su + sd;
    if (!q4_hip_experts_alloc_a(arena, n_expert + (sh ? 1u : 0u), pb)) return false;
    /* two staging packs: one is filled while the other's upload is in flight */
    uint8_t *stage = (uint8_t *)q4_hip_host_alloc_coh(2 * pb);
    if (!stage) return false;
    bool ok = true;
    for (uint32_t e = 0; ok && e < n_expert + (sh ? 1u : 0u); e++) {
        uint8_t *p = stage + (uint64_t)(e & 1u) * pb;
        if (e >= 2 && (e & 1u) == 0) q4_hip_copy_wait();   /* both staging packs may be in flight */
        const bool shared = e == n_expert;
        memcpy(p, shared ? sh_gate : gate_exps + (uint64_t)e * sg, sg);
        memcpy(p + sg, shared ? sh_up : up_exps + (uint64_t)e * su, su);
        memcpy(p + sg + su, shared ? sh_down : down_exps + (uint64_t)e * sd, sd);
        ok = q4_hip_experts_put_async_a(arena, e, p, pb);
    }
    q4_hip_copy_wait();
    q4_hip_host_free_coh(stage);
    if (!ok) return false;
    L->arena = arena;
    L->first_slot = 0;
    L->shared_slot = sh ? (int32_t)n_expert : -1;
    L->n_embd = n_embd;
    L->n_ff = n_ff;
    L->n_expert = n_expert;
    q4b_moe_layer_offsets(L);
    return true;
}

bool q4b_moe_layer_load_gguf(q4b_moe_layer *L, int arena, const void *gguf, int32_t layer) {
    const q4b_gguf *g = (const q4b_gguf *)gguf;
    const q4b_gguf_tensor *tg, *tu, *td;
    uint64_t og, ou, od, pb;
    uint32_t n_expert;
    if (!L || !q4b_gguf_expert_parts(g, layer, &tg, &tu, &td, &og, &ou, &od, &pb, &n_expert)) return false;
    uint8_t *stage = (uint8_t *)q4_hip_host_alloc_coh(2 * pb);
    if (!stage) return false;
    const bool sh = q4b_gguf_read_shared_pack(g, layer, stage, pb) == (int64_t)pb;
    bool ok = q4_hip_experts_alloc_a(arena, n_expert + (sh ? 1u : 0u), pb);
    if (ok && sh) ok = q4_hip_experts_put_async_a(arena, n_expert, stage, pb);
    if (ok && sh) q4_hip_copy_wait();
    for (uint32_t e = 0; ok && e < n_expert; e++) {
        uint8_t *p = stage + (uint64_t)(e & 1u) * pb;
        if (e >= 2 && (e & 1u) == 0) q4_hip_copy_wait();   /* both staging packs may be in flight */
        ok = q4b_gguf_read_pack(g, layer, (int32_t)e, p) == (int64_t)pb &&
             q4_hip_experts_put_async_a(arena, e, p, pb);
    }
    q4_hip_copy_wait();
    q4_hip_host_free_coh(stage);
    if (!ok) return false;
    L->arena = arena;
    L->first_slot = 0;
    L->shared_slot = sh ? (int32_t)n_expert : -1;
    L->n_embd = (uint32_t)tg->ne[0];
    L->n_ff = (uint32_t)tg->ne[1];
    L->n_expert = n_expert;
    L->og = og;
    L->ou = ou;
    L->od = od;
    return true;
}

uint64_t q4_moe_layer_dev_ws_floats(const q4b_moe_layer *L) {
    /* xn | router logits (+16 pad) | h of up to 64 experts */
    return (uint64_t)L->n_embd + L->n_expert + 16u + 64ull * L->n_ff;
}

bool q4_moe_layer_dev(const q4b_moe_layer *L, const float *d_x, float *d_y, float *d_ws) {
    if (!L || !d_x || !d_y || !d_ws || !q4_hip_ok()) return false;
    if (L->n_expert > 512 || L->topk == 0 || L->topk > 63) return false;
    if (!q4_hip_moe_tok_ok(Q4_T_IQ3_S, Q4_T_IQ3_S, Q4_T_IQ3_S, L->n_embd, L->n_ff)) return false;
    float *d_xn = d_ws;
    float *d_rlog = d_xn + L->n_embd;
    float *d_h = d_rlog + L->n_expert + 16;
    const uint8_t *base = q4_hip_experts_base_a(L->arena);
    const uint64_t stride = q4_hip_experts_stride_a(L->arena);
    if (!base) return false;
    int32_t ids[64];
    float wts[64];
    if (!q4_hip_grouped_rms(d_x, L->d_norm_w, d_xn, L->n_embd, 1, L->eps)) return false;
    if (!q4_hip_gemv_dd(Q4_T_F32, (const uint8_t *)L->d_router, L->n_expert, L->n_embd, d_xn, d_rlog, 1.f))
        return false;
    if (!q4_hip_fill(d_y, 0.f, L->n_embd)) return false;
    if (!q4_hip_softmax_topk(d_rlog, L->n_expert, L->topk, ids, wts)) return false; /* host gets the picks */
    uint32_t n = L->topk;
    for (uint32_t k = 0; k < n; k++) ids[k] += (int32_t)L->first_slot;   /* expert id -> arena slot */
    if (L->shared_slot >= 0) {  /* the always-on shared expert rides along with weight 1 */
        ids[n] = L->shared_slot;
        wts[n] = 1.f;
        n++;
    }
    return q4_hip_moe_exec(base, stride, ids, wts, n, Q4_T_IQ3_S, L->og, Q4_T_IQ3_S, L->ou, Q4_T_IQ3_S,
                           L->od, d_xn, d_h, NULL, NULL, d_y, L->n_ff, L->n_embd, L->n_embd);
}

bool q4_moe_layer_dev_fused(const q4b_moe_layer *L, const float *d_x, float *d_y, int32_t *d_ids,
                            float *d_wts) {
    if (!L || !d_x || !d_y || !q4_hip_ok()) return false;
    const uint8_t *base = q4_hip_experts_base_a(L->arena);
    const uint64_t stride = q4_hip_experts_stride_a(L->arena);
    if (!base) return false;
    return q4_cuda_moe_decode(base + (uint64_t)L->first_slot * stride, stride, L->og, L->ou, L->od,
                              L->shared_slot >= 0 ? L->shared_slot - (int32_t)L->first_slot : -1, d_x,
                              L->d_norm_w, L->eps, L->d_router, L->n_expert, L->topk, L->n_embd, L->n_ff,
                              d_y, d_ids, d_wts);
}

bool q4_moe_layer_dev_n(const q4b_moe_layer *L, const float *d_x, float *d_y, uint32_t n_tok, void *d_ws,
                        uint64_t ws_bytes) {
    if (!L || !d_x || !d_y || !d_ws || n_tok == 0 || !q4_hip_ok()) return false;
    const uint8_t *base = q4_hip_experts_base_a(L->arena);
    const uint64_t stride = q4_hip_experts_stride_a(L->arena);
    if (!base) return false;
    return q4_cuda_moe_layer_n(base + (uint64_t)L->first_slot * stride, stride, L->og, L->ou, L->od,
                               L->shared_slot >= 0 ? L->shared_slot - (int32_t)L->first_slot : -1, d_x,
                               L->d_norm_w, L->eps, L->d_router, L->n_expert, L->topk, L->n_embd, L->n_ff,
                               n_tok, d_y, NULL, NULL, d_ws, ws_bytes);
}
