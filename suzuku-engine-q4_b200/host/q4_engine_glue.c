/* Engine-side glue for libq4cuda.so: the device-layer functions whose arguments are the
 * engine's own model structs (src/q4.h:1161,1168 take a q4_gguf).  The library cannot know
 * those layouts, so this file is compiled WITH the engine, against its q4.h:
 *
 *     cc -c -I<engine>/src q4_engine_glue.c        (added to the engine's object list)
 *
 * It reads the model through the engine's accessors and asks the library what it covers.
 */
#include "q4.h"

/* Largest gate+up and down byte counts of one expert over the layers the grouped product
 * takes (gate and up of one type, both accepted by q4_mmq_supported): the per-expert strides
 * of the expert-indexed buffers q4_mmq_wbuf hands out.  q4_mmq_pad() is added as the engine
 * does at its call site (src/q4_moe.c:3630-3640); this library's pad is 0. */
void q4_mmq_wbuf_size(const q4_gguf *g, uint64_t *gu_max, uint64_t *d_max) {
    uint64_t gu = 0, d = 0;
    if (g && q4_mmq_on()) {
        const uint64_t n_ff = g->n_ff_exp;
        for (uint32_t layer = 0; layer < g->n_layer; layer++) {
            const q4_tensor *tg, *tu, *td;
            uint64_t og, ou, od, total;
            if (!q4_expert_parts(g, (int32_t)layer, &tg, &tu, &td, &og, &ou, &od, &total)) continue;
            if (tg->ggml_type != tu->ggml_type) continue;
            if (!q4_mmq_supported(tg->ggml_type, 2u * n_ff) || !q4_mmq_supported(td->ggml_type, g->n_embd))
                continue;
            const uint64_t gu_bytes = od - og + q4_mmq_pad(q4_row_bytes(tg->ggml_type, g->n_embd));
            const uint64_t d_bytes = total - od + q4_mmq_pad(q4_row_bytes(td->ggml_type, n_ff));
            if (gu_bytes > gu) gu = gu_bytes;
            if (d_bytes > d) d = d_bytes;
        }
    }
    if (gu_max) *gu_max = gu;
    if (d_max) *d_max = d;
}

/* Bytes of the two buffers for all experts (what the engine's planner sets aside). */
void q4_mmq_wbuf_need(const q4_gguf *g, uint64_t *gu_need, uint64_t *d_need) {
    uint64_t gu = 0, d = 0;
    q4_mmq_wbuf_size(g, &gu, &d);
    const uint64_t n_exp = g ? g->n_expert : 0;
    if (gu_need) *gu_need = gu * n_exp;
    if (d_need) *d_need = d * n_exp;
}
