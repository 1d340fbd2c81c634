/* Expert packs out of a GGUF model file (host side, plain C, no device code).
 *
 * The reference finds a layer's routed experts as three stacked tensors,
 * blk.<layer>.ffn_gate_exps.weight / ffn_up_exps.weight / ffn_down_exps.weight, each holding
 * all experts' matrices of one kind back to back, and assembles expert e's pack as its
 * gate | up | down slices (src/q4_expert.c:962-993: q4_expert_parts, load_one).  This file
 * does the same from the file itself: a reader of the GGUF container (header, metadata
 * key/values, tensor directory; versions 2 and 3, little endian) that keeps only what the
 * slicing needs, and the slice/pack routines.  The shared expert's tensors
 * (ffn_gate_shexp / ffn_up_shexp / ffn_down_shexp) are plain 2-D tensors read whole.
 */
#ifndef Q4_GGUF_EXPERTS_H
#define Q4_GGUF_EXPERTS_H

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct q4b_gguf_tensor {
    char name[128];
    uint32_t n_dims;
    uint64_t ne[4];         /* ne[0] = columns (fastest), ne[1] = rows, ne[2] = experts */
    uint32_t type;          /* ggml type id (IQ3_S = 21, IQ4_NL = 20, IQ4_XS = 23, F32 = 0) */
    uint64_t offset;        /* from the start of the data section */
    uint64_t nbytes;
} q4b_gguf_tensor;

typedef struct q4b_gguf {
    int fd;
    uint32_t version;
    uint64_t n_tensors;
    uint64_t data_off;      /* file offset of the data section */
    uint32_t alignment;
    q4b_gguf_tensor *tensors;
} q4b_gguf;

/* Bytes of one row of `ncols` values of a ggml type this path knows (0 = unknown type or a
 * width the type's block size does not divide): src/q4_quant.c:79 q4_row_bytes. */
uint64_t q4b_gguf_row_bytes(uint32_t type, uint64_t ncols);

bool q4b_gguf_open(q4b_gguf *g, const char *path);
void q4b_gguf_close(q4b_gguf *g);
const q4b_gguf_tensor *q4b_gguf_find(const q4b_gguf *g, const char *name);

/* The three stacked tensors of a layer and the pack geometry they imply
 * (src/q4_expert.c:962-982): offsets of gate | up | down inside a pack and the pack size. */
bool q4b_gguf_expert_parts(const q4b_gguf *g, int32_t layer, const q4b_gguf_tensor **gate,
                           const q4b_gguf_tensor **up, const q4b_gguf_tensor **down, uint64_t *off_gate,
                           uint64_t *off_up, uint64_t *off_down, uint64_t *total, uint32_t *n_expert);
/* Expert eid's pack into dst (total bytes): three reads at e * slice of the stacked tensors
 * (src/q4_expert.c:984-993).  Returns the pack size, or -1. */
int64_t q4b_gguf_read_pack(const q4b_gguf *g, int32_t layer, int32_t eid, uint8_t *dst);
/* The shared expert's pack (gate | up | down of the *_shexp tensors), same layout.  -1 if the
 * layer has none. */
int64_t q4b_gguf_read_shared_pack(const q4b_gguf *g, int32_t layer, uint8_t *dst, uint64_t cap);

#ifdef __cplusplus
}
#endif
#endif
