// Shared declarations for the q4cuda library (sm_100a only).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "iq4nl_codes.h"

#define Q4_T_F32 0u
#define Q4_T_IQ3_S 21u

#define Q4B_IQ3S_BYTES 110u
#define Q4B_QK 256u

// ---- process-wide state (q4b_runtime.cu) ----
struct Q4bState {
    bool ok;
    int device;
    int n_sm;
    cudaStream_t stream;       // the one compute stream every op is enqueued on
    cudaStream_t copy_stream;  // expert uploads
    cudaStream_t aux_stream;   // work forked off the compute stream and joined back (two kernels side by side)
    cudaEvent_t ev_fork, ev_join;
    // activation-quantisation scratch (library-owned, allocated by init/warm)
    int8_t *xq;    // [Q4B_XQ_SLICES][Q4B_XQ_MAXLEN]
    float *xd;     // [Q4B_XQ_SLICES][Q4B_XQ_MAXLEN/32]
    int32_t *xbs;  // [Q4B_XQ_SLICES][Q4B_XQ_MAXLEN/32]
    // staged expert list for q4_hip_moe_exec / _stage (mapped host memory)
    int32_t *es_h, *es_d;
    float *ew_h, *ew_d;
    int32_t *en_h, *en_d;
    // pinned words for synchronous small results
    int32_t *topk_ids_h;
    float *topk_wts_h;
    int32_t *topk_ids_d;
    float *topk_wts_d;
    uint32_t *err_d;  // device error word (bounded waits, argument checks)
    uint32_t *flag_h, *flag_d;  // pinned, mapped word for the host hand-off of the decode call
    uint32_t flag_epoch;
    uint32_t *err_h;
    uint32_t *codes_d;  // the 512 codebook entries byte-expanded (c_j in byte j), device memory
    uint32_t *grid3xxs_d;  // IQ3_XXS codebook: 256 words of four magnitude bytes
    uint2 *grid2s_d;       // IQ2_S codebook: 1024 pairs of words, eight magnitude bytes
    // scratch of the fused layer entry points (q4_cuda_moe_decode*)
    float *xn;        // [Q4B_MAX_TOK][Q4B_XQ_MAXLEN] normalised rows
    float *logits;    // [Q4B_MAX_TOK][1024]
    int32_t *r_ids;   // [Q4B_MAX_TOK][64]
    float *r_wts;     // [Q4B_MAX_TOK][64]
    int32_t *r_cnt;   // [Q4B_MAX_TOK]
    float *hbuf;      // [Q4B_XQ_SLICES][Q4B_XQ_MAXLEN] hidden rows
};
extern Q4bState g_q4b;

#define Q4B_XQ_SLICES 80u     // >= 64 experts per exec + shared + tokens of a window
#define Q4B_XQ_MAXLEN 16384u  // widest activation row the decode path quantises
#define Q4B_MAX_TOK 8u        // tokens per fused decode / verify call
#define Q4B_MAX_MARKS 2048u   // q4_cuda_timer_mark slots

#define Q4B_CHECK(call)                                                              \
    do {                                                                             \
        cudaError_t e_ = (call);                                                     \
        if (e_ != cudaSuccess) {                                                     \
            fprintf(stderr, "q4cuda: %s failed at %s:%d: %s\n", #call, __FILE__,     \
                    __LINE__, cudaGetErrorString(e_));                               \
            return false;                                                            \
        }                                                                            \
    } while (0)

static inline bool q4b_launch_ok(const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        fprintf(stderr, "q4cuda: launch of %s failed: %s\n", what, cudaGetErrorString(e));
        return false;
    }
    return true;
}

#ifdef __CUDACC__

// The 512-entry codebook as packed 12-bit codes (four 3-bit codes per entry).
// The library is compiled as ONE translation unit (q4cuda.cu includes every
// other .cu), so this definition exists once.
__constant__ uint16_t c_iq3s_codes[512];

// Expand entry idx to four bytes c_j (0..7); magnitude_j = 2 c_j + 1.
__device__ __forceinline__ uint32_t q4b_code_bytes(uint32_t code12) {
    return (code12 & 7u) | ((code12 & 0x38u) << 5) | ((code12 & 0x1c0u) << 10) |
           ((code12 & 0xe00u) << 15);
}

// Fill a 512-word shared table with the byte-expanded codes.
__device__ __forceinline__ void q4b_fill_code_table(uint32_t *tab) {
    for (uint32_t i = threadIdx.x; i < 512u; i += blockDim.x)
        tab[i] = q4b_code_bytes(c_iq3s_codes[i]);
}

// 4 sign bits (bit j = element j negative) -> 0x00/0xFF byte mask.
__device__ __forceinline__ uint32_t q4b_sign_mask4(uint32_t nib) {
    // bit j lands on bit 8j+7 (no two products share a position), then the
    // permute replicates each byte's top bit over the byte.
    const uint32_t t = (nib & 0xfu) * 0x10204080u;
    uint32_t m;
    // prmt with selector bit 3 set: copy the top bit of the chosen byte to all
    // eight bits (__byte_perm drops that selector bit, so use the instruction).
    asm("prmt.b32 %0, %1, %1, 0xba98;" : "=r"(m) : "r"(t));
    return m;
}

// Integer dot of one 32-weight sub-block with 32 int8 activations.
//   qs:   the sub-block's eight index bytes (two little-endian words)
//   qh:   its high-bit byte, sg: its 32 sign bits
//   q:    eight words of int8x4 activations, qsum: their sum
// Returns sum_i sign_i * magnitude_i * q_i exactly:
//   magnitude = 2c+1 and a negated value is 2(~c)+1, so the dot is
//   2 * sum (c ^ mask) q  +  sum q.
__device__ __forceinline__ int32_t q4b_group_idot(uint32_t qs_lo, uint32_t qs_hi, uint32_t qh,
                                                  uint32_t sg, const uint32_t *tab,
                                                  const int *q, int32_t qsum) {
    int32_t acc = 0;
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const uint32_t w = k < 4 ? qs_lo : qs_hi;
        const uint32_t idx = ((w >> (8 * (k & 3))) & 0xffu) | (((qh >> k) & 1u) << 8);
        const uint32_t c = tab[idx];
        const uint32_t m = q4b_sign_mask4(sg >> (4 * k));
        acc = __dp4a((int)(c ^ m), q[k], acc);
    }
    return 2 * acc + qsum;
}

__device__ __forceinline__ uint32_t q4b_ld_u16(const uint8_t *p) {
    return *reinterpret_cast<const uint16_t *>(p);
}
// 4 bytes from a 2-byte-aligned address.
__device__ __forceinline__ uint32_t q4b_ld_u32_a2(const uint8_t *p) {
    return q4b_ld_u16(p) | (q4b_ld_u16(p + 2) << 16);
}

__device__ __forceinline__ float q4b_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float q4b_warp_max(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// silu(g) * u exactly as the CPU path writes it: g / (1 + exp(-g)) * u.
__device__ __forceinline__ float q4b_swiglu(float g, float u) {
    return __fdiv_rn(g, 1.f + expf(-g)) * u;
}

#endif  // __CUDACC__
