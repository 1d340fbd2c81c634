// The remaining formats a routed expert's projections may come in (src/q4_rocm.cu:4926-4944):
// IQ3_XXS (18) and IQ2_S (22) for gate and up, Q2_0 (42) for down, in the one-token exec calls.
// Included inside q4b_decode.cu's unnamed namespace, before the host side.
//
// Block layouts (public ggml formats):
//   IQ3_XXS  98 B / 256: f16 d | qs[64]: one codebook index per 4 values | 8 x u32: four 7-bit
//            indices into the even-parity sign table (one per 8 values) and a 4-bit scale s;
//            value = d * (0.5 + s) * 0.5 * magnitude * sign        (src/q4_quant.c:424-452)
//   IQ2_S    82 B / 256: f16 d | qs[32]: low 8 index bits, one per 8 values | signs[32]: one byte
//            per 8 values | qh[8]: two more index bits per entry | scales[8]: two 4-bit scales per
//            32 values (first / last 16); value = d * (0.5 + s) * 0.25 * magnitude * sign  (:290-322)
//   Q2_0     18 B / 64: f16 d | 16 bytes of 2-bit codes c; value = d * (c - 1)            (:177-188)
// The codebooks sit in device memory as magnitude bytes (g_q4b.grid3xxs_d: 256 words of four,
// g_q4b.grid2s_d: 1024 pairs of words of eight), expanded at init from the packed level numbers of
// iq3xxs_codes.h / iq2s_codes.h.  With 8-bit activations the dot of a 32-group is the exact integer
//   IQ3_XXS: (2 s + 1) * sum(sign * magnitude * q)              times d / 4 * dx
//   IQ2_S:   (2 s0 + 1) * sum_first16 + (2 s1 + 1) * sum_last16 times d / 8 * dx
//   Q2_0:    sum(c * q) - sum(q)                                times d * dx
// which is what the reference's CPU kernels form (src/q4_cpuexp.c:814-852, 895-931, 1113-1145).

#define Q4_T_IQ3_XXS 18u
#define Q4_T_IQ2_S 22u
#define Q4_T_Q2_0 42u

__host__ __device__ inline uint64_t small_row_bytes(uint32_t type, uint64_t ncols) {
    return type == Q4_T_IQ3_XXS ? (ncols / 256u) * 98u : type == Q4_T_IQ2_S ? (ncols / 256u) * 82u : (ncols / 64u) * 18u;
}

// q with the bytes negated where the mask byte is 0xFF
__device__ __forceinline__ int neg_where(int q, uint32_t mask) { return (int)__vsub4((uint32_t)q ^ mask, mask); }

// One 32-group: signed magnitudes as eight words (word k = values 4k..4k+3, already sign-applied is
// not possible for unsigned magnitudes, so the signs come back as eight byte masks), the integer
// sub-scale factor of each half, and the block's fp16 d.
struct SmallGroup {
    uint32_t mag[8];
    uint32_t neg[8];
    int ls0, ls1;      // 2 s + 1 of values 0..15 and 16..31
    int s0, s1;        // the raw 4-bit scales (dequantisation)
    float d;
};

template <uint32_t T>
__device__ __forceinline__ void small_group(const uint8_t *row, uint32_t g, const uint32_t *grid3,
                                            const uint2 *grid2, SmallGroup &G) {
    if (T == Q4_T_IQ3_XXS) {
        const uint8_t *blk = row + (uint64_t)(g >> 3) * 98u;
        const uint32_t ib = g & 7u;
        const uint8_t *qs = blk + 2u + 8u * ib;
        const uint32_t aux = q4b_ld_u32_a2(blk + 66u + 4u * ib);
        const uint32_t i01 = q4b_ld_u16(qs), i23 = q4b_ld_u16(qs + 2), i45 = q4b_ld_u16(qs + 4), i67 = q4b_ld_u16(qs + 6);
        const uint32_t idx[8] = {i01 & 0xffu, i01 >> 8, i23 & 0xffu, i23 >> 8, i45 & 0xffu, i45 >> 8, i67 & 0xffu, i67 >> 8};
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const uint32_t s7 = (aux >> (7 * l)) & 127u;
            const uint32_t sb = s7 | ((__popc(s7) & 1u) << 7);     // the sign table: even parity
            G.mag[2 * l] = __ldg(grid3 + idx[2 * l]);
            G.mag[2 * l + 1] = __ldg(grid3 + idx[2 * l + 1]);
            G.neg[2 * l] = q4b_sign_mask4(sb);
            G.neg[2 * l + 1] = q4b_sign_mask4(sb >> 4);
        }
        G.s0 = G.s1 = (int)(aux >> 28);
        G.d = __half2float(__ushort_as_half((unsigned short)q4b_ld_u16(blk)));
    } else {
        const uint8_t *blk = row + (uint64_t)(g >> 3) * 82u;
        const uint32_t ib = g & 7u;
        const uint32_t qs = q4b_ld_u32_a2(blk + 2u + 4u * ib), sg = q4b_ld_u32_a2(blk + 34u + 4u * ib);
        const uint32_t qh = blk[66u + ib], sb = blk[74u + ib];
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const uint32_t idx = ((qs >> (8 * l)) & 0xffu) | ((qh << (8 - 2 * l)) & 0x300u);
            const uint2 m = __ldg(grid2 + idx);
            const uint32_t s8 = (sg >> (8 * l)) & 0xffu;
            G.mag[2 * l] = m.x;
            G.mag[2 * l + 1] = m.y;
            G.neg[2 * l] = q4b_sign_mask4(s8);
            G.neg[2 * l + 1] = q4b_sign_mask4(s8 >> 4);
        }
        G.s0 = (int)(sb & 15u);
        G.s1 = (int)(sb >> 4);
        G.d = __half2float(__ushort_as_half((unsigned short)q4b_ld_u16(blk)));
    }
    G.ls0 = 2 * G.s0 + 1;
    G.ls1 = 2 * G.s1 + 1;
}

// exact integer sums of the two halves of a group against 32 int8 activations (eight words)
__device__ __forceinline__ void small_group_isums(const SmallGroup &G, const int *q, int *lo, int *hi) {
    int a = 0, b = 0;
#pragma unroll
    for (int k = 0; k < 4; k++) {
        a = __dp4a((int)G.mag[k], neg_where(q[k], G.neg[k]), a);
        b = __dp4a((int)G.mag[4 + k], neg_where(q[4 + k], G.neg[4 + k]), b);
    }
    *lo = a;
    *hi = b;
}

// Q2_0: the eight code bytes of group g (32 values) as eight words of codes 0..3
__device__ __forceinline__ float q20_group(const uint8_t *row, uint32_t g, uint32_t cw[8]) {
    const uint8_t *blk = row + (uint64_t)(g >> 1) * 18u;
    const uint8_t *qs = blk + 2u + 8u * (g & 1u);
    const uint32_t w0 = q4b_ld_u32_a2(qs), w1 = q4b_ld_u32_a2(qs + 4);
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const uint32_t b = ((k < 4 ? w0 : w1) >> (8 * (k & 3))) & 0xffu;
        cw[k] = (b | (b << 6) | (b << 12) | (b << 18)) & 0x03030303u;
    }
    return __half2float(__ushort_as_half((unsigned short)q4b_ld_u16(blk)));
}

// ---- stage kernels: dequantisation and the integer part of every group's dot ----
template <uint32_t T>
__global__ void small_dequant_k(const uint8_t *__restrict__ w, uint64_t n_groups, uint32_t gpr,
                                const uint32_t *__restrict__ grid3, const uint2 *__restrict__ grid2,
                                float *__restrict__ out) {
    const uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_groups) return;
    const uint64_t r = t / gpr;
    const uint32_t g = (uint32_t)(t - r * gpr);
    const uint8_t *row = w + r * small_row_bytes(T, 32ull * gpr);
    float *o = out + t * 32u;
    if (T == Q4_T_Q2_0) {
        uint32_t cw[8];
        const float d = q20_group(row, g, cw);
#pragma unroll
        for (int i = 0; i < 32; i++) o[i] = __fmul_rn(d, (float)((int)((cw[i >> 2] >> (8 * (i & 3))) & 3u) - 1));
        return;
    }
    SmallGroup G;
    small_group<T>(row, g, grid3, grid2, G);
    const float step = T == Q4_T_IQ3_XXS ? 0.5f : 0.25f;
#pragma unroll
    for (int i = 0; i < 32; i++) {
        const float db = __fmul_rn(__fmul_rn(G.d, __fadd_rn(0.5f, (float)(i < 16 ? G.s0 : G.s1))), step);
        const float m = (float)((G.mag[i >> 2] >> (8 * (i & 3))) & 0xffu);
        const float sgn = ((G.neg[i >> 2] >> (8 * (i & 3))) & 1u) ? -1.f : 1.f;
        o[i] = __fmul_rn(__fmul_rn(db, m), sgn);
    }
}

template <uint32_t T>
__global__ void small_idot_k(const uint8_t *__restrict__ w, uint64_t nrows, uint32_t gpr,
                             const uint32_t *__restrict__ grid3, const uint2 *__restrict__ grid2,
                             const int8_t *__restrict__ q, int32_t *__restrict__ I) {
    const uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= nrows * gpr) return;
    const uint64_t r = t / gpr;
    const uint32_t g = (uint32_t)(t - r * gpr);
    const uint8_t *row = w + r * small_row_bytes(T, 32ull * gpr);
    int qv[8];
#pragma unroll
    for (int k = 0; k < 8; k++) qv[k] = reinterpret_cast<const int *>(q)[g * 8u + k];
    if (T == Q4_T_Q2_0) {
        uint32_t cw[8];
        (void)q20_group(row, g, cw);
        int s = 0;
#pragma unroll
        for (int k = 0; k < 8; k++) s = __dp4a((int)cw[k], qv[k], s);
        I[t] = s;
        return;
    }
    SmallGroup G;
    small_group<T>(row, g, grid3, grid2, G);
    int lo, hi;
    small_group_isums(G, qv, &lo, &hi);
    I[t] = lo + hi;
}

// ---- gate/up + SwiGLU with rows of type T (IQ3_XXS or IQ2_S): one warp per (expert, hidden unit) ----
template <uint32_t T>
__global__ void moe_gux_k(const uint8_t *__restrict__ bg, const uint8_t *__restrict__ bu, uint64_t stride,
                          const int32_t *__restrict__ slots, const int32_t *__restrict__ n_dev,
                          const int8_t *__restrict__ xq, const float *__restrict__ xd, uint32_t in_dim,
                          uint32_t n_ff, const uint32_t *__restrict__ grid3, const uint2 *__restrict__ grid2,
                          float *__restrict__ h) {
    const uint32_t e = blockIdx.y;
    if (n_dev && e >= (uint32_t)*n_dev) return;
    const uint32_t f = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (f >= n_ff) return;
    const uint32_t lane = threadIdx.x & 31u, ng = in_dim >> 5;
    const uint64_t rb = small_row_bytes(T, in_dim);
    const uint8_t *rg = bg + (uint64_t)slots[e] * stride + (uint64_t)f * rb;
    const uint8_t *ru = bu + (uint64_t)slots[e] * stride + (uint64_t)f * rb;
    const float unit = T == Q4_T_IQ3_XXS ? 0.25f : 0.125f;
    float ag = 0.f, au = 0.f;
    for (uint32_t g = lane; g < ng; g += 32) {
        int qv[8];
#pragma unroll
        for (int k = 0; k < 8; k++) qv[k] = reinterpret_cast<const int *>(xq)[g * 8u + k];
        const float dx = xd[g];
        SmallGroup G;
        int lo, hi;
        small_group<T>(rg, g, grid3, grid2, G);
        small_group_isums(G, qv, &lo, &hi);
        ag = fmaf(__fmul_rn(__fmul_rn(G.d, unit), dx), (float)(lo * G.ls0 + hi * G.ls1), ag);
        small_group<T>(ru, g, grid3, grid2, G);
        small_group_isums(G, qv, &lo, &hi);
        au = fmaf(__fmul_rn(__fmul_rn(G.d, unit), dx), (float)(lo * G.ls0 + hi * G.ls1), au);
    }
    ag = q4b_warp_sum(ag);
    au = q4b_warp_sum(au);
    if (lane == 0) h[(uint64_t)e * n_ff + f] = q4b_swiglu(ag, au);
}

// ---- down projection with Q2_0 rows: the counterpart of moe_ya_k (same reduction shape) ----
__global__ void moe_ya20_k(const uint8_t *__restrict__ bd, uint64_t stride, const int32_t *__restrict__ slots,
                           const float *__restrict__ wts, uint32_t n_host, const int32_t *__restrict__ n_dev,
                           const int8_t *__restrict__ hq, const float *__restrict__ hd,
                           const int32_t *__restrict__ hbs, uint64_t q_slice, uint64_t d_slice, uint32_t n_ff,
                           uint32_t n_embd, float *__restrict__ y) {
    const uint32_t r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= n_embd) return;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t n = n_dev ? (uint32_t)*n_dev : n_host;
    const uint32_t ng = n_ff >> 5;
    const uint64_t rb = small_row_bytes(Q4_T_Q2_0, n_ff);
    float acc = 0.f;
    for (uint32_t it = lane; it < n * ng; it += 32) {
        const uint32_t e = it / ng, g = it - e * ng;
        const int *qg = reinterpret_cast<const int *>(hq + (uint64_t)e * q_slice) + g * 8u;
        uint32_t cw[8];
        const float d = q20_group(bd + (uint64_t)slots[e] * stride + (uint64_t)r * rb, g, cw);
        int s = 0;
#pragma unroll
        for (int k = 0; k < 8; k++) s = __dp4a((int)cw[k], qg[k], s);
        const float dd = __fmul_rn(d, hd[(uint64_t)e * d_slice + g]);
        acc = fmaf(__fmul_rn(wts[e], dd), (float)(s - hbs[(uint64_t)e * d_slice + g]), acc);
    }
    acc = q4b_warp_sum(acc);
    if (lane == 0) y[r] += acc;
}
