// The dense product of up to 8 activation rows in 8-bit form: y[t][r] = scale * W[r] . q8(x[t])
// (src/q4.h:913-927, src/q4_mmvq.cu).  Weight types: Q6_K, Q4_K, Q5_K (ggml K-quant super-blocks),
// IQ4_XS and IQ4_NL here; IQ3_S goes through the grouped expert product.
//
// Arithmetic (what makes a row's result independent of the number of rows in the call): the
// activations are quantised per 32 values with d = amax / 127, q = rint(v / d), and the integer sum
// of each half of a group is kept.  A weight row is cut into runs of 16 consecutive values that
// share one scale; each value of a run is a * w + c with integer w.  The lanes of one warp take
// the row's runs round robin and add  dx * (a * dot(w, q) + c * sum16(q))  with explicit fused
// multiply-adds, then the 32 partial sums are added by the xor butterfly.  Every activation row
// goes through exactly these operations, so calls of 1 .. 8 rows give the same bits per row.

namespace mv {

constexpr uint32_t MAXK = Q4B_XQ_MAXLEN;

// ------------------------------------------------------------------ activations
// One warp per 32 values (src/q4_mmvq.cu:36-57): a division by d, not a product with 127 / amax.
__global__ void quant8d_k(const float *__restrict__ x, uint64_t n_groups, int8_t *__restrict__ q,
                          float *__restrict__ d, int32_t *__restrict__ s16) {
    const uint64_t g = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (g >= n_groups) return;
    const uint32_t lane = threadIdx.x & 31u;
    const float v = x[g * 32u + lane];
    const float a = q4b_warp_max(fabsf(v));
    const float dg = __fdiv_rn(a, 127.f);
    const int qi = dg > 0.f ? __float2int_rn(__fdiv_rn(v, dg)) : 0;
    q[g * 32u + lane] = (int8_t)qi;
    int s = qi;
#pragma unroll
    for (int o = 8; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);   // halves of the group
    if (lane == 0) d[g] = dg;
    if ((lane & 15u) == 0) s16[2 * g + (lane >> 4)] = s;
}

// ------------------------------------------------------------------ weight runs
struct Run {
    uint32_t w[4];   // 16 weights, one per byte (unsigned 0..63, or signed codebook values)
    float a, c;
};

__device__ __forceinline__ float ld_f16(const uint8_t *p) {
    return __half2float(__ushort_as_half((unsigned short)q4b_ld_u16(p)));
}

// four 4-bit codes, one per byte, through the IQ4_NL codebook: the 16 values sit in four
// registers and two byte permutes pick by the low three bits; bit 3 chooses between them
constexpr int8_t kNl[16] = Q4B_IQ4NL_VALUES;
__host__ __device__ constexpr uint32_t nl_word(int i) {
    return (uint32_t)(uint8_t)kNl[i] | ((uint32_t)(uint8_t)kNl[i + 1] << 8) | ((uint32_t)(uint8_t)kNl[i + 2] << 16) |
           ((uint32_t)(uint8_t)kNl[i + 3] << 24);
}
__device__ __forceinline__ uint32_t nl_codes4(uint32_t nib) {
    const uint32_t low = nib & 0x07070707u;
    const uint32_t t = (low | (low >> 4)) & 0x00FF00FFu;
    const uint32_t sel = (t | (t >> 8)) & 0xFFFFu;          // one selector nibble per byte
    constexpr uint32_t T0 = nl_word(0), T1 = nl_word(4), T2 = nl_word(8), T3 = nl_word(12);
    const uint32_t lo = __byte_perm(T0, T1, sel);
    const uint32_t hi = __byte_perm(T2, T3, sel);
    const uint32_t pick = ((nib >> 3) & 0x01010101u) * 0xFFu;
    return (lo & ~pick) | (hi & pick);
}

// 6-bit scale and minimum of sub-block j in the 12 packed bytes of a Q4_K / Q5_K block
__device__ __forceinline__ void k_scale_min(const uint8_t *p, int j, int *sc, int *mn) {
    if (j < 4) {
        *sc = p[j] & 63;
        *mn = p[j + 4] & 63;
    } else {
        *sc = (p[j + 4] & 15) | ((p[j - 4] >> 6) << 4);
        *mn = (p[j + 4] >> 4) | ((p[j] >> 6) << 4);
    }
}

// 16 bytes from an address aligned to A bytes
template <int A> __device__ __forceinline__ void ld16(const uint8_t *p, uint32_t v[4]) {
    if constexpr (A >= 16) {
        const uint4 t = *reinterpret_cast<const uint4 *>(p);
        v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
    } else if constexpr (A >= 8) {
        const uint2 t0 = *reinterpret_cast<const uint2 *>(p), t1 = *reinterpret_cast<const uint2 *>(p + 8);
        v[0] = t0.x, v[1] = t0.y, v[2] = t1.x, v[3] = t1.y;
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) v[i] = q4b_ld_u32_a2(p + 4 * i);
    }
}

template <uint32_t TY> struct Fmt;

// Q6_K, 210 bytes: ql[128] | qh[64] | int8 scales[16] | f16 d.  Each half (128 values) is four
// strips of 32; strip s has its low nibbles in ql bytes 32*(s&1).. of the half (upper nibble for
// s >= 2) and its two high bits in bits 2s..2s+1 of the half's 32 qh bytes.  Values are stored + 32.
template <> struct Fmt<14u> {
    static constexpr uint32_t bytes = 210, vals = 256, align = 2;
    static constexpr bool has_c = true;
    __device__ static uint32_t first(uint32_t r) { return 128u * (r >> 3) + 32u * ((r >> 1) & 3u) + 16u * (r & 1u); }
    __device__ static void decode(const uint8_t *blk, uint32_t r, Run &R) {
        const uint32_t half = r >> 3, strip = (r >> 1) & 3u, lo = 16u * (r & 1u);
        uint32_t l[4], h[4];
        ld16<2>(blk + 64u * half + 32u * (strip & 1u) + lo, l);
        ld16<2>(blk + 128u + 32u * half + lo, h);
#pragma unroll
        for (int i = 0; i < 4; i++)
            R.w[i] = ((l[i] >> (4u * (strip >> 1))) & 0x0F0F0F0Fu) | (((h[i] >> (2u * strip)) & 0x03030303u) << 4);
        R.a = __fmul_rn(ld_f16(blk + 208), (float)(int8_t)blk[192u + 8u * half + 2u * strip + (r & 1u)]);
        R.c = __fmul_rn(-32.f, R.a);
    }
};
// Q4_K, 144 bytes: f16 d | f16 dmin | scales[12] | qs[128]; sub-blocks 2p, 2p+1 are the low and
// high nibbles of qs bytes 32p..32p+31
template <> struct Fmt<12u> {
    static constexpr uint32_t bytes = 144, vals = 256, align = 16;
    static constexpr bool has_c = true;
    __device__ static uint32_t first(uint32_t r) { return 16u * r; }
    __device__ static void decode(const uint8_t *blk, uint32_t r, Run &R) {
        const uint32_t j = r >> 1, lo = 16u * (r & 1u);
        uint32_t v[4];
        ld16<16>(blk + 16u + 32u * (j >> 1) + lo, v);
#pragma unroll
        for (int i = 0; i < 4; i++) R.w[i] = (v[i] >> (4u * (j & 1u))) & 0x0F0F0F0Fu;
        int sc, mn;
        k_scale_min(blk + 4, (int)j, &sc, &mn);
        R.a = __fmul_rn(ld_f16(blk), (float)sc);
        R.c = __fmul_rn(-ld_f16(blk + 2), (float)mn);
    }
};
// Q5_K, 176 bytes: as Q4_K with qh[32] before qs; bit j of qh byte l is bit 4 of value l of sub-block j
template <> struct Fmt<13u> {
    static constexpr uint32_t bytes = 176, vals = 256, align = 16;
    static constexpr bool has_c = true;
    __device__ static uint32_t first(uint32_t r) { return 16u * r; }
    __device__ static void decode(const uint8_t *blk, uint32_t r, Run &R) {
        const uint32_t j = r >> 1, lo = 16u * (r & 1u);
        uint32_t v[4], h[4];
        ld16<16>(blk + 48u + 32u * (j >> 1) + lo, v);
        ld16<16>(blk + 16u + lo, h);
#pragma unroll
        for (int i = 0; i < 4; i++)
            R.w[i] = ((v[i] >> (4u * (j & 1u))) & 0x0F0F0F0Fu) | (((h[i] >> j) & 0x01010101u) << 4);
        int sc, mn;
        k_scale_min(blk + 4, (int)j, &sc, &mn);
        R.a = __fmul_rn(ld_f16(blk), (float)sc);
        R.c = __fmul_rn(-ld_f16(blk + 2), (float)mn);
    }
};
// IQ4_XS, 136 bytes: f16 d | u16 scales_h | scales_l[4] | qs[128]; group ib (32 values) = low then
// high nibbles of qs bytes 16 ib .. 16 ib + 15 through the codebook, 6-bit scale - 32
template <> struct Fmt<23u> {
    static constexpr uint32_t bytes = 136, vals = 256, align = 8;
    static constexpr bool has_c = false;
    __device__ static uint32_t first(uint32_t r) { return 16u * r; }
    __device__ static void decode(const uint8_t *blk, uint32_t r, Run &R) {
        const uint32_t ib = r >> 1, hi = r & 1u;
        uint32_t v[4];
        ld16<8>(blk + 8u + 16u * ib, v);
#pragma unroll
        for (int i = 0; i < 4; i++) R.w[i] = nl_codes4((v[i] >> (4u * hi)) & 0x0F0F0F0Fu);
        const uint32_t sh = q4b_ld_u16(blk + 2);
        const int ls = (int)(((blk[4u + (ib >> 1)] >> (4u * (ib & 1u))) & 15u) | (((sh >> (2u * ib)) & 3u) << 4));
        R.a = __fmul_rn(ld_f16(blk), (float)(ls - 32));
        R.c = 0.f;
    }
};
// IQ4_NL, 18 bytes per 32 values: f16 d | qs[16]
template <> struct Fmt<20u> {
    static constexpr uint32_t bytes = 18, vals = 32, align = 2;
    static constexpr bool has_c = false;
    __device__ static uint32_t first(uint32_t r) { return 16u * r; }
    __device__ static void decode(const uint8_t *blk, uint32_t r, Run &R) {
        uint32_t v[4];
        ld16<2>(blk + 2, v);
#pragma unroll
        for (int i = 0; i < 4; i++) R.w[i] = nl_codes4((v[i] >> (4u * r)) & 0x0F0F0F0Fu);
        R.a = ld_f16(blk);
        R.c = 0.f;
    }
};

// ------------------------------------------------------------------ the product
// One warp per weight row, 8 rows per block.  The activation rows (at most 8 x 16384 bytes) stay
// in L1/L2; the weights are read once.
template <uint32_t TY, int NT>
__global__ void __launch_bounds__(256) dense_rows_k(const uint8_t *__restrict__ w, const int8_t *__restrict__ xq,
                                                    const float *__restrict__ xd, const int32_t *__restrict__ xs,
                                                    float *__restrict__ y, uint32_t K, uint32_t rows, float scale) {
    using F = Fmt<TY>;
    const uint32_t row = blockIdx.x * 8u + (threadIdx.x >> 5);
    if (row >= rows) return;
    const uint32_t lane = threadIdx.x & 31u;
    constexpr uint32_t rpb = F::vals / 16u;
    const uint32_t n_runs = K / 16u;
    const uint8_t *wr = w + (uint64_t)row * (K / F::vals) * F::bytes;
    float acc[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) acc[t] = 0.f;
    for (uint32_t run = lane; run < n_runs; run += 32u) {
        const uint32_t b = run / rpb, r = run % rpb;
        Run R;
        F::decode(wr + (uint64_t)b * F::bytes, r, R);
        const uint32_t e0 = b * F::vals + F::first(r);
        int4 xv[NT];
        float dx[NT];
        int sx[NT];
#pragma unroll
        for (int t = 0; t < NT; t++) {
            xv[t] = *reinterpret_cast<const int4 *>(xq + (size_t)t * K + e0);
            dx[t] = xd[(size_t)t * (K >> 5) + (e0 >> 5)];
            sx[t] = F::has_c ? xs[(size_t)t * (K >> 4) + (e0 >> 4)] : 0;
        }
#pragma unroll
        for (int t = 0; t < NT; t++) {
            // weights below 128 (or signed codebook values): the signed 4-way dot is exact for both
            int s = __dp4a((int)R.w[0], xv[t].x, 0);
            s = __dp4a((int)R.w[1], xv[t].y, s);
            s = __dp4a((int)R.w[2], xv[t].z, s);
            s = __dp4a((int)R.w[3], xv[t].w, s);
            float v = __fmul_rn(R.a, (float)s);
            if (F::has_c) v = __fmaf_rn(R.c, (float)sx[t], v);
            acc[t] = __fmaf_rn(dx[t], v, acc[t]);
        }
    }
#pragma unroll
    for (int t = 0; t < NT; t++) {
        float a = acc[t];
#pragma unroll
        for (int o = 16; o; o >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, o));
        if (lane == 0) y[(size_t)t * rows + row] = __fmul_rn(scale, a);
    }
}

// scratch of the quantised rows: q [8][MAXK], d [8][MAXK / 32], s16 [8][MAXK / 16]
int8_t *g_q = nullptr;
float *g_d = nullptr;
int32_t *g_s = nullptr;
// what the scratch of either kind holds (q4_mmvq_hold lets calls on the same x reuse it)
const float *g_hold = nullptr;
const float *g_cur_x = nullptr;
uint64_t g_cur_k = 0;
uint32_t g_cur_n = 0;
int g_cur_kind = -1;   // 0: rows of the grouped product (IQ3_S), 1: rows of this file's product
int g_mode = 1;        // 0 off, 1 calls of 2..8 rows, 2 calls of 1..8 rows inside a verify scope only
int g_scope = 0;

bool warm() {
    if (g_q) return true;
    const size_t bytes = (size_t)8 * MAXK + (size_t)8 * (MAXK / 32) * 4 + (size_t)8 * (MAXK / 16) * 4;
    void *p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    g_q = (int8_t *)p;
    g_d = (float *)(g_q + (size_t)8 * MAXK);
    g_s = (int32_t *)(g_d + (size_t)8 * (MAXK / 32));
    return true;
}
void shutdown() {
    cudaFree(g_q);
    g_q = nullptr;
    g_d = nullptr;
    g_s = nullptr;
    g_hold = g_cur_x = nullptr;
    g_cur_kind = -1;
}

template <uint32_t TY>
bool launch(uint32_t n, const uint8_t *w, float *y, uint32_t K, uint32_t rows, float scale) {
    const unsigned grid = (rows + 7u) / 8u;
    switch (n) {
#define Q4B_MV_CASE(N)                                                                              \
    case N:                                                                                         \
        dense_rows_k<TY, N><<<grid, 256, 0, g_q4b.stream>>>(w, g_q, g_d, g_s, y, K, rows, scale); \
        break;
        Q4B_MV_CASE(1) Q4B_MV_CASE(2) Q4B_MV_CASE(3) Q4B_MV_CASE(4) Q4B_MV_CASE(5) Q4B_MV_CASE(6) Q4B_MV_CASE(7)
        Q4B_MV_CASE(8)
#undef Q4B_MV_CASE
    default: return false;
    }
    g_q4b_launches.fetch_add(1, std::memory_order_relaxed);
    return q4b_launch_ok("mmvq_dense");
}

bool dense_type(uint32_t ty) { return ty == 14u || ty == 12u || ty == 13u || ty == 23u || ty == 20u; }

// whole blocks and the row alignment the type's loads need (checked before anything is queued)
template <uint32_t TY> bool fits(const uint8_t *w, uint64_t K) {
    return K % Fmt<TY>::vals == 0 && ((uintptr_t)w % Fmt<TY>::align) == 0 &&
           (K / Fmt<TY>::vals * Fmt<TY>::bytes) % Fmt<TY>::align == 0;
}
bool dense_fits(uint32_t ty, const uint8_t *w, uint64_t K) {
    switch (ty) {
    case 14u: return fits<14u>(w, K);
    case 12u: return fits<12u>(w, K);
    case 13u: return fits<13u>(w, K);
    case 23u: return fits<23u>(w, K);
    case 20u: return fits<20u>(w, K);
    default: return false;
    }
}

}  // namespace mv

bool q4b_mmvq_warm() { return mv::warm(); }
void q4b_mmvq_shutdown() { mv::shutdown(); }

extern "C" void q4_mmvq_warm(void) {
    (void)elem::warm();
    (void)mv::warm();
}
// 0 off; 1 calls of 2..8 rows anywhere; 2 calls of 1..8 rows, only between q4_mmvq_verify(1) and
// q4_mmvq_verify(0) (src/q4_mmvq.cu:271-288).  The reference's per-type thresholds inside modes 1
// and 2 (from 3 rows for some types, short Q4_K tensors only) record where its own float kernels
// were faster on its hardware; this library has no float n-row kernels to fall back to and takes
// every covered type at every n of the mode.
extern "C" int q4_mmvq_on(void) { return g_q4b.ok ? mv::g_mode : 0; }
extern "C" void q4_mmvq_set(int v) { mv::g_mode = v < 0 || v > 2 ? 0 : v; }
extern "C" void q4_mmvq_verify(int on) { mv::g_scope = on ? 1 : 0; }
// Between hold(x) and release(), calls on the same x (same width, no more rows) reuse its
// quantisation; the caller promises x is not rewritten inside the scope (src/q4_mmvq.cu:339-349).
extern "C" void q4_mmvq_hold(const float *d_x) {
    mv::g_hold = d_x;
    mv::g_cur_x = nullptr;
}
extern "C" void q4_mmvq_release(void) {
    mv::g_hold = nullptr;
    mv::g_cur_x = nullptr;
}

extern "C" bool q4_mmvq_n(uint32_t ty, const uint8_t *d_w, uint64_t nrows, uint64_t ncols, const float *d_x,
                          float *d_y, float scale, uint32_t n) {
    const int mode = q4_mmvq_on();
    if (!mode || !d_w || !d_x || !d_y || n < 1 || n > 8 || ncols > mv::MAXK || (ncols % 32) || !nrows ||
        nrows > 0x7fffffffull)
        return false;
    if (mode == 2 ? !mv::g_scope : n < 2) return false;
    const bool dense = mv::dense_type(ty);
    const bool held = mv::g_hold && mv::g_hold == d_x && mv::g_cur_x == d_x && mv::g_cur_k == ncols &&
                      mv::g_cur_kind == (dense ? 1 : 0) && (dense ? mv::g_cur_n >= n : mv::g_cur_n == n);
    if (!dense) {
        // IQ3_S: the rows go through the grouped expert product as one "expert" that owns all n rows,
        // quantised like every other activation of that product
        if (!grouped::shape_ok(ty, nrows, ncols) || !elem::g_mv_xq) return false;
        if (!held) {
            if (!q4_mmq_quantize(d_x, nullptr, elem::g_mv_xq, ty, ncols, n)) return false;
            mv::g_cur_x = d_x, mv::g_cur_k = ncols, mv::g_cur_n = n, mv::g_cur_kind = 0;
        }
        if (!q4_mmq_mul_id(d_w, ty, nrows, ncols, 0, 1, elem::g_mv_xq, elem::g_mv_bounds + 2 * n, n, n, d_y, nrows))
            return false;
        return scale == 1.0f || q4_hip_scale(d_y, scale, (uint64_t)n * nrows);
    }
    if (!mv::g_q || !mv::dense_fits(ty, d_w, ncols)) return false;   // q4_mmvq_warm allocates, outside any stream capture
    const uint32_t K = (uint32_t)ncols, R = (uint32_t)nrows;
    if (!held) {
        const uint64_t ngr = (uint64_t)n * (K / 32u);
        mv::quant8d_k<<<(unsigned)((ngr + 7) / 8), 256, 0, g_q4b.stream>>>(d_x, ngr, mv::g_q, mv::g_d, mv::g_s);
        g_q4b_launches.fetch_add(1, std::memory_order_relaxed);
        if (!q4b_launch_ok("mmvq_quant")) return false;
        mv::g_cur_x = d_x, mv::g_cur_k = ncols, mv::g_cur_n = n, mv::g_cur_kind = 1;
    }
    switch (ty) {
    case 14u: return mv::launch<14u>(n, d_w, d_y, K, R, scale);
    case 12u: return mv::launch<12u>(n, d_w, d_y, K, R, scale);
    case 13u: return mv::launch<13u>(n, d_w, d_y, K, R, scale);
    case 23u: return mv::launch<23u>(n, d_w, d_y, K, R, scale);
    default: return mv::launch<20u>(n, d_w, d_y, K, R, scale);
    }
}
