// The small device routines the engine's MoE layer code issues around the expert products:
// elementwise updates, one-row reductions, the shared expert's gate, the decode layer's
// pack/final pair, the multi-segment GEMV, the per-token exec over device lists and the
// 2..8-row GEMV on 8-bit activations.  Same names, argument meaning and "false = nothing was
// enqueued" rule as the reference (src/q4_rocm.cu:4628-4700, 4708-4900, 5619-5660,
// 11550-11556, 15763-15808, 15920-16024; src/q4_mmvq.cu; src/q4_mmq.cu:576-601).
// Part of the single translation unit q4cuda.cu.
namespace elem {

// ---- elementwise: one grid-stride kernel per operation, float4 where the arrays allow ----
struct OpSilu      { __device__ float operator()(float y, float, float) const { return y / (1.f + expf(-y)); } };
struct OpSigmoid   { __device__ float operator()(float y, float, float) const { return 1.f / (1.f + expf(-y)); } };
struct OpScale     { float s; __device__ float operator()(float y, float, float) const { return y * s; } };
struct OpScaleSilu { float s; __device__ float operator()(float y, float, float) const { const float v = y * s; return v / (1.f + expf(-v)); } };
struct OpMul       { __device__ float operator()(float, float a, float b) const { return a * b; } };
struct OpAdd       { __device__ float operator()(float, float a, float b) const { return a + b; } };
struct OpMulSig    { __device__ float operator()(float, float a, float g) const { return a / (1.f + expf(-g)); } };
struct OpSiluMul   { __device__ float operator()(float y, float u, float) const { return y / (1.f + expf(-y)) * u; } };
struct OpAxpy      { float a; __device__ float operator()(float y, float x, float) const { return y + a * x; } };
struct OpAxpyD     { const float *a; __device__ float operator()(float y, float x, float) const { return y + *a * x; } };

// y[i] = op(y[i], a[i], b[i]); a and b may be null (the op then ignores them) or alias y.
template <class Op, bool VEC>
__global__ void __launch_bounds__(256) map_k(float *y, const float *a, const float *b, uint64_t n, Op op) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (VEC) {
        const uint64_t n4 = n >> 2;
        for (; i < n4; i += stride) {
            float4 vy = reinterpret_cast<float4 *>(y)[i];
            const float4 va = a ? reinterpret_cast<const float4 *>(a)[i] : make_float4(0, 0, 0, 0);
            const float4 vb = b ? reinterpret_cast<const float4 *>(b)[i] : make_float4(0, 0, 0, 0);
            vy.x = op(vy.x, va.x, vb.x);
            vy.y = op(vy.y, va.y, vb.y);
            vy.z = op(vy.z, va.z, vb.z);
            vy.w = op(vy.w, va.w, vb.w);
            reinterpret_cast<float4 *>(y)[i] = vy;
        }
        if (blockIdx.x == 0)   // the last n % 4 elements
            for (uint64_t j = (n4 << 2) + threadIdx.x; j < n; j += blockDim.x)
                y[j] = op(y[j], a ? a[j] : 0.f, b ? b[j] : 0.f);
    } else {
        for (; i < n; i += stride) y[i] = op(y[i], a ? a[i] : 0.f, b ? b[i] : 0.f);
    }
}

template <class Op>
bool map(const char *what, float *y, const float *a, const float *b, uint64_t n, Op op) {
    const bool vec = n >= 1024 && (((uintptr_t)y | (uintptr_t)a | (uintptr_t)b) & 15u) == 0;
    const uint64_t items = vec ? n >> 2 : n;
    uint64_t blocks = (items + 255) / 256;
    const uint64_t cap = (uint64_t)g_q4b.n_sm * 8u;  // beyond this the grid strides
    if (blocks > cap) blocks = cap;
    if (vec)
        map_k<Op, true><<<(unsigned)blocks, 256, 0, g_q4b.stream>>>(y, a, b, n, op);
    else
        map_k<Op, false><<<(unsigned)blocks, 256, 0, g_q4b.stream>>>(y, a, b, n, op);
    g_q4b_launches++;
    return q4b_launch_ok(what);
}

// ---- one-row reductions (one CTA; the rows here are a few thousand floats) ----
__device__ __forceinline__ float block_dot(const float *a, const float *b, uint32_t n, float *red) {
    float acc = 0.f;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) acc += a[i] * b[i];
    acc = q4b_warp_sum(acc);
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    float d = 0.f;
    for (uint32_t k = 0; k < (blockDim.x >> 5); k++) d += red[k];
    return d;
}
template <bool SIG>
__global__ void __launch_bounds__(256) dot_k(const float *a, const float *b, float *out, uint32_t n) {
    __shared__ float red[8];
    const float d = block_dot(a, b, n, red);
    if (threadIdx.x == 0) *out = SIG ? 1.f / (1.f + expf(-d)) : d;
}

// ---- per-token rows: y[t] += g_t * x[t], the gate g_t one scalar per token ----
// One CTA per token sweeps the whole row (float4 when the row allows), after the gate functor
// has produced the token's scalar for all its threads: a table entry, or the sigmoid of a dot
// product the CTA forms first (the shared expert's gate, src/q4_moe.c:1404-1435).
struct GateTable {
    const float *g;
    __device__ float operator()(uint32_t t, uint32_t, float *) const { return g[t]; }
};
struct GateSigmoidDot {
    const float *w, *x;
    __device__ float operator()(uint32_t t, uint32_t n, float *red) const {
        const float d = block_dot(w, x + (size_t)t * n, n, red);
        return 1.f / (1.f + expf(-d));
    }
};
template <class Gate>
__global__ void __launch_bounds__(256) gated_rows_k(float *y, const float *x, uint32_t n, Gate gate) {
    __shared__ float red[8];
    const uint32_t t = blockIdx.x;
    const OpAxpy op{gate(t, n, red)};
    float *yr = y + (size_t)t * n;
    const float *xr = x + (size_t)t * n;
    if ((n & 3u) == 0 && ((((uintptr_t)yr) | ((uintptr_t)xr)) & 15u) == 0) {
        for (uint32_t i = threadIdx.x; i < (n >> 2); i += blockDim.x) {
            float4 vy = reinterpret_cast<float4 *>(yr)[i];
            const float4 vx = reinterpret_cast<const float4 *>(xr)[i];
            vy.x = op(vy.x, vx.x, 0.f);
            vy.y = op(vy.y, vx.y, 0.f);
            vy.z = op(vy.z, vx.z, 0.f);
            vy.w = op(vy.w, vx.w, 0.f);
            reinterpret_cast<float4 *>(yr)[i] = vy;
        }
    } else {
        for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) yr[i] = op(yr[i], xr[i], 0.f);
    }
}

// ---- decode layer head and tail (the engine's pack / final pair, src/q4.h:971-976) ----
// Head, one CTA: y = 0; the shared expert's projections through the SwiGLU functor in place;
// the optional gate scalar sigmoid(x . sgate); the optional counter bump last.
__global__ void __launch_bounds__(256) moe_pack_k(float *y, const float *x, const float *sgate, float *dot,
                                                  uint32_t *flag, uint32_t n_embd, float *sm,
                                                  const float *sm2, uint32_t n_sm) {
    __shared__ float red[8];
    const OpSiluMul act{};
    for (uint32_t j = threadIdx.x; j < n_sm; j += blockDim.x) sm[j] = act(sm[j], sm2[j], 0.f);
    for (uint32_t j = threadIdx.x; j < n_embd; j += blockDim.x) y[j] = 0.f;
    if (sgate) {
        const float g = GateSigmoidDot{sgate, x}(0, n_embd, red);
        if (threadIdx.x == 0) *dot = g;
    }
    __syncthreads();
    if (flag && threadIdx.x == 0) *flag += 1u;
}
// Tail: the hc stream factors 2 sigmoid(inj[c] / hc) are formed once per CTA in shared memory;
// the CTA then walks its share of the row, forms the layer's sum once per element and adds its
// multiples to the hc residual streams.
constexpr uint32_t FINAL_MAX_HC = 64;
__global__ void __launch_bounds__(256) moe_final_k(float *res, const float *y, const float *hy, const float *sh,
                                                   const float *dot, const float *inj, uint32_t n_embd,
                                                   uint32_t hc) {
    __shared__ float factor[FINAL_MAX_HC];
    for (uint32_t c = threadIdx.x; c < hc; c += blockDim.x) factor[c] = hc_stream_factor(inj, 0, hc, c);
    __syncthreads();
    const float gate = dot ? *dot : 1.f;
    const uint32_t step = gridDim.x * blockDim.x;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n_embd; i += step) {
        const float sum = (y[i] + hy[i]) + sh[i] * gate;
        float *stream = res + i;
        for (uint32_t c = 0; c < hc; c++, stream += n_embd) *stream = __fmaf_rn(sum, factor[c], *stream);
    }
}

// ---- multi-segment GEMV: up to 8 matrices against one vector in one launch ----
struct Segs {
    const uint8_t *w[8];
    float *out[8];
    uint32_t first[9];  // first global row of a segment; first[nseg] = total
    uint32_t ty[8];
    uint32_t tiled[8];
    float act[8];
    uint32_t nseg;
};
// One warp per row (8 per CTA).  act != 0: v = act * v, then SiLU (the scale + activation
// epilogue the reference gives its shared-expert gate rows).
__global__ void __launch_bounds__(256) gemv_m_k(const __grid_constant__ Segs S, const float *__restrict__ x,
                                                uint32_t in_dim) {
    __shared__ uint32_t tab[512];
    q4b_fill_code_table(tab);
    __syncthreads();
    const uint32_t row = blockIdx.x * 8u + (threadIdx.x >> 5), lane = threadIdx.x & 31u;
    if (row >= S.first[S.nseg]) return;
    uint32_t s = 0;
    while (s + 1 < S.nseg && row >= S.first[s + 1]) s++;
    const uint32_t r = row - S.first[s];
    float acc = 0.f;
    if (S.ty[s] == Q4_T_F32) {
        const float *wr = reinterpret_cast<const float *>(S.w[s]) + (size_t)r * in_dim;
        for (uint32_t i = lane; i < in_dim; i += 32) acc += wr[i] * x[i];
    } else if (S.tiled[s]) {
        acc = iq3s_row_dot_f32<true>(S.w[s], r, in_dim, x, tab, lane);
    } else {
        acc = iq3s_row_dot_f32<false>(S.w[s], r, in_dim, x, tab, lane);
    }
    acc = q4b_warp_sum(acc);
    if (lane == 0) {
        const float a = S.act[s];
        if (a != 0.f) {
            acc *= a;
            acc = acc / (1.f + expf(-acc));
        }
        S.out[s][r] = acc;
    }
}

// ---- per-token exec over packed device lists: scatter them into the window layout ----
struct TokOff {
    uint32_t off[9];
};
__global__ void tok_lists_k(const int32_t *__restrict__ slots, const float *__restrict__ wts,
                            const __grid_constant__ TokOff O, uint32_t n_tok, int32_t *__restrict__ es,
                            float *__restrict__ ew, int32_t *__restrict__ nh) {
    const uint32_t t = threadIdx.x >> 6, k = threadIdx.x & 63u;
    if (t >= n_tok) return;
    const uint32_t cnt = O.off[t + 1] - O.off[t];
    if (k == 0) nh[t] = (int32_t)cnt;
    if (k < cnt) {
        es[t * 64u + k] = slots[O.off[t] + k];
        ew[t * 64u + k] = wts[O.off[t] + k];
    }
}

// library-owned scratch: window lists for exec_tok; q8 rows and bounds of the IQ3_S rows of q4_mmvq_n
int32_t *g_tok_es = nullptr;
float *g_tok_ew = nullptr;
int32_t *g_tok_nh = nullptr;
void *g_mv_xq = nullptr;        // q8 of up to 8 rows of Q4B_XQ_MAXLEN
int32_t *g_mv_bounds = nullptr; // [9][2]: {0, n}
// expert-indexed weight buffers handed out by q4_mmq_wbuf
uint8_t *g_wbuf_gu = nullptr, *g_wbuf_d = nullptr;
uint64_t g_wbuf_gu_bytes = 0, g_wbuf_d_bytes = 0;
bool g_wbuf_tiled = false;
bool g_wbuf_lent = false;   // the buffers are the caller's memory (q4_mmq_wbuf_lend)

bool warm() {
    if (!g_tok_es) {
        if (cudaMalloc(&g_tok_es, 512 * 4) != cudaSuccess || cudaMalloc(&g_tok_ew, 512 * 4) != cudaSuccess ||
            cudaMalloc(&g_tok_nh, 8 * 4) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
    }
    if (!g_mv_xq) {
        int32_t b[18];
        for (int n = 0; n < 9; n++) {
            b[2 * n] = 0;
            b[2 * n + 1] = n;
        }
        if (cudaMalloc(&g_mv_xq, q8_bytes(8, Q4B_XQ_MAXLEN)) != cudaSuccess ||
            cudaMalloc(&g_mv_bounds, sizeof b) != cudaSuccess ||
            cudaMemcpy(g_mv_bounds, b, sizeof b, cudaMemcpyHostToDevice) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
    }
    return true;
}

}  // namespace elem

bool q4b_elem_warm() { return elem::warm(); }
bool q4b_wbuf_tiled(const void *p) {
    const uint8_t *q = (const uint8_t *)p;
    return elem::g_wbuf_tiled &&
           ((elem::g_wbuf_gu && q >= elem::g_wbuf_gu && q < elem::g_wbuf_gu + elem::g_wbuf_gu_bytes) ||
            (elem::g_wbuf_d && q >= elem::g_wbuf_d && q < elem::g_wbuf_d + elem::g_wbuf_d_bytes));
}
void q4b_elem_shutdown() {
    using namespace elem;
    cudaFree(g_tok_es);
    cudaFree(g_tok_ew);
    cudaFree(g_tok_nh);
    cudaFree(g_mv_xq);
    cudaFree(g_mv_bounds);
    if (!g_wbuf_lent) {
        cudaFree(g_wbuf_gu);
        cudaFree(g_wbuf_d);
    }
    g_wbuf_lent = false;
    g_tok_es = nullptr;
    g_tok_ew = nullptr;
    g_tok_nh = nullptr;
    g_mv_xq = nullptr;
    g_mv_bounds = nullptr;
    g_wbuf_gu = g_wbuf_d = nullptr;
    g_wbuf_gu_bytes = g_wbuf_d_bytes = 0;
    g_wbuf_tiled = false;
}

// ------------------------------------------------------------------ entry points
extern "C" void q4_hip_clear(void) { (void)cudaGetLastError(); }

extern "C" bool q4_hip_silu(float *d, uint64_t n) {
    return g_q4b.ok && d && n && elem::map("silu", d, nullptr, nullptr, n, elem::OpSilu{});
}
extern "C" bool q4_hip_sigmoid(float *d, uint64_t n) {
    return g_q4b.ok && d && n && elem::map("sigmoid", d, nullptr, nullptr, n, elem::OpSigmoid{});
}
extern "C" bool q4_hip_scale(float *d, float s, uint64_t n) {
    return g_q4b.ok && d && n && elem::map("scale", d, nullptr, nullptr, n, elem::OpScale{s});
}
extern "C" bool q4_hip_scale_silu(float *x, float s, uint64_t n) {
    return g_q4b.ok && x && n && elem::map("scale_silu", x, nullptr, nullptr, n, elem::OpScaleSilu{s});
}
extern "C" bool q4_hip_mul(float *y, const float *a, const float *b, uint64_t n) {
    return g_q4b.ok && y && a && b && n && elem::map("mul", y, a, b, n, elem::OpMul{});
}
extern "C" bool q4_hip_add(float *y, const float *a, const float *b, uint64_t n) {
    return g_q4b.ok && y && a && b && n && elem::map("add", y, a, b, n, elem::OpAdd{});
}
extern "C" bool q4_hip_mul_sig(float *y, const float *a, const float *g, uint64_t n) {
    return g_q4b.ok && y && a && g && n && elem::map("mul_sig", y, a, g, n, elem::OpMulSig{});
}
extern "C" bool q4_hip_silu_mul(float *g, const float *u, uint64_t n) {
    return g_q4b.ok && g && u && n && elem::map("silu_mul", g, u, nullptr, n, elem::OpSiluMul{});
}
extern "C" bool q4_hip_axpy(float *y, const float *x, float a, uint64_t n) {
    return g_q4b.ok && y && x && n && elem::map("axpy", y, x, nullptr, n, elem::OpAxpy{a});
}
extern "C" bool q4_hip_axpy_dalpha(float *y, const float *x, const float *d_alpha, uint64_t n) {
    return g_q4b.ok && y && x && d_alpha && n && elem::map("axpy_dalpha", y, x, nullptr, n, elem::OpAxpyD{d_alpha});
}
extern "C" bool q4_hip_axpy_rows(float *d_y, const float *d_x, const float *d_sg, uint32_t n, uint32_t n_tok) {
    if (!g_q4b.ok || !d_y || !d_x || !d_sg || !n || !n_tok) return false;
    elem::gated_rows_k<<<n_tok, 256, 0, g_q4b.stream>>>(d_y, d_x, n, elem::GateTable{d_sg});
    g_q4b_launches++;
    return q4b_launch_ok("axpy_rows");
}
extern "C" bool q4_hip_dot(const float *a, const float *b, float *out, uint32_t n) {
    if (!g_q4b.ok || !a || !b || !out) return false;
    elem::dot_k<false><<<1, 256, 0, g_q4b.stream>>>(a, b, out, n);
    g_q4b_launches++;
    return q4b_launch_ok("dot");
}
extern "C" bool q4_hip_dot_sigmoid(const float *a, const float *b, float *out, uint32_t n) {
    if (!g_q4b.ok || !a || !b || !out) return false;
    elem::dot_k<true><<<1, 256, 0, g_q4b.stream>>>(a, b, out, n);
    g_q4b_launches++;
    return q4b_launch_ok("dot_sigmoid");
}
extern "C" bool q4_hip_sgate_axpy(float *d_y, const float *d_sh, const float *d_w, const float *d_x, uint32_t n,
                                  uint32_t n_tok) {
    if (!g_q4b.ok || !d_y || !d_sh || !d_w || !d_x || !n || !n_tok) return false;
    elem::gated_rows_k<<<n_tok, 256, 0, g_q4b.stream>>>(d_y, d_sh, n, elem::GateSigmoidDot{d_w, d_x});
    g_q4b_launches++;
    return q4b_launch_ok("sgate_axpy");
}

// qx asks the reference to quantise x for the exec that follows; the exec entry points here
// quantise x themselves (same Q8 values), so it needs nothing.
extern "C" bool q4_hip_moe_pack(float *d_y, const float *d_x, const float *d_sgate, float *d_dot, void *flag_d,
                                uint32_t n_embd, bool qx, float *sm, const float *sm2, uint32_t n_sm) {
    (void)qx;
    if (!g_q4b.ok || !d_y || !d_x || !n_embd) return false;
    if (d_sgate && !d_dot) return false;
    if (n_sm && (!sm || !sm2)) return false;
    elem::moe_pack_k<<<1, 256, 0, g_q4b.stream>>>(d_y, d_x, d_sgate, d_dot, (uint32_t *)flag_d, n_embd, sm, sm2,
                                                  n_sm);
    g_q4b_launches++;
    return q4b_launch_ok("moe_pack");
}
extern "C" bool q4_hip_moe_final(float *res, const float *y, const float *hy, const float *sh, const float *dot,
                                 const float *inj, uint32_t n_embd, uint32_t hc) {
    if (!g_q4b.ok || !n_embd || !hc || hc > elem::FINAL_MAX_HC) return false;
    for (const float *p : {(const float *)res, y, hy, sh, inj})
        if (!p) return false;
    uint32_t blocks = (n_embd + 255u) / 256u;
    if (blocks > (uint32_t)g_q4b.n_sm * 4u) blocks = (uint32_t)g_q4b.n_sm * 4u;
    elem::moe_final_k<<<blocks, 256, 0, g_q4b.stream>>>(res, y, hy, sh, dot, inj, n_embd, hc);
    g_q4b_launches++;
    return q4b_launch_ok("moe_final");
}

// Segment types: F32 (any width) and IQ3_S (width a multiple of 256), the two the MoE path's
// shared-expert and gate tensors come in here.
extern "C" bool q4_hip_gemv_m(const q4_seg_t *segs, uint32_t nseg, const float *d_x, uint32_t in_dim) {
    if (!g_q4b.ok || !segs || !d_x || !nseg || nseg > 8 || !in_dim) return false;
    elem::Segs S;
    memset(&S, 0, sizeof S);
    S.nseg = nseg;
    uint32_t tot = 0;
    for (uint32_t i = 0; i < nseg; i++) {
        if (!segs[i].w || !segs[i].out || !segs[i].rows) return false;
        if (segs[i].ty != Q4_T_F32 && !(segs[i].ty == Q4_T_IQ3_S && (in_dim % Q4B_QK) == 0)) return false;
        S.w[i] = segs[i].w;
        S.out[i] = segs[i].out;
        S.ty[i] = segs[i].ty;
        S.tiled[i] = segs[i].ty == Q4_T_IQ3_S && q4b_ptr_tiled(segs[i].w) ? 1u : 0u;
        S.act[i] = segs[i].act;
        S.first[i] = tot;
        tot += segs[i].rows;
    }
    S.first[nseg] = tot;
    elem::gemv_m_k<<<(tot + 7u) / 8u, 256, 0, g_q4b.stream>>>(S, d_x, in_dim);
    g_q4b_launches++;
    return q4b_launch_ok("gemv_m");
}

// Per-token exec over packed device lists (token t owns entries [h_off[t], h_off[t+1])).  Two to
// eight tokens of IQ3_S experts go through the window path, which decodes every distinct expert
// once for all the tokens that picked it; anything else runs token by token.  Either way a
// token's result is what q4_hip_moe_exec_dev gives for it alone.
extern "C" bool q4_hip_moe_exec_tok(const uint8_t *base, uint64_t stride, const int32_t *d_slots,
                                    const float *d_wts, const uint32_t *h_off, uint32_t n_tok, uint32_t gt,
                                    uint64_t og, uint32_t ut, uint64_t ou, uint32_t dt, uint64_t od,
                                    const float *d_x, float *d_h, float *d_h2, float *d_y, uint32_t n_ff,
                                    uint32_t in_dim, uint32_t n_embd) {
    (void)d_h2;
    if (!g_q4b.ok || !base || !d_slots || !d_wts || !h_off || !n_tok || !d_x || !d_h || !d_y || !n_embd)
        return false;
    if (!shape_ok(gt, ut, dt, in_dim, n_ff) || !place_ok(gt, dt, base)) return false;
    for (uint32_t t = 0; t < n_tok; t++)
        if (h_off[t + 1] < h_off[t] || h_off[t + 1] - h_off[t] > 64u) return false;
    if (h_off[n_tok] == h_off[0]) return true;
    if (n_tok >= 2 && n_tok <= 8 && n_embd <= 16384u && q4_hip_moe_win_ok(gt, ut, dt, in_dim, n_ff, n_tok) &&
        grouped::shape_ok(Q4_T_IQ3_S, n_embd, n_ff) && elem::warm()) {
        elem::TokOff O;
        for (uint32_t t = 0; t <= 8; t++) O.off[t] = h_off[t < n_tok ? t : n_tok];
        elem::tok_lists_k<<<1, 512, 0, g_q4b.stream>>>(d_slots, d_wts, O, n_tok, elem::g_tok_es, elem::g_tok_ew,
                                                      elem::g_tok_nh);
        g_q4b_launches++;
        if (!q4b_launch_ok("tok_lists")) return false;
        return q4_hip_moe_exec_win(base, stride, elem::g_tok_es, elem::g_tok_ew, elem::g_tok_nh, n_tok, gt, og, ut,
                                   ou, dt, od, d_x, d_h, d_y, n_ff, in_dim, n_embd);
    }
    for (uint32_t t = 0; t < n_tok; t++) {
        const uint32_t cnt = h_off[t + 1] - h_off[t];
        if (!cnt) continue;
        if (!quant_x(d_x + (size_t)t * in_dim, in_dim)) return false;
        if (!moe_exec_tail(base, stride, d_slots + h_off[t], d_wts + h_off[t], cnt, nullptr, og, ou, od,
                           d_h + (size_t)h_off[t] * n_ff, d_y + (size_t)t * n_embd, n_ff, in_dim, n_embd, dt, gt))
            return false;
    }
    return true;
}

// ---- expert-indexed weight buffers and the gather into them (src/q4.h:1144-1174) ----
// The engine gathers when its arena slots are not in expert order; with every expert resident
// in slot = id it can pass the arena itself to q4_mmq_mul_id and skip both calls.
extern "C" int q4_xg_on(void) { return 0; }  // the fp16 prefill product of the reference: not offered

// Lend mode (src/q4.h:1165-1169): from the first q4_mmq_wbuf_lend on, the two buffers are the
// caller's memory (or absent) and q4_mmq_wbuf never allocates again.
extern "C" bool q4_mmq_wbuf_lend(void *gu, uint64_t gu_bytes, void *d, uint64_t d_bytes) {
    if (!g_q4b.ok) return false;
    if (!elem::g_wbuf_lent) {
        cudaStreamSynchronize(g_q4b.stream);
        cudaFree(elem::g_wbuf_gu);
        cudaFree(elem::g_wbuf_d);
        elem::g_wbuf_lent = true;
    }
    elem::g_wbuf_gu = (uint8_t *)gu;
    elem::g_wbuf_d = (uint8_t *)d;
    elem::g_wbuf_gu_bytes = gu ? gu_bytes : 0;
    elem::g_wbuf_d_bytes = d ? d_bytes : 0;
    elem::g_wbuf_tiled = false;
    return true;
}

extern "C" bool q4_mmq_wbuf(uint64_t gu_bytes, uint64_t d_bytes, uint32_t n_exp, uint8_t **gu, uint8_t **d) {
    if (!g_q4b.ok || !gu || !d || !n_exp) return false;
    const uint64_t need_gu = gu_bytes * n_exp, need_d = d_bytes * n_exp;
    if (elem::g_wbuf_lent) {   // borrowed buffers only
        if (!elem::g_wbuf_gu || !elem::g_wbuf_d || need_gu > elem::g_wbuf_gu_bytes || need_d > elem::g_wbuf_d_bytes)
            return false;
        *gu = elem::g_wbuf_gu;
        *d = elem::g_wbuf_d;
        return true;
    }
    if (need_gu > elem::g_wbuf_gu_bytes) {
        cudaStreamSynchronize(g_q4b.stream);
        cudaFree(elem::g_wbuf_gu);
        elem::g_wbuf_gu = nullptr;
        elem::g_wbuf_gu_bytes = 0;
        if (cudaMalloc(&elem::g_wbuf_gu, need_gu) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        elem::g_wbuf_gu_bytes = need_gu;
    }
    if (need_d > elem::g_wbuf_d_bytes) {
        cudaStreamSynchronize(g_q4b.stream);
        cudaFree(elem::g_wbuf_d);
        elem::g_wbuf_d = nullptr;
        elem::g_wbuf_d_bytes = 0;
        if (cudaMalloc(&elem::g_wbuf_d, need_d) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        elem::g_wbuf_d_bytes = need_d;
    }
    *gu = elem::g_wbuf_gu;
    *d = elem::g_wbuf_d;
    return true;
}

namespace elem {
// Pair p copies slot[p]'s gate|up bytes to gu + eid[p] * gu_dst and its down bytes to
// d + eid[p] * d_dst, 16 bytes per thread; the destination tails beyond the byte counts are zeroed.
__global__ void __launch_bounds__(256) gather16_k(const uint8_t *__restrict__ abase, uint64_t astride,
                                                  uint64_t goff, uint64_t gu_bytes, uint64_t doff,
                                                  uint64_t d_bytes, uint64_t gu_dst, uint64_t d_dst,
                                                  const int32_t *__restrict__ eid,
                                                  const int32_t *__restrict__ slot, uint8_t *__restrict__ gu,
                                                  uint8_t *__restrict__ d) {
    const uint32_t p = blockIdx.y;
    const uint8_t *src = abase + (uint64_t)slot[p] * astride;
    uint8_t *g = gu + (uint64_t)eid[p] * gu_dst, *dd = d + (uint64_t)eid[p] * d_dst;
    const uint64_t ng = gu_dst >> 4, nd = d_dst >> 4;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < ng + nd;
         i += (uint64_t)gridDim.x * blockDim.x) {
        if (i < ng) {
            reinterpret_cast<uint4 *>(g)[i] =
                (i << 4) < gu_bytes ? reinterpret_cast<const uint4 *>(src + goff)[i] : zero;
        } else {
            const uint64_t j = i - ng;
            reinterpret_cast<uint4 *>(dd)[j] =
                (j << 4) < d_bytes ? reinterpret_cast<const uint4 *>(src + doff)[j] : zero;
        }
    }
}
}  // namespace elem

extern "C" bool q4_mmq_gather(const uint8_t *abase, uint64_t astride, uint64_t goff, uint64_t gu_bytes,
                              uint64_t doff, uint64_t d_bytes, uint64_t gu_dst, uint64_t d_dst,
                              const int32_t *d_eid, const int32_t *d_slot, uint32_t n, uint8_t *d_gu,
                              uint8_t *d_d) {
    if (!abase || !d_eid || !d_slot || !d_gu || !d_d || !n) return !n;
    if (!g_q4b.ok || gu_dst < gu_bytes || d_dst < d_bytes) return false;
    // the copy moves 16-byte words: every address, offset, size and stride must be a whole number of them
    for (const uint64_t v : {(uint64_t)(uintptr_t)abase, (uint64_t)(uintptr_t)d_gu, (uint64_t)(uintptr_t)d_d, astride,
                             goff, doff, gu_bytes, d_bytes, gu_dst, d_dst})
        if (v % 16u) return false;
    const bool tiled = q4b_ptr_tiled(abase);
    // a tiled arena's bytes stay tiled in the copy: whole 880-byte tiles must move together
    if (tiled && ((goff % Q4B_TILE_BYTES) || (doff % Q4B_TILE_BYTES) || (gu_bytes % Q4B_TILE_BYTES) ||
                  (d_bytes % Q4B_TILE_BYTES) || (gu_dst % Q4B_TILE_BYTES) || (d_dst % Q4B_TILE_BYTES)))
        return false;
    if (d_gu == elem::g_wbuf_gu || d_d == elem::g_wbuf_d) elem::g_wbuf_tiled = tiled;
    else if (tiled) return false;  // only the library's own buffers can be marked as tiled
    const uint64_t items = (gu_dst + d_dst) >> 4;
    uint64_t bx = (items + 255) / 256;
    if (bx > 64) bx = 64;
    elem::gather16_k<<<dim3((unsigned)bx, n), 256, 0, g_q4b.stream>>>(abase, astride, goff, gu_bytes, doff, d_bytes,
                                                                     gu_dst, d_dst, d_eid, d_slot, d_gu, d_d);
    g_q4b_launches++;
    return q4b_launch_ok("mmq_gather");
}
