// The rest of the device symbols the engine's MoE layer code (src/q4_moe.c) references, so
// that it links against this library unchanged.  Three kinds:
//   * real: host-memory helpers, GEMV forms with host operands or a row gather, small aliases;
//   * declined: alternates of a product this library serves another way (the engine tries
//     q4_mmq_mul_id first; these answer false = "nothing was enqueued", the reference's own
//     rule for an uncovered type, src/q4_rocm.cu:5433-5438), and formats outside the path;
//   * absent machinery: the CPU-miss wait, the routing mailbox, prefetch prediction and the
//     verify-timeline diagnostics belong to expert offload, which a B200 with every expert
//     resident does not have; their entry points answer false / 0 and enqueue nothing.
// Part of the single translation unit q4cuda.cu.
namespace compat {

// y[b][r] = scale * W[r] . x[which ? which[b] : b]; one warp per row, grid.y = batch.
template <bool TILED>
__global__ void __launch_bounds__(256) gemv_which_k(uint32_t type, const uint8_t *__restrict__ w, uint64_t nrows,
                                                    uint32_t ncols, const float *__restrict__ x,
                                                    const int32_t *__restrict__ which, float *__restrict__ y,
                                                    float scale) {
    __shared__ uint32_t tab[512];
    q4b_fill_code_table(tab);
    __syncthreads();
    const uint64_t r = (uint64_t)blockIdx.x * 8u + (threadIdx.x >> 5);
    if (r >= nrows) return;
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t src = which ? (uint64_t)which[blockIdx.y] : (uint64_t)blockIdx.y;
    const float *xb = x + src * ncols;
    float acc = 0.f;
    if (type == Q4_T_F32) {
        const float *wr = reinterpret_cast<const float *>(w) + r * ncols;
        for (uint32_t i = lane; i < ncols; i += 32) acc += wr[i] * xb[i];
    } else {
        acc = iq3s_row_dot_f32<TILED>(w, r, ncols, xb, tab, lane);
    }
    acc = q4b_warp_sum(acc);
    if (lane == 0) y[(uint64_t)blockIdx.y * nrows + r] = scale * acc;
}

bool type_shape_ok(uint32_t type, uint64_t nrows, uint64_t ncols) {
    return nrows && ncols && ncols <= 0xffffffffull &&
           (type == Q4_T_F32 || (type == Q4_T_IQ3_S && (ncols % Q4B_QK) == 0));
}
uint64_t matrix_bytes(uint32_t type, uint64_t nrows, uint64_t ncols) {
    return type == Q4_T_F32 ? nrows * ncols * 4u : nrows * (ncols / Q4B_QK) * Q4B_IQ3S_BYTES;
}

}  // namespace compat

// ---- real ----
extern "C" bool q4_hip_host_register(void *p, size_t n) {
    if (!g_q4b.ok || !p || !n) return false;
    if (cudaHostRegister(p, n, cudaHostRegisterMapped | cudaHostRegisterPortable) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return true;
}
extern "C" void *q4_hip_host_devptr(void *p) {
    void *d = nullptr;
    if (!g_q4b.ok || !p || cudaHostGetDevicePointer(&d, p, 0) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return d;
}
void q4b_stack_forget_host(const void *h);
extern "C" void q4_hip_host_unregister(void *p) {
    if (g_q4b.ok && p) q4b_stack_forget_host(p);
    if (g_q4b.ok && p && cudaHostUnregister(p) != cudaSuccess) cudaGetLastError();
}
// Ordered with the expert uploads: the copy stream.
extern "C" bool q4_hip_copy_memset(void *dst, int v, size_t n) {
    if (!g_q4b.ok || !dst) return false;
    if (!n) return true;
    Q4B_CHECK(cudaMemsetAsync(dst, v, n, g_q4b.copy_stream));
    return true;
}
extern "C" bool q4_hip_moe_act(float *d_g, const float *d_u, uint64_t n) { return q4_hip_silu_mul(d_g, d_u, n); }
extern "C" void q4_hip_mark_pt(int slot) { (void)slot; }   // step-profile boundary marks: not kept

extern "C" bool q4_hip_gemv_dd_n_which(uint32_t ggml_type, const uint8_t *d_w, uint64_t nrows, uint64_t ncols,
                                       const float *d_x, float *d_y, float scale, uint32_t n_batch,
                                       const int32_t *which) {
    if (!which) return q4_hip_gemv_dd_n(ggml_type, d_w, nrows, ncols, d_x, d_y, scale, n_batch);
    if (!g_q4b.ok || !d_w || !d_x || !d_y || !n_batch || !compat::type_shape_ok(ggml_type, nrows, ncols))
        return false;
    const dim3 grid((unsigned)((nrows + 7) / 8), n_batch);
    if (ggml_type == Q4_T_IQ3_S && q4b_ptr_tiled(d_w))
        compat::gemv_which_k<true><<<grid, 256, 0, g_q4b.stream>>>(ggml_type, d_w, nrows, (uint32_t)ncols, d_x,
                                                                   which, d_y, scale);
    else
        compat::gemv_which_k<false><<<grid, 256, 0, g_q4b.stream>>>(ggml_type, d_w, nrows, (uint32_t)ncols, d_x,
                                                                    which, d_y, scale);
    g_q4b_launches++;
    return q4b_launch_ok("gemv_which");
}

// Host operands: x and y (and for q4_hip_gemv the matrix) are copied; synchronous like the
// reference's (src/q4.h:1061-1065).  Set-up paths only: they allocate and free.
extern "C" bool q4_hip_gemv_dev(uint32_t ggml_type, const uint8_t *d_w, uint64_t nrows, uint64_t ncols,
                                const float *x, float *y, float scale) {
    if (!g_q4b.ok || !d_w || !x || !y || !compat::type_shape_ok(ggml_type, nrows, ncols)) return false;
    float *d_x = nullptr, *d_y = nullptr;
    bool ok = cudaMalloc(&d_x, ncols * 4) == cudaSuccess && cudaMalloc(&d_y, nrows * 4) == cudaSuccess &&
              cudaMemcpyAsync(d_x, x, ncols * 4, cudaMemcpyHostToDevice, g_q4b.stream) == cudaSuccess &&
              q4_hip_gemv_dd(ggml_type, d_w, nrows, ncols, d_x, d_y, scale) &&
              cudaMemcpyAsync(y, d_y, nrows * 4, cudaMemcpyDeviceToHost, g_q4b.stream) == cudaSuccess &&
              cudaStreamSynchronize(g_q4b.stream) == cudaSuccess;
    if (!ok) cudaGetLastError();
    cudaFree(d_x);
    cudaFree(d_y);
    return ok;
}
extern "C" bool q4_hip_gemv(uint32_t ggml_type, const uint8_t *w, uint64_t nrows, uint64_t ncols, const float *x,
                            float *y, float scale) {
    if (!g_q4b.ok || !w || !x || !y || !compat::type_shape_ok(ggml_type, nrows, ncols)) return false;
    const uint64_t nb = compat::matrix_bytes(ggml_type, nrows, ncols);
    uint8_t *d_w = nullptr;
    bool ok = cudaMalloc(&d_w, nb) == cudaSuccess &&
              cudaMemcpyAsync(d_w, w, nb, cudaMemcpyHostToDevice, g_q4b.stream) == cudaSuccess &&
              q4_hip_gemv_dev(ggml_type, d_w, nrows, ncols, x, y, scale);
    if (!ok) cudaGetLastError();
    cudaFree(d_w);
    return ok;
}

// ---- declined: the engine reaches these only after q4_mmq_mul_id / q4_hip_moe_exec* refuse ----
extern "C" bool q4_hip_moe_pf(uint32_t, const uint8_t *, uint64_t, uint64_t, const int32_t *, const uint32_t *,
                              const uint32_t *, const int32_t *, const float *, float *, uint32_t, uint32_t,
                              uint32_t) { return false; }
extern "C" bool q4_hip_moe_pf2(uint32_t, const uint8_t *, uint64_t, uint64_t, uint64_t, const int32_t *,
                               const uint32_t *, const uint32_t *, const int32_t *, const float *, float *,
                               float *, uint32_t, uint32_t, uint32_t) { return false; }
extern "C" bool q4_hip_moe_wmma(uint32_t, const uint8_t *, uint64_t, uint64_t, const int32_t *, const uint32_t *,
                                const uint32_t *, const int32_t *, const float *, float *, uint32_t, uint32_t,
                                uint32_t) { return false; }
extern "C" bool q4_hip_moe_wmma2(uint32_t, const uint8_t *, uint64_t, uint64_t, uint64_t, const int32_t *,
                                 const uint32_t *, const uint32_t *, const int32_t *, const float *, float *,
                                 uint32_t, uint32_t, uint32_t) { return false; }
// Q4_K and Q8_0 dense forms: formats outside this path
extern "C" bool q4_hip_gateup_q4k(const uint8_t *, const uint8_t *, const float *, float *, uint32_t, uint32_t) {
    return false;
}
extern "C" bool q4_hip_gateup_q4k_n_which(const uint8_t *, const uint8_t *, const float *, float *, uint32_t,
                                          uint32_t, uint32_t, const int32_t *) { return false; }
extern "C" bool q4_hip_q8_reuse(const uint8_t *, uint64_t, uint64_t, const float *, const int32_t *, float *, float,
                                uint32_t) { return false; }
// the fp16 prefill product (q4_xg_on() is 0, so the engine never gets past the first question)
extern "C" bool q4_xg_gu_type(uint32_t) { return false; }
extern "C" bool q4_xg_dn_type(uint32_t) { return false; }
extern "C" bool q4_xg_shape_ok(uint32_t, uint32_t) { return false; }
extern "C" uint32_t q4_xg_tile_cap(uint32_t, uint32_t) { return 0; }
extern "C" uint32_t q4_xg_tiles(const uint32_t *, const uint32_t *, const int32_t *, uint32_t, int32_t *, uint32_t) {
    return 0;
}
extern "C" bool q4_xg_cvt(const float *, void *, uint64_t) { return false; }
extern "C" bool q4_xg_gu(uint32_t, const uint8_t *, uint64_t, uint64_t, uint64_t, uint32_t, uint32_t, const int32_t *,
                         uint32_t, const void *, const int32_t *, void *) { return false; }
extern "C" bool q4_xg_dn(uint32_t, const uint8_t *, uint64_t, uint64_t, uint32_t, uint32_t, const int32_t *, uint32_t,
                         const void *, float *) { return false; }

// ---- expert offload machinery: not present where every expert is resident ----
extern "C" bool q4_hip_route_dev(const float *, const int32_t *, int32_t *, float *, int32_t *, const int32_t *,
                                 int32_t *, float *, int32_t *, uint32_t, void *, unsigned long long *,
                                 unsigned long long *, unsigned long long *, uint32_t, uint32_t) { return false; }
extern "C" bool q4_hip_route_dev_n(const float *, const int32_t *, int32_t *, float *, int32_t *, void *,
                                   unsigned long long *, unsigned long long *, unsigned long long *, uint32_t,
                                   uint32_t, uint32_t) { return false; }
extern "C" bool q4_hip_cpx_wait(void *, void *, void *) { return false; }
extern "C" bool q4_hip_cpx_spin_init(void) { return false; }
extern "C" bool q4_hip_cpx_spin(const unsigned long long *, const unsigned long long *) { return false; }
extern "C" unsigned long long q4_hip_cpx_wait_timeouts(void) { return 0; }
extern "C" void q4_hip_cpx_wait_reset(void) {}
extern "C" unsigned long long q4_hip_cpx_wait_lastseen(void) { return 0; }
// prefetch prediction record: u64 seq, u64 tseq, i32 n, pad, i32 ids[16], f32 sc[16] (src/q4.h:293-300)
extern "C" size_t q4_hip_pred_size(void) { return 8 + 8 + 4 + 4 + 16 * 4 + 16 * 4; }
extern "C" bool q4_hip_pred_sel(const float *, const int32_t *, const unsigned long long *, unsigned long long *,
                                void *, uint32_t, uint32_t, uint32_t, float) { return false; }
// verify-timeline stamps (diagnostic)
extern "C" bool q4_hip_vtl_init(void) { return false; }
extern "C" bool q4_hip_vtl_stamp(uint32_t) { return false; }
extern "C" bool q4_hip_vtl_read(double *, uint32_t, double) { return false; }
extern "C" double q4_hip_vtl_calib(void) { return 0.0; }
