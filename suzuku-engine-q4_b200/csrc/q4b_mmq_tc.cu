// Grouped IQ3_S x int8 product on the tensor cores (tcgen05, kind::i8, int32
// accumulators in tensor memory) for the many-rows-per-expert case of
// q4_mmq_mul_id (src/q4_mmq.cu:387, the reference's tile kernel mmq_iq3s_k).
//
// Arithmetic.  The product is defined per 32-element group (src/q4_mmq.cu:130-
// 217): I[m][n][g] = sum_k w[m][k] q[n][k] with w = sign * grid byte (odd, |w| <=
// 15) and q the 8-bit activation, then out[m][n] = sum_g (float)I * (ls * d) *
// dq[n][g].  A group is exactly one K = 32 step of the 8-bit MMA, so every I is
// produced by one instruction into its own accumulator columns and is exact; the
// scale of a group differs per weight row AND per activation row, so the
// scaling cannot be folded into the MMA and runs on the CUDA cores.
//
// One CTA owns 128 weight rows of one expert (the M side of the MMA; a weight
// row is a lane of tensor memory, so its scale is a per-thread scalar) and walks
// the expert's activation rows 64 at a time (the N side).  Per step of 128 k
// (four groups):
//   all 512 threads   decode 128 rows x 4 groups of IQ3_S into int8 core
//                     matrices in shared memory (K-major, no swizzle; the K
//                     chunks are 144 bytes apart so the 16-byte stores of a
//                     quarter warp fall in different banks)
//   TMA               activation rows [64][128 B] through a rank-3 map
//                     (16 B, row, chunk) that lands them as core matrices, and
//                     their group scales [64][4] through a rank-2 map
//   one thread        four MMAs 128 x N x 32, one per group, then a commit
//   all 16 warps      tcgen05.ld of the previous step's accumulators, int ->
//                     float, two multiply-adds per element into registers
// Steps are double-buffered in shared and tensor memory: the MMAs of step i+1
// run under the scaling of step i.  Every wait is bounded; a wait that gives up
// sets the error word and the CTA runs to its end (results then undefined).
#include <cuda.h>

#include "q4b_internal.cuh"
#include "q4b_tile.cuh"

namespace mmqtc {

constexpr uint32_t NT = 512;           // threads
constexpr uint32_t MT = 128;           // weight rows per CTA
constexpr uint32_t NB = 64;            // activation rows per pass
constexpr uint32_t KS = 128;           // k per step (four groups)
constexpr uint32_t A_LBO = 144;        // bytes between the K chunks of a core-matrix row group
constexpr uint32_t A_SBO = 8 * A_LBO;  // bytes between 8-row groups
constexpr uint32_t A_BYTES = (MT / 8) * A_SBO;
constexpr uint32_t B_LBO = NB * 16;    // [chunk][row][16 B]
constexpr uint32_t B_SBO = 128;
constexpr uint32_t B_BYTES = 8 * B_LBO;
constexpr uint32_t DA_BYTES = NB * 16;  // [row][4 floats]
constexpr uint32_t NSTAGE_B = 3;
constexpr uint32_t TMEM_COLS = 512;

struct __align__(128) Smem {
    uint8_t a[2][A_BYTES];
    uint8_t b[NSTAGE_B][B_BYTES];
    float da[NSTAGE_B][NB][4];
    float sw[2][4][MT];
    uint32_t tab2[512];        // doubled code bytes (2c per byte)
    unsigned long long bar_mma[2];
    unsigned long long bar_b[NSTAGE_B];
    uint32_t tmem_base;
    uint32_t failed;
};
// more than half of an SM's shared memory, so that two of these CTAs (each wants
// all 512 columns of tensor memory) are never resident together
constexpr uint32_t SMEM_BYTES = 120 * 1024;
static_assert(sizeof(Smem) + 128 <= SMEM_BYTES, "shared memory layout");

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(unsigned long long *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
// Bounded wait on a phase parity.  Returns false after giving up.
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, uint32_t parity, uint32_t limit) {
    const uint32_t a = smem_u32(bar);
    for (uint32_t i = 0; i < limit; i++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(a), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

// K-major, no swizzle: start address, leading (K chunk) and stride (8-row group)
// byte offsets in 16-byte units, descriptor version 1.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)((lbo >> 4) & 0x3fffu) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3fffu) << 32) | (1ull << 46);
}
// D int32, A and B signed 8-bit, both K-major, M = 128.
__device__ __forceinline__ uint32_t instr_desc(uint32_t n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((MT >> 4) << 24);
}
__device__ __forceinline__ void mma_i8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, 0, 0;\n\t"  // accumulate = false: D = A * B
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        :
        : "r"(tmem_d), "l"(da), "l"(db), "r"(idesc)
        : "memory");
}
__device__ __forceinline__ void mma_commit(unsigned long long *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int32_t *v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
          "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
          "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, int32_t *v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
        : "r"(taddr)
        : "memory");
}
// Packed fp32 pairs (sm_100 f32x2 arithmetic): two products / two fused multiply-adds per
// instruction, each rounded like the scalar form.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long mul2(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b,
                                                   unsigned long long c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, unsigned long long *bar,
                                            int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_u32(dst)),
        "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, unsigned long long *bar,
                                            int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst)),
        "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
        : "memory");
}

struct Args {
    const uint8_t *w;            // first matrix (expert 0), device
    uint64_t expert_stride;
    const int32_t *act;          // entry -> expert slot, or null (entry = slot)
    const uint32_t *n_act;       // live entries, or null
    const int32_t *bounds;       // entry i owns activation rows [bounds[i], bounds[i+1])
    uint32_t cols, w_rows;
    float *dst;
    uint64_t ld_dst;
    const uint32_t *codes;       // byte-expanded code table, device
    uint32_t *err;               // device error word
    uint32_t min_rows;           // entries with fewer rows are left to the CUDA-core kernel
    const uint2 *work;           // (entry, first row) per pass, built by worklist_k
    const uint32_t *n_work;
    uint32_t pass_rows;          // activation rows per pass: 64, or 16 to spread a small call over more CTAs
};

// One item per (entry with min_rows or more rows, pass of NB rows): a hot expert's
// rows spread over many CTAs.  One block; entries are scanned 1024 at a time.
__global__ void __launch_bounds__(1024) worklist_k(const int32_t *__restrict__ bounds,
                                                   const uint32_t *__restrict__ n_act, uint32_t n_entries,
                                                   uint32_t min_rows, uint2 *__restrict__ work,
                                                   uint32_t *__restrict__ n_work, uint32_t cap,
                                                   uint32_t pass_rows) {
    __shared__ uint32_t wsum[32];
    __shared__ uint32_t base_s;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t n_ent = n_act ? min(*n_act, n_entries) : n_entries;
    if (tid == 0) base_s = 0;
    __syncthreads();
    for (uint32_t e0 = 0; e0 < n_ent; e0 += blockDim.x) {
        const uint32_t e = e0 + tid;
        int32_t r0 = 0, nr = 0;
        if (e < n_ent) {
            r0 = bounds[e];
            nr = bounds[e + 1] - r0;
        }
        const uint32_t np =
            (nr > 0 && (uint32_t)nr >= min_rows) ? ((uint32_t)nr + pass_rows - 1u) / pass_rows : 0u;
        uint32_t inc = np;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= (uint32_t)o) inc += t;
        }
        if (lane == 31u) wsum[warp] = inc;
        __syncthreads();
        uint32_t off = base_s;
        for (uint32_t wv = 0; wv < warp; wv++) off += wsum[wv];
        uint32_t pos = off + inc - np;
        for (uint32_t p = 0; p < np; p++, pos++)
            if (pos < cap) work[pos] = make_uint2(e, (uint32_t)r0 + p * pass_rows);
        __syncthreads();
        if (tid == blockDim.x - 1u) base_s = off + inc;
        __syncthreads();
    }
    if (tid == 0) *n_work = min(base_s, cap);
}

constexpr uint32_t WAIT_LIMIT = 1u << 21;   // polls before a wait gives up (about a second)
constexpr uint32_t ERR_MMQ_TC = 0x400u;

// One 32-weight group as true int8 weights: byte = sign * (2c + 1).  With t = 2c
// (even) and m the 0x00/0xFF sign mask, t ^ (m | 1) is 2c+1 or ~(2c) = -(2c+1).
template <bool TILED>
__device__ __forceinline__ void decode_group_w(const Iq3Fields &f, const uint32_t *tab2, uint32_t *wv) {
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const uint32_t wq = k < 4 ? f.qs_lo : f.qs_hi;
        const uint32_t idx = ((wq >> (8 * (k & 3))) & 0xffu) | (((f.qh >> k) & 1u) << 8);
        uint32_t m;
        if (TILED) {
            const uint32_t t = f.sg << k;
            m = q4b_prmt(t, t, 0xba98u);
        } else {
            m = q4b_sign_mask4(f.sg >> (4 * k));
        }
        wv[k] = tab2[idx] ^ (m | 0x01010101u);
    }
}

template <bool TILED>
__global__ void __launch_bounds__(NT, 1) mmq_tc_k(const Args a, const __grid_constant__ CUtensorMap map_q,
                                                  const __grid_constant__ CUtensorMap map_d) {
    // used directly (no integer round trip), so that the compiler keeps these as
    // shared-space accesses; dynamic shared memory starts on the declared alignment
    extern __shared__ __align__(128) uint8_t smem_raw[];
    Smem &s = *reinterpret_cast<Smem *>(smem_raw);
    if (blockIdx.y >= *a.n_work) return;
    const uint2 item = a.work[blockIdx.y];
    const uint32_t entry = item.x;
    const int32_t r0 = (int32_t)item.y;
    const int32_t r1 = min(a.bounds[entry + 1], r0 + (int32_t)a.pass_rows);   // this CTA's pass of the rows
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t B = a.cols >> 8;                 // super-blocks per weight row
    const uint32_t n_it = a.cols / KS;              // steps per pass
    const uint8_t *mat = a.w + (uint64_t)(a.act ? a.act[entry] : (int32_t)entry) * a.expert_stride;
    const uint32_t row0 = blockIdx.x * MT;

    s.tab2[tid] = __ldg(a.codes + tid) << 1;
    if (tid == 0) {
        mbar_init(&s.bar_mma[0], 1);
        mbar_init(&s.bar_mma[1], 1);
        for (uint32_t i = 0; i < NSTAGE_B; i++) mbar_init(&s.bar_b[i], 1);
        s.failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&s.tmem_base)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s.tmem_base;

    // decode role: weight row d_row of the CTA's 128, group d_g of the step's four
    const uint32_t d_row = tid >> 2, d_g = tid & 3u;
    const uint64_t d_blk0 = (uint64_t)(row0 + d_row) * B;
    const uint32_t d_off = (d_row >> 3) * A_SBO + (2u * d_g) * A_LBO + (d_row & 7u) * 16u;
    // scaling role: tensor-memory lanes of this warp's quadrant, 16 of the 64 columns
    const uint32_t e_q = warp & 3u, e_cs = warp >> 2;
    const uint32_t e_row = 32u * e_q + lane;
    const uint32_t e_taddr = tmem + ((32u * e_q) << 16) + 16u * e_cs;

    uint32_t gi = 0;        // steps issued so far by this CTA, across passes (buffer phases)
    uint32_t wait_limit = WAIT_LIMIT;
    for (int32_t rc = r0; rc < r1; rc += (int32_t)NB) {
        const uint32_t nrows = min((uint32_t)(r1 - rc), NB);
        const uint32_t n_mma = (nrows + 15u) & ~15u;
        const uint32_t idesc = instr_desc(n_mma);
        const bool e_live = 16u * e_cs < nrows;
        // per output column two running sums, over the even and the odd groups, held as one
        // packed pair so that a step's scaling is one packed multiply and one packed FMA per
        // two groups; they are added once at the end
        unsigned long long acc2[16];
#pragma unroll
        for (int j = 0; j < 16; j++) acc2[j] = 0ull;

        // producer side of step `it` (global step index g): activations by TMA
        auto issue_b = [&](uint32_t it, uint32_t g) {
            const uint32_t sb = g % NSTAGE_B;
            mbar_expect_tx(&s.bar_b[sb], B_BYTES + DA_BYTES);
            tma_load_3d(s.b[sb], &map_q, &s.bar_b[sb], 0, rc, (int)(it * 8u));
            tma_load_2d(&s.da[sb][0][0], &map_d, &s.bar_b[sb], (int)(it * 4u), rc);
        };
        auto load_fields = [&](uint32_t it) {
            return iq3_fields<TILED>(mat, d_blk0 + (it >> 1), (it & 1u) * 4u + d_g);
        };
        auto decode_to = [&](const Iq3Fields &f, uint32_t buf) {
            uint32_t wv[8];
            decode_group_w<TILED>(f, s.tab2, wv);
            uint8_t *p = s.a[buf] + d_off;
            *reinterpret_cast<uint4 *>(p) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
            *reinterpret_cast<uint4 *>(p + A_LBO) = make_uint4(wv[4], wv[5], wv[6], wv[7]);
            s.sw[buf][d_g][d_row] = __fmul_rn((float)f.ls, f.d);
        };
        auto issue_mma = [&](uint32_t g) {   // one thread
            const uint32_t buf = g & 1u, sb = g % NSTAGE_B;
            if (!mbar_wait(&s.bar_b[sb], (g / NSTAGE_B) & 1u, wait_limit)) {
                atomicOr(a.err, ERR_MMQ_TC | 1u);
                s.failed = 1;
            }
            tc_fence_after();
            const uint32_t a_addr = smem_u32(s.a[buf]), b_addr = smem_u32(s.b[sb]);
#pragma unroll
            for (uint32_t k = 0; k < 4; k++)
                mma_i8(tmem + buf * 256u + k * NB, smem_desc(a_addr + 2u * k * A_LBO, A_LBO, A_SBO),
                       smem_desc(b_addr + 2u * k * B_LBO, B_LBO, B_SBO), idesc);
            mma_commit(&s.bar_mma[buf]);
        };

        // prologue: step 0 of this pass
        if (tid == 0) {
            issue_b(0, gi);
            if (n_it > 1) issue_b(1, gi + 1);
        }
        // the fields of a step are fetched two steps before they are decoded
        Iq3Fields fcur = load_fields(0);
        Iq3Fields fnext = n_it > 1 ? load_fields(1) : fcur;
        Iq3Fields fnext2 = n_it > 2 ? load_fields(2) : fcur;
        decode_to(fcur, gi & 1u);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        if (tid == 0) issue_mma(gi);

        for (uint32_t it = 0; it < n_it; it++) {
            const uint32_t g = gi + it, buf = g & 1u, sb = g % NSTAGE_B;
            if (it + 1 < n_it) {
                fcur = fnext;
                fnext = fnext2;
                if (it + 3 < n_it) fnext2 = load_fields(it + 3);
                if (it + 2 < n_it && tid == 0) issue_b(it + 2, g + 2);
                decode_to(fcur, buf ^ 1u);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            __syncthreads();
            if (it + 1 < n_it && tid == 0) issue_mma(g + 1);
            // scaling of step it
            if (!mbar_wait(&s.bar_mma[buf], (g >> 1) & 1u, wait_limit)) {
                atomicOr(a.err, ERR_MMQ_TC | 2u);
                s.failed = 1;
            }
            tc_fence_after();
            if (e_live) {
                const unsigned long long sw01 = pack2(s.sw[buf][0][e_row], s.sw[buf][1][e_row]);
                const unsigned long long sw23 = pack2(s.sw[buf][2][e_row], s.sw[buf][3][e_row]);
#pragma unroll
                for (uint32_t h = 0; h < 2; h++) {       // two groups at a time ...
#pragma unroll
                    for (uint32_t cq = 0; cq < 2; cq++) {  // ... and eight columns: 16 accumulator words live
                        int32_t c0[8], c1[8];
                        tmem_ld8(e_taddr + buf * 256u + (2u * h) * NB + 8u * cq, c0);
                        tmem_ld8(e_taddr + buf * 256u + (2u * h + 1u) * NB + 8u * cq, c1);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const unsigned long long dq = *reinterpret_cast<const unsigned long long *>(
                                &s.da[sb][16u * e_cs + 8u * cq + j][2u * h]);
                            const unsigned long long t =
                                mul2(pack2((float)c0[j], (float)c1[j]), h ? sw23 : sw01);
                            acc2[8 * cq + j] = fma2(t, dq, acc2[8 * cq + j]);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncthreads();
            if (s.failed) wait_limit = 1024u;   // keep going to the end, without long waits
        }
        gi += n_it;
        if (e_live) {
            float *o = a.dst + (uint64_t)(rc + 16 * (int32_t)e_cs) * a.ld_dst + row0 + e_row;
#pragma unroll
            for (int j = 0; j < 16; j++) {
                float even, odd;
                unpack2(acc2[j], even, odd);
                if (16u * e_cs + j < nrows) o[(uint64_t)j * a.ld_dst] = even + odd;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS)
                     : "memory");
    }
}


// ---- host side ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;
static bool g_ready = false, g_tried = false;
constexpr uint32_t WORK_CAP = 1u << 16;   // passes per launch: entries + rows / 64 must fit
static uint2 *g_work = nullptr;           // two lists, used alternately, so that two launches in a
static uint32_t *g_n_work = nullptr;      // row (gate/up, then down) never share one
static uint32_t g_work_turn = 0;

// Resolve the driver's tensor-map encoder (no link-time dependency on the driver
// library) and raise the kernels' shared-memory limit.  Called once, from init.
bool warm() {
    if (g_tried) return g_ready;
    g_tried = true;
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || !fn) {
        cudaGetLastError();
        return false;
    }
    g_encode = (EncodeTiledFn)fn;
    if (cudaFuncSetAttribute(mmq_tc_k<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
            cudaSuccess ||
        cudaFuncSetAttribute(mmq_tc_k<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
            cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    if (cudaMalloc(&g_work, 2 * WORK_CAP * sizeof(uint2)) != cudaSuccess ||
        cudaMalloc(&g_n_work, 2 * sizeof(uint32_t)) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    g_ready = true;
    return true;
}

bool shape_ok(uint64_t w_rows, uint64_t w_cols) {
    return w_rows != 0 && (w_rows % MT) == 0 && w_cols != 0 && (w_cols % 256u) == 0 && w_cols <= 65536u;
}

// q: int8 [rows][cols] row-major; d: float [rows][cols/32].
bool launch(const uint8_t *w, uint64_t expert_stride, const int32_t *act, const uint32_t *n_act,
            uint32_t n_entries, const int32_t *bounds, const int8_t *q, const float *dq, uint64_t rows,
            uint32_t cols, uint32_t w_rows, float *dst, uint64_t ld_dst, bool tiled, uint32_t min_rows,
            cudaStream_t stream) {
    if (!g_ready || !shape_ok(w_rows, cols) || rows == 0 || rows > 0x7fffffffull) return false;
    // a small call (decode batches: a handful of entries reach the threshold) is cut into
    // passes of 16 rows so that its few entries still spread over many SMs
    const uint32_t pass_rows = rows <= 2048u ? 16u : NB;
    const uint64_t max_items = (uint64_t)n_entries + rows / pass_rows;
    if (max_items > WORK_CAP) return false;
    CUtensorMap map_q, map_d;
    {
        // (16 bytes, row, 16-byte chunk of the row): a box lands as [chunk][row][16 B]
        const cuuint64_t dims[3] = {16, rows, cols / 16u};
        const cuuint64_t strides[2] = {cols, 16};
        const cuuint32_t box[3] = {16, NB, 8};
        const cuuint32_t es[3] = {1, 1, 1};
        if (g_encode(&map_q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, (void *)q, dims, strides, box, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
    }
    {
        const cuuint64_t dims[2] = {cols / 32u, rows};
        const cuuint64_t strides[1] = {(cuuint64_t)(cols / 32u) * 4u};
        const cuuint32_t box[2] = {4, NB};
        const cuuint32_t es[2] = {1, 1};
        if (g_encode(&map_d, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)dq, dims, strides, box, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                     CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
    }
    Args a;
    a.w = w;
    a.expert_stride = expert_stride;
    a.act = act;
    a.n_act = n_act;
    a.bounds = bounds;
    a.cols = cols;
    a.w_rows = w_rows;
    a.dst = dst;
    a.ld_dst = ld_dst;
    a.codes = g_q4b.codes_d;
    a.err = g_q4b.err_d;
    a.min_rows = min_rows;
    const uint32_t turn = g_work_turn++ & 1u;
    a.work = g_work + turn * WORK_CAP;
    a.n_work = g_n_work + turn;
    a.pass_rows = pass_rows;
    worklist_k<<<1, 1024, 0, stream>>>(bounds, n_act, n_entries, min_rows, g_work + turn * WORK_CAP,
                                            g_n_work + turn, WORK_CAP, pass_rows);
    const dim3 grid(w_rows / MT, (unsigned)max_items);
    if (tiled)
        mmq_tc_k<true><<<grid, NT, SMEM_BYTES, stream>>>(a, map_q, map_d);
    else
        mmq_tc_k<false><<<grid, NT, SMEM_BYTES, stream>>>(a, map_q, map_d);
    return true;
}

}  // namespace mmqtc
