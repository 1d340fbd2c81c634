// Grouped IQ3_S x 8-bit product on the tensor cores (tcgen05, fp32 accumulators in tensor
// memory) for the many-rows-per-expert case of q4_mmq_mul_id (src/q4_mmq.cu:387, the
// reference's tile kernel mmq_iq3s_k).
//
// Arithmetic.  The product is defined per 32-element group (src/q4_mmq.cu:130-217):
//   out[m][n] = sum_g (float)I[m][n][g] * (ls[m][g] * d[m]) * dq[n][g],  I = sum_k w q
// with w = sign * grid byte (odd, |w| <= 15), ls = 1 + 2 s (odd, <= 31), d the super-block's
// fp16 scale and q, dq the 8-bit activation and its group scale.  The group scale differs per
// weight row AND per activation row, so with 8-bit integer MMAs (one K = 32 instruction per
// group) every group's int32 sums have to come back to the CUDA cores for int -> float and two
// multiplies: 3.3 instructions per output element and group, 30 times the MMA's own time -
// that form of this kernel ran with the tensor pipe 3 % busy.  Here the scales ride in the
// operands instead:
//   A[m][k] = w * ls                as fp16: an integer of magnitude <= 465, exact
//   B[n][k] = q * dq[n][g] / rs[n]  as the sum of two fp16 numbers (rs = a power of two that
//                                   brings the row's largest value below 1): 22 bits
// and the fp16 MMA accumulates A * B in fp32 over the eight groups of a super-block, whose
// sum needs one multiply by d[m] (and the whole row one by rs[n]) on the CUDA cores: 1/8
// fused multiply-add per element and group instead of 3.3 instructions.  The products are
// the reference's integers times the reference's scales; a term q * dq differs from the exact
// one by at most max(2^-22 of its size, 2^-25 of rs) -- the second plane of a value far below
// the row's maximum falls into fp16's subnormal range, whose spacing is 2^-24 of rs -- and the
// group sums are added in fp32 by the tensor core instead of after an exact integer sum.  The
// error is therefore small against the row's largest group, not against every group: a row
// with one channel 1000 times the rest keeps ~15 bits for the rest (tested: the outputs still
// agree with the CUDA-core kernels to < 1e-4 rel-L2); q4_cuda_mmq_tc_mode(0) avoids it.  With unit scales the result
// is the exact integer product (tested bit for bit); against the CUDA-core kernels, which do
// form the integer sums, the outputs agree to ~1e-6 rel-L2.
//
// One CTA owns 128 weight rows of one expert (the M side; a weight row is a lane of tensor
// memory, so d[m] is a per-thread scalar) and one pass of up to 64 activation rows (N side).
// Per step of 128 k (four groups; two steps = one super-block = one accumulator):
//   16 warps          decode 128 rows x 4 groups of IQ3_S into fp16 rows of 128 bytes in
//                     shared memory under the 128-byte swizzle (the layout TMA writes for the
//                     other operand; a quarter warp's 16-byte stores hit eight different
//                     16-byte columns); the fields of a step are loaded two steps ahead
//                     into registers that are never moved (the loop is unrolled by two);
//                     a CTA walks several 128-row tiles of its pass in one pipeline
//   copy warp         the two fp16 planes of the activation rows as [rows][128 B] TMA boxes
//                     under the 128-byte swizzle, second plane stored right behind the first,
//                     so that one MMA takes both as its N side
//   MMA warp          waits for both operands, issues 8 MMAs 128 x 2N x 16 with precomputed
//                     descriptors and commits; it does nothing else, because one thread's
//                     instruction stream is slow (~60 cycles per MMA, ~250 per barrier test
//                     while the other warps keep the shared-memory pipe busy)
//   16 warps          after every second step: tcgen05.ld of the finished super-block's
//                     accumulator (both planes' halves), one add and one FMA per element
// The warps meet only through mbarriers (weights full / MMAs done / accumulator read /
// activations landed / stage free): weights and activations are double-buffered in shared
// memory, super-blocks in tensor memory.  Every wait is bounded; a wait that gives up sets
// the error word and the CTA runs to its end (results then undefined).
//
// What was measured on the way (a 20k-row call, 160 experts, 1024 x 2048 weights): all warps
// decoding and one of them also issuing, with __syncthreads between the stages, 0.74 ms; the
// issue moved to its own warp 0.59; both planes in one MMA 0.58; copies in a second extra warp
// 0.50; field registers that are not moved (a move waits for its load) 0.44.  Asking for
// 200 KB of shared memory instead of 168 KB cost 15 %: the scattered field loads live on the
// L1 cache that is left.  A 16-byte-wide TMA box that lands as core matrices directly costs one
// request per 16 bytes (~2000 cycles per step); an unswizzled weight layout was as fast as the
// swizzled one.
#include <cuda.h>

#include "q4b_internal.cuh"
#include "q4b_tile.cuh"

namespace mmqtc {

constexpr uint32_t NDW = 16;           // decode + epilogue warps
constexpr uint32_t NT = 32 * (NDW + 2); // plus one warp that issues the MMAs and one that issues the copies
constexpr uint32_t MT = 128;           // weight rows per CTA
constexpr uint32_t NB = 128;           // activation rows per pass at most (the MMA's N is two planes of them: 256)
constexpr uint32_t KS = 128;           // k per step (four groups = 16 K chunks of 8 halves)
constexpr uint32_t A_ATOM = MT * 128;  // 64 k of the CTA's weight rows: [row][128 B], 128-byte swizzle
constexpr uint32_t A_BYTES = 2 * A_ATOM;         // a step: 32 KB
// An activation atom: 64 k of the pass's rows, first plane then second plane, [plane][row][128 B]
// under the 128-byte swizzle: 2 * box * 128 bytes, box = rows per pass of the launch (16, 64 or 128).
constexpr uint32_t B_SBO = 1024;       // eight rows of 128 bytes
constexpr uint32_t NSTAGE_B = 2;
constexpr uint32_t NA = 2;             // weight-operand buffers (decode runs up to NA steps ahead of the MMAs)
constexpr uint32_t NACC = 2;           // accumulators: super-blocks in flight between MMA and epilogue
// an accumulator: the two planes' products side by side, 2 * box columns; NACC of them are allocated

struct __align__(1024) Smem {
    uint8_t a[NA][A_BYTES];
    uint16_t dr[3][MT];        // d (its fp16 bits) of the weight rows of the last three super-blocks: the
                               // decode of the fastest warp is at most two super-blocks ahead of the
                               // slowest warp's epilogue (operand buffers and their barriers bound it)
    uint32_t tabk[512];        // code bytes 2c with bit 7 flipped
    unsigned long long bar_mma[NA];    // a step's MMAs are complete (operand buffer free)
    unsigned long long a_full[NA];     // all decode warps have written a step's weights
    unsigned long long acc_empty[NACC];  // all epilogue warps have read a super-block's accumulator
    unsigned long long bar_b[NSTAGE_B];     // a step's activation planes have landed
    unsigned long long b_empty[NSTAGE_B];   // the MMAs that read a stage are complete
    uint32_t tmem_base;
    uint32_t failed;
};
// behind it: b[NSTAGE_B][2][atom], every [row][128 B] block on a 1024-byte boundary
constexpr uint32_t B_OFF = (uint32_t)((sizeof(Smem) + 1023u) & ~1023u);
__host__ __device__ constexpr uint32_t b_atom_bytes(uint32_t box) { return 2u * box * 128u; }
// What a launch asks for decides how the SM's 256 KB are split between shared memory and L1, and the
// decode warps' field loads live in L1 (a CTA reads its 110 KB of weight fields again and again).
// Measured on the prefill step: passes of up to 64 rows 1.084 ms when asking for 136 KB, 1.16 ms for
// the 131 KB they need; passes of 128 rows 1.018 ms for the 195 KB they need, 1.042 ms with 1 KB more.
__host__ __device__ constexpr uint32_t smem_bytes(uint32_t box) {
    return box > 64u ? B_OFF + NSTAGE_B * 2u * b_atom_bytes(box) : 136u * 1024u;
}
static_assert(B_OFF + NSTAGE_B * 2u * b_atom_bytes(64) <= 136u * 1024u, "shared memory layout");
static_assert(smem_bytes(NB) <= 227u * 1024u, "shared memory layout");

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
__device__ __forceinline__ void mbar_arrive(unsigned long long *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait on a phase parity.  Returns false after giving up.
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, uint32_t parity, uint32_t limit) {
    const uint32_t a = smem_u32(bar);
    for (uint32_t i = 0; i < limit; i++) {
        uint32_t ok;
        // the time hint (ns) lets the hardware park the thread instead of having it poll: the
        // MMA and copy warps wait most of the time and would otherwise take issue slots from
        // the decode warps on their schedulers
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(a), "r"(parity), "r"(2000u)
            : "memory");
        if (ok) return true;
    }
    return false;
}

// K-major rows of 128 bytes under the 128-byte swizzle (what a TMA load with that swizzle
// writes): 8-row groups 1024 bytes apart; the K offset inside the 128 bytes is part of the
// start address.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | (1ull << 16) | ((uint64_t)(B_SBO >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}
__device__ __forceinline__ uint64_t desc64(uint32_t lo, uint32_t hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
// D fp32, A and B fp16, both K-major, M = 128.
__device__ __forceinline__ uint32_t instr_desc(uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((MT >> 4) << 24);
}
// D (+)= A * B; acc = 0 overwrites the accumulator.
__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        :
        : "r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc)
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
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t *v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
          "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
          "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
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
    uint32_t pass_rows;          // activation rows per pass: 128 or 64, or 16 to spread a small call over more CTAs
    uint32_t box_rows;           // rows per activation copy = the MMA's N per plane
    uint32_t mt_per_cta;         // 128-row weight tiles one CTA walks (grid.x = tiles / this)
    const float *rs;             // per activation row: the power of two its fp16 planes were divided by
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

constexpr uint32_t WAIT_LIMIT = 1u << 19;   // tries (of up to 2 us each) before a wait gives up: about a second
constexpr uint32_t ERR_MMQ_TC = 0x400u;

// One 32-weight group as fp16 integers w * ls (w = sign * (2c + 1)), 32 halves in 16 words.
// With t = 2c (even) and m the 0x00/0xFF sign mask, y = ((t ^ 0x80) ^ m) | 1 is the byte
// w + 128 (t + 1 or ~t, bit 7 flipped).  A byte y under a high byte 0x64 is the fp16 number
// 1024 + y, and the fused (1024 + y) * ls - 1152 * ls = w * ls is exact: every operand and the
// result are integers within fp16's exact range.
template <bool TILED>
__device__ __forceinline__ void decode_group_h(const Iq3Fields &f, const uint32_t *tabk, uint32_t *hv) {
    const __half ls = __uint2half_rn(f.ls);
    const __half2 L2 = __half2half2(ls);
    const __half2 C2 = __half2half2(__hmul(ls, __float2half_rn(-1152.f)));
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const uint32_t wq = k < 4 ? f.qs_lo : f.qs_hi;
        // (a byte permute that assembles the index in one instruction made no difference here)
        const uint32_t idx = ((wq >> (8 * (k & 3))) & 0xffu) | (((f.qh >> k) & 1u) << 8);
        uint32_t m;
        if (TILED) {
            const uint32_t t = f.sg << k;
            m = q4b_prmt(t, t, 0xba98u);
        } else {
            m = q4b_sign_mask4(f.sg >> (4 * k));
        }
        const uint32_t y = (tabk[idx] ^ m) | 0x01010101u;
        const uint32_t h01 = q4b_prmt(y, 0x64646464u, 0x5140u);
        const uint32_t h23 = q4b_prmt(y, 0x64646464u, 0x7362u);
        const __half2 r01 = __hfma2(*reinterpret_cast<const __half2 *>(&h01), L2, C2);
        const __half2 r23 = __hfma2(*reinterpret_cast<const __half2 *>(&h23), L2, C2);
        hv[2 * k] = *reinterpret_cast<const uint32_t *>(&r01);
        hv[2 * k + 1] = *reinterpret_cast<const uint32_t *>(&r23);
    }
}

// A group's fields as loaded, with nothing computed from them yet: the loads are issued
// steps ahead of the decode, and arithmetic on a loaded value would wait for it on the spot.
struct RawFields {
    uint32_t qs_lo, qs_hi, qh, sg, sc, d;
};
template <bool TILED>
__device__ __forceinline__ RawFields raw_fields(const uint8_t *mat, uint64_t bi, uint32_t ib) {
    RawFields r;
    if (TILED) {
        const uint8_t *t = mat + (bi >> 3) * Q4B_TILE_BYTES;
        const uint32_t b = (uint32_t)(bi & 7u);
        const uint2 qs = *reinterpret_cast<const uint2 *>(t + Q4B_TILE_OFF_QS + 64u * b + 8u * ib);
        r.qs_lo = qs.x;
        r.qs_hi = qs.y;
        r.qh = t[Q4B_TILE_OFF_QH + 8u * b + ib];
        r.sg = *reinterpret_cast<const uint32_t *>(t + Q4B_TILE_OFF_SG + 32u * b + 4u * ib);
        r.sc = t[Q4B_TILE_OFF_SC + 4u * b + (ib >> 1)];
        r.d = *reinterpret_cast<const uint16_t *>(t + 2u * b);
    } else {   // the engine's byte order: unaligned fields are assembled (and waited for) here
        const Iq3Fields f = iq3_fields<false>(mat, bi, ib);
        r.qs_lo = f.qs_lo;
        r.qs_hi = f.qs_hi;
        r.qh = f.qh;
        r.sg = f.sg;
        r.sc = ((f.ls - 1u) >> 1) * 0x11u;
        r.d = __half_as_ushort(__float2half_rn(f.d));
    }
    return r;
}
__device__ __forceinline__ Iq3Fields cook_fields(uint32_t ib, const RawFields &r) {
    Iq3Fields f;
    f.qs_lo = r.qs_lo;
    f.qs_hi = r.qs_hi;
    f.qh = r.qh;
    f.sg = r.sg;
    f.ls = 1u + 2u * ((ib & 1u) ? (r.sc >> 4) : (r.sc & 15u));
    f.d = __half2float(__ushort_as_half((unsigned short)r.d));
    return f;
}

// A thread's 16 finished sums of one weight row: out[j] = v[j] * rs[j] for the first n columns.
// Not inlined: it runs once per tile, and inlined into the unrolled step loop its predicated
// stores were issued every step (a third more instructions).
__device__ __noinline__ void store_tile(float *o, uint64_t ld, const float *rs, uint32_t n, float4 a0, float4 a1,
                                        float4 a2, float4 a3) {
    const float v[16] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w, a2.x, a2.y, a2.z, a2.w, a3.x, a3.y, a3.z, a3.w};
#pragma unroll
    for (int j = 0; j < 16; j++)
        if ((uint32_t)j < n) o[(uint64_t)j * ld] = v[j] * __ldg(rs + j);
}

// NSL: 16-column slabs of the accumulator per epilogue thread: 1 for passes of up to 64 rows, 2 for 128
// (16 more running sums per thread: at 96 registers that spills a little, so the narrow passes keep
// their own instance).
template <bool TILED, uint32_t NSL>
__global__ void __launch_bounds__(NT, 1) mmq_tc_k(const Args a, const __grid_constant__ CUtensorMap map_h1,
                                                  const __grid_constant__ CUtensorMap map_h2) {
    // used directly (no integer round trip), so that the compiler keeps these as
    // shared-space accesses; dynamic shared memory starts on the declared alignment
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    Smem &s = *reinterpret_cast<Smem *>(smem_raw);
    if (blockIdx.y >= *a.n_work) return;
    const uint2 item = a.work[blockIdx.y];
    const uint32_t entry = item.x;
    const int32_t rc = (int32_t)item.y;                                       // this CTA's pass of the rows
    const int32_t r1 = min(a.bounds[entry + 1], rc + (int32_t)min(a.pass_rows, NB));
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t B = a.cols >> 8;                 // super-blocks per weight row
    const uint32_t n_it = a.cols / KS;              // steps (even: two per super-block)
    const uint8_t *mat = a.w + (uint64_t)(a.act ? a.act[entry] : (int32_t)entry) * a.expert_stride;
    const uint32_t n_mt = a.mt_per_cta;             // 128-row tiles of weight rows this CTA walks
    const uint32_t row0 = blockIdx.x * MT * n_mt;
    const uint32_t n_s = n_it * n_mt;               // steps over all its tiles: one pipeline
    const uint32_t nrows = (uint32_t)(r1 - rc);
    const uint32_t box = a.box_rows;                // rows a copy brings = rows per pass: 16, 64 or 128
    const uint32_t idesc = instr_desc(2u * box);
    const uint32_t b_atom = b_atom_bytes(box);
    const uint32_t acc_cols = 2u * box;             // columns of one accumulator
    const uint32_t tmem_cols = max(32u, NACC * acc_cols);   // 64, 256 or 512: a power of two
    uint8_t *const sb_base = smem_raw + B_OFF;

    if (tid < 512u) s.tabk[tid] = (__ldg(a.codes + tid) << 1) ^ 0x80808080u;
    if (tid == 0) {
        for (uint32_t i = 0; i < NA; i++) {
            mbar_init(&s.bar_mma[i], 1);
            mbar_init(&s.a_full[i], NDW);
        }
        for (uint32_t i = 0; i < NACC; i++) mbar_init(&s.acc_empty[i], NDW);
        for (uint32_t i = 0; i < NSTAGE_B; i++) {
            mbar_init(&s.bar_b[i], 1);
            mbar_init(&s.b_empty[i], 1);
        }
        s.failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&s.tmem_base)),
                     "r"(tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s.tmem_base;

    // A bounded wait that records its failure; afterwards the CTA keeps going with short waits.
    uint32_t wait_limit = WAIT_LIMIT;
    auto wait = [&](unsigned long long *bar, uint32_t parity, uint32_t code) {
        if (!mbar_wait(bar, parity, wait_limit)) {
            atomicOr(a.err, ERR_MMQ_TC | code);
            wait_limit = 1024u;
        }
    };

    if (warp == NDW) {
        // ---- the MMA warp (one lane): waits for both operands of a step, issues its MMAs, commits ----
        if (lane == 0) {
            const uint64_t a_d0 = smem_desc_sw128(smem_u32(s.a[0])), b_d0 = smem_desc_sw128(smem_u32(sb_base));
            const uint32_t a_lo0 = (uint32_t)a_d0, a_hi = (uint32_t)(a_d0 >> 32);
            const uint32_t b_lo0 = (uint32_t)b_d0, b_hi = (uint32_t)(b_d0 >> 32);
            for (uint32_t it = 0; it < n_s; it++) {   // it: step over all tiles
                const uint32_t buf = it % NA, sb = it % NSTAGE_B, sbk = it >> 1, accb = sbk % NACC;
                // the accumulator of this super-block was read out NACC super-blocks ago
                if ((it & 1u) == 0 && sbk >= NACC) wait(&s.acc_empty[accb], (sbk / NACC - 1u) & 1u, 4u);
                wait(&s.a_full[buf], (it / NA) & 1u, 8u);
                wait(&s.bar_b[sb], (it / NSTAGE_B) & 1u, 1u);
                tc_fence_after();
                // descriptors differ from step to step only in the start-address field (low word)
                const uint32_t a_lo = a_lo0 + buf * (A_BYTES >> 4), b_lo = b_lo0 + sb * ((2u * b_atom) >> 4);
                const uint32_t d_addr = tmem + accb * acc_cols;
#pragma unroll
                for (uint32_t k = 0; k < 8; k++)   // one MMA per 16 k: both planes are its N side
                    mma_f16(d_addr, desc64(a_lo + (k >> 2) * (A_ATOM >> 4) + (k & 3u) * 2u, a_hi),
                            desc64(b_lo + (k >> 2) * (b_atom >> 4) + (k & 3u) * 2u, b_hi), idesc,
                            k ? 1u : (it & 1u));
                mma_commit(&s.bar_mma[buf]);
                mma_commit(&s.b_empty[sb]);
            }
        }
    } else if (warp == NDW + 1u) {
        // ---- the copy warp (one lane): both activation planes of a step by TMA, NSTAGE_B - 1 ahead ----
        if (lane == 0) {
            uint32_t it = 0;   // step within the tile: every tile reads the same rows again
            for (uint32_t st = 0; st < n_s; st++, it = it + 1u == n_it ? 0u : it + 1u) {
                // the stage was last read by step st - NSTAGE_B
                const uint32_t sb = st % NSTAGE_B;
                if (st >= NSTAGE_B) wait(&s.b_empty[sb], (st / NSTAGE_B - 1u) & 1u, 16u);
                mbar_expect_tx(&s.bar_b[sb], 4u * box * 128u);
#pragma unroll
                for (uint32_t at = 0; at < 2; at++) {
                    uint8_t *dstb = sb_base + (sb * 2u + at) * b_atom;
                    tma_load_2d(dstb, &map_h1, &s.bar_b[sb], (int)(it * KS + at * 64u), rc);
                    tma_load_2d(dstb + box * 128u, &map_h2, &s.bar_b[sb], (int)(it * KS + at * 64u), rc);
                }
            }
        }
    } else {
        // ---- the 16 decode + epilogue warps ----
        // decode: a warp takes eight weight rows (one 8-row group of core matrices) x the step's
        // four groups; lanes 8g..8g+7 hold group g, so a quarter warp's 16-byte stores of one K
        // chunk are 128 contiguous bytes, and the warp's loads still cover 8 rows x 4 adjacent groups
        const uint32_t d_row = (warp << 3) | (lane & 7u), d_g = lane >> 3;
        const uint32_t d_blk0 = (row0 + d_row) * B;   // in tile m: + m * MT * B (a matrix has < 2^32 blocks)
        // swizzled position of 16-byte chunk j (0..3) of this thread's group: atom d_g / 2, row d_row,
        // chunk (4 (d_g & 1) + j) ^ (row & 7)
        const uint32_t d_base = (d_g >> 1) * A_ATOM + d_row * 128u;
        const uint32_t d_c0 = 4u * (d_g & 1u), d_x = lane & 7u;
        // epilogue: tensor-memory lanes of this warp's quadrant; of the pass's columns (activation
        // rows) the 16-column slabs e_cs and, in a pass of more than 64 rows, e_cs + 4
        const uint32_t e_q = warp & 3u, e_cs = warp >> 2;
        const uint32_t e_row = 32u * e_q + lane;
        const uint32_t e_taddr = tmem + ((32u * e_q) << 16) + 16u * e_cs;
        bool e_live[NSL];
        float acc[NSL][16];
#pragma unroll
        for (uint32_t h = 0; h < NSL; h++) {
            e_live[h] = 16u * (e_cs + 4u * h) < nrows;
#pragma unroll
            for (int j = 0; j < 16; j++) acc[h][j] = 0.f;
        }

        // steps are fetched in order: (tile, step in tile) advance by counters, not divisions
        uint32_t pf_it = 0;
        uint32_t pf_blk = d_blk0;   // first block of this thread's row in the tile being fetched
        auto load_next_fields = [&]() {
            const RawFields r = raw_fields<TILED>(mat, (uint64_t)(pf_blk + (pf_it >> 1)), (pf_it & 1u) * 4u + d_g);
            if (++pf_it == n_it) {
                pf_it = 0;
                pf_blk += MT * B;
            }
            return r;
        };
        uint32_t rt_it = 0, rt_m = 0;   // (step in tile, tile) of the next step to retire
        // step `done` has completed: its operand buffer is free; with an odd step the super-block's
        // accumulator is complete and is folded into the running sums
        auto retire = [&](uint32_t done) {
            wait(&s.bar_mma[done % NA], (done / NA) & 1u, 2u);
            if (done & 1u) {
                const uint32_t sbk = done >> 1;
                tc_fence_after();
#pragma unroll
                for (uint32_t h = 0; h < NSL; h++) {
                    if (e_live[h]) {   // warp-uniform
                        const float dr = __half2float(__ushort_as_half(s.dr[sbk % 3u][e_row]));
                        uint32_t v[16], v2[16];
                        tmem_ld16(e_taddr + (sbk % NACC) * acc_cols + 64u * h, v);
                        tmem_ld16(e_taddr + (sbk % NACC) * acc_cols + 64u * h + box, v2);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; j++)
                            acc[h][j] = fmaf(dr, __uint_as_float(v[j]) + __uint_as_float(v2[j]), acc[h][j]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&s.acc_empty[sbk % NACC]);
                if (rt_it + 1u == n_it) {   // the tile's last super-block: write its rows out
#pragma unroll
                    for (uint32_t h = 0; h < NSL; h++) {
                        const uint32_t cs = e_cs + 4u * h;
                        if (e_live[h])
                            store_tile(a.dst + (uint64_t)(rc + 16 * (int32_t)cs) * a.ld_dst + row0 + rt_m * MT + e_row,
                                       a.ld_dst, a.rs + rc + 16 * (int32_t)cs, min(16u, nrows - 16u * cs),
                                       make_float4(acc[h][0], acc[h][1], acc[h][2], acc[h][3]),
                                       make_float4(acc[h][4], acc[h][5], acc[h][6], acc[h][7]),
                                       make_float4(acc[h][8], acc[h][9], acc[h][10], acc[h][11]),
                                       make_float4(acc[h][12], acc[h][13], acc[h][14], acc[h][15]));
#pragma unroll
                        for (int j = 0; j < 16; j++) acc[h][j] = 0.f;
                    }
                }
            }
            if (++rt_it == n_it) {
                rt_it = 0;
                rt_m++;
            }
        };
        // The fields of a step are fetched PF steps before they are decoded, into a slot that is
        // never moved (the loop is unrolled by PF): a register move would wait for its load.
        // (measured: 2 steps ahead 1.15 ms per prefill step, 3 ahead 1.17 - an odd unroll makes the step's
        // parity a run-time value in every stage -, 4 ahead spills)
        constexpr uint32_t PF = 2;
        RawFields fq[PF];
#pragma unroll
        for (uint32_t u = 0; u < PF; u++)
            if (u < n_s) fq[u] = load_next_fields();
            else fq[u] = fq[0];
        for (uint32_t it0 = 0; it0 < n_s; it0 += PF) {
#pragma unroll
            for (uint32_t u = 0; u < PF; u++) {
                const uint32_t it = it0 + u;   // step over all tiles; steps per tile are even
                if (it >= n_s) break;
                if (it >= NA) retire(it - NA);
                {
                    uint32_t hv[16];
                    const Iq3Fields f = cook_fields((it & 1u) * 4u + d_g, fq[u]);
                    decode_group_h<TILED>(f, s.tabk, hv);
                    uint8_t *p = s.a[it % NA] + d_base;
#pragma unroll
                    for (uint32_t c = 0; c < 4; c++)
                        *reinterpret_cast<uint4 *>(p + (((d_c0 + c) ^ d_x) << 4)) =
                            make_uint4(hv[4 * c], hv[4 * c + 1], hv[4 * c + 2], hv[4 * c + 3]);
                    if (d_g == 0 && (it & 1u) == 0) s.dr[(it >> 1) % 3u][d_row] = (uint16_t)fq[u].d;
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&s.a_full[it % NA]);
                if (it + PF < n_s) fq[u] = load_next_fields();
            }
        }
        for (uint32_t t = n_s > NA ? n_s - NA : 0u; t < n_s; t++) retire(t);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols)
                     : "memory");
    }
}

// The fp16 planes of the quantised activation rows: x = q * dq (the value the 8-bit row stands
// for), divided by the power of two rs that brings the row's largest magnitude below 1, as
// h1 = fp16(x / rs) and h2 = fp16(x / rs - h1).  A row is taken by tpr = min(256, cols / 8)
// threads, eight values each per turn; a CTA of 256 threads holds 256 / tpr rows.
__global__ void __launch_bounds__(256) planes_k(const int8_t *__restrict__ q, const float *__restrict__ dq,
                                                uint64_t rows, uint32_t cols, uint32_t tpr,
                                                __half *__restrict__ h1, __half *__restrict__ h2,
                                                float *__restrict__ rs) {
    __shared__ float red[8];
    const uint32_t tid = threadIdx.x, rpb = 256u / tpr, sub = tid / tpr, t = tid - sub * tpr;
    const uint64_t row = (uint64_t)blockIdx.x * rpb + sub;
    const bool live = sub < rpb && row < rows;   // 256 % tpr threads at the end of the CTA have no row
    const uint32_t gpr = cols >> 5;
    const float *d = dq + (live ? row : 0) * gpr;
    float m = 0.f;
    if (live)
        for (uint32_t c = t * 8u; c < cols; c += tpr * 8u) m = fmaxf(m, d[c >> 5]);   // every group is seen
    m = q4b_warp_max(m);
    if ((tid & 31u) == 0) red[tid >> 5] = m;
    __syncthreads();
    if (!live) return;
    const uint32_t w0 = sub * (tpr >> 5), w1 = w0 + (tpr >> 5);   // the row's warps (tpr is a multiple of 32)
    m = red[w0];
    for (uint32_t i = w0 + 1u; i < w1; i++) m = fmaxf(m, red[i]);
    int e = 0;
    if (m > 0.f) (void)frexpf(m * 127.f, &e);   // 127 dq = the group's largest magnitude
    const float inv = ldexpf(1.f, -e);
    if (t == 0) rs[row] = ldexpf(1.f, e);
    const int8_t *qr = q + row * cols;
    __half *o1 = h1 + row * cols, *o2 = h2 + row * cols;
    for (uint32_t c = t * 8u; c < cols; c += tpr * 8u) {   // eight values per thread and turn
        const uint2 w = *reinterpret_cast<const uint2 *>(qr + c);
        const float sc = d[c >> 5] * inv;
        uint32_t p1[4], p2[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t word = i < 2 ? w.x : w.y;
            const int qa = (int)(int8_t)(word >> (16 * (i & 1))), qb = (int)(int8_t)(word >> (16 * (i & 1) + 8));
            const float xa = (float)qa * sc, xb = (float)qb * sc;
            const __half2 a1 = __floats2half2_rn(xa, xb);
            const float2 back = __half22float2(a1);
            const __half2 a2 = __floats2half2_rn(xa - back.x, xb - back.y);
            p1[i] = *reinterpret_cast<const uint32_t *>(&a1);
            p2[i] = *reinterpret_cast<const uint32_t *>(&a2);
        }
        *reinterpret_cast<uint4 *>(o1 + c) = make_uint4(p1[0], p1[1], p1[2], p1[3]);
        *reinterpret_cast<uint4 *>(o2 + c) = make_uint4(p2[0], p2[1], p2[2], p2[3]);
    }
}


// ---- host side ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;
static bool g_ready = false, g_tried = false;
constexpr uint32_t WORK_CAP = 1u << 16;   // passes per launch: entries + rows / (rows per pass) must fit
#ifndef Q4B_PASS128_MIN_ROWS
#define Q4B_PASS128_MIN_ROWS 8192
#endif
constexpr uint64_t PASS128_MIN_ROWS = Q4B_PASS128_MIN_ROWS;   // calls with at least this many rows take 128 of them per pass
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
    if (cudaFuncSetAttribute(mmq_tc_k<true, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(64)) !=
            cudaSuccess ||
        cudaFuncSetAttribute(mmq_tc_k<false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(64)) !=
            cudaSuccess ||
        cudaFuncSetAttribute(mmq_tc_k<true, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(NB)) !=
            cudaSuccess ||
        cudaFuncSetAttribute(mmq_tc_k<false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(NB)) !=
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

// q: int8 [rows][cols] row-major; dq: float [rows][cols/32]; h1, h2: fp16 [rows][cols] and
// rs: float [rows], scratch this call fills (planes_k) before the product reads it.
bool launch(const uint8_t *w, uint64_t expert_stride, const int32_t *act, const uint32_t *n_act,
            uint32_t n_entries, const int32_t *bounds, const int8_t *q, const float *dq, __half *h1,
            __half *h2, float *rs, uint64_t rows, uint32_t cols, uint32_t w_rows, float *dst,
            uint64_t ld_dst, bool tiled, uint32_t min_rows, cudaStream_t stream) {
    if (!g_ready || !shape_ok(w_rows, cols) || rows == 0 || rows > 0x7fffffffull) return false;
    // a small call (decode batches: a handful of entries reach the threshold) is cut into
    // passes of 16 rows so that its few entries still spread over many SMs
    // a large one in passes of 128 rows: an expert's weights are decoded once per pass, and with a
    // skewed routing most rows belong to experts with hundreds of them
    const uint32_t pass_rows = rows <= 2048u ? 16u : rows < PASS128_MIN_ROWS ? 64u : NB;
    const uint64_t max_items = (uint64_t)n_entries + rows / pass_rows;
    if (max_items > WORK_CAP || max_items > 65535u) return false;   // the pass index is gridDim.y
    CUtensorMap maps[2];
    for (int pl = 0; pl < 2; pl++) {
        // rows of fp16; a box is 64 k (128 bytes) of NB rows, stored with the 128-byte swizzle
        const cuuint64_t dims[2] = {cols, rows};
        const cuuint64_t strides[1] = {(cuuint64_t)cols * 2u};
        const cuuint32_t box[2] = {64, pass_rows < NB ? pass_rows : NB};
        const cuuint32_t es[2] = {1, 1};
        if (g_encode(&maps[pl], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)(pl ? h2 : h1), dims, strides, box, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
    }
    {
        const uint32_t tpr = cols / 8u < 256u ? cols / 8u : 256u;   // cols % 256 == 0: a multiple of 32
        const uint32_t rpb = 256u / tpr;
        planes_k<<<(unsigned)((rows + rpb - 1) / rpb), 256, 0, stream>>>(q, dq, rows, cols, tpr, h1, h2, rs);
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
    a.rs = rs;
    a.box_rows = pass_rows < NB ? pass_rows : NB;
    worklist_k<<<1, 1024, 0, stream>>>(bounds, n_act, n_entries, min_rows, g_work + turn * WORK_CAP,
                                            g_n_work + turn, WORK_CAP, pass_rows);
    // a CTA walks enough 128-row tiles of its pass for about 16 steps: start-up (work item,
    // table, pipeline fill) is then paid once per 16 steps also where a tile has few (K = 512: 4)
    const uint32_t n_tiles = w_rows / MT, n_it = cols / KS;
    uint32_t mt = 1;
    for (uint32_t c = 1; c <= n_tiles && c * n_it <= 16u; c++)
        if (n_tiles % c == 0) mt = c;
    a.mt_per_cta = mt;
    const dim3 grid(n_tiles / mt, (unsigned)max_items);
    const uint32_t smem = smem_bytes(a.box_rows);
    if (a.box_rows > 64u) {
        if (tiled)
            mmq_tc_k<true, 2><<<grid, NT, smem, stream>>>(a, maps[0], maps[1]);
        else
            mmq_tc_k<false, 2><<<grid, NT, smem, stream>>>(a, maps[0], maps[1]);
    } else {
        if (tiled)
            mmq_tc_k<true, 1><<<grid, NT, smem, stream>>>(a, maps[0], maps[1]);
        else
            mmq_tc_k<false, 1><<<grid, NT, smem, stream>>>(a, maps[0], maps[1]);
    }
    return true;
}

}  // namespace mmqtc
