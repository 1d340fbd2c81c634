// Grouped IQ3_S x int8 product for FEW activation rows per expert (batched decode,
// verify windows, expert-parallel shards): a persistent kernel, one CTA per SM, that
// streams every live expert's weight tiles HBM -> shared memory exactly once with
// 1-D bulk async copies and keeps the activation bytes a lane needs in registers.
//
// Same arithmetic and entry points as grouped_rows_k (q4b_grouped.cu), which stays
// the general form; this kernel needs the tiled arena format and 1, 2, 4 or 8
// super-blocks per weight row.
//
// Work: the live entries (those with rows) times the matrix's chunks of 64 tiles
// (56,320 contiguous bytes; the last chunk of a matrix may be shorter).  CTAs split
// that list by estimated cost into contiguous shares, so a CTA stays on one expert
// for many chunks.  One lane keeps two chunks in flight (full/empty mbarriers); each
// of the 16 warps takes four tiles of a chunk, one after the other: lane l decodes
// block l/4, groups 2(l%4) and 2(l%4)+1 into registers and dots the decoded codes
// with the expert's activation rows; after its last tile's fields are read the warp
// releases the stage.  The first three rows' bytes for exactly those 64 columns stay
// in registers from tile to tile (they change only when the CTA moves to the next
// expert); further rows come from L1/L2 per tile.
// The kernel is bound by instruction issue, so what is paid per loop trip counts:
// measured on 48 layers of 64 tokens (ms): one tile per trip with row guards 18.6;
// straight-line code per row count 16.8; two tiles per trip (5 chunks in flight)
// 16.0, three (3) 15.4, four (2) 14.8, five (2) 15.5.
// 16 warps x 128 registers: measured faster than more warps with fewer registers
// (a few spilled registers cost more here than the lost occupancy) and than 12 warps
// with 162 registers and no spills (15.4 against 14.7 ms).
#include "q4b_tile.cuh"

namespace few {

constexpr uint32_t NCW = 16;                 // warps
// Two shapes of the ring, picked per call by the amount of work (see launch()): <TPW, NSTAGE> = tiles a
// warp takes from a chunk (loop and ring tests are paid once for all of them) and chunks in flight.
constexpr uint32_t NT = NCW * 32;
constexpr uint32_t RB = 3;                   // activation rows held in registers (2: 14 % slower, 4 spills)
constexpr uint32_t MAX_ENTRIES = 1024;
constexpr uint32_t WAIT_LIMIT = 1u << 21;    // tries before a wait gives up ...
constexpr unsigned long long WAIT_NS = 500000000ull;   // ... or half a second, whichever comes first
constexpr uint32_t ERR_FEW = 0x800u;

template <uint32_t TPW, uint32_t NSTAGE> struct Smem {
    uint32_t tab[32 * 512];                  // code table, one column per lane
    uint8_t stage[NSTAGE][NCW * TPW * Q4B_TILE_BYTES];
    unsigned long long full[NSTAGE], empty[NSTAGE];
    uint32_t live[MAX_ENTRIES];              // compacted live entries
    uint32_t cost[MAX_ENTRIES + 1];          // cost of all chunks before entry i (prefix)
    uint32_t wcount[32];
    uint32_t n_live;
};
template <uint32_t TPW, uint32_t NSTAGE> constexpr uint32_t smem_bytes() { return sizeof(Smem<TPW, NSTAGE>) + 128; }

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
// Bounded in time: `limit` tries, and every 1024 tries a look at the clock (a try parks the thread
// for a hardware-chosen time; giving it a time hint made it wake late: 14.8 -> 22.9 ms on 48 layers
// of 64 tokens).  limit < 2048 (after an earlier give-up) skips the clock.
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, uint32_t parity, uint32_t limit,
                                          uint32_t *err) {
    const uint32_t a = smem_u32(bar);
    unsigned long long t0 = 0;
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
        if ((i & 1023u) == 1023u) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
            if (t0 == 0) t0 = t;
            else if (t - t0 > WAIT_NS) break;
        }
    }
    atomicOr(err, ERR_FEW);
    return false;
}

struct Args {
    const uint8_t *w;
    uint64_t expert_stride;
    const int32_t *act;
    const uint32_t *n_act;
    uint32_t n_entries;
    const int32_t *bounds;
    const int8_t *xq;
    const float *xd;
    const int32_t *xbs;
    uint32_t cols, w_rows;
    float *dst;
    uint64_t ld_dst;
    const uint32_t *codes;
    uint32_t *err;
    uint32_t max_rows;   // entries with more rows than this are left to the tensor-core kernel
};

// Relative cost of one chunk of an entry with `rows` activation rows: the decode, the
// row dots, and from five rows on the re-fetch of the rows' bytes for every tile.
__device__ __forceinline__ uint32_t chunk_cost(uint32_t rows) {
    return 6u + 2u * rows + (rows > RB ? rows : 0u);
}

// BB = super-blocks per weight row (1, 2, 4 or 8), a template parameter so that the row
// geometry and the depth of the shuffle sum are compile-time constants.
template <uint32_t BB, uint32_t TPW, uint32_t NSTAGE>
__global__ void __launch_bounds__(NT, 1) grouped_few_k(const Args a) {
    constexpr uint32_t CT = NCW * TPW;           // tiles per chunk
    constexpr uint32_t CHUNK_BYTES = CT * Q4B_TILE_BYTES;
    // used directly (no integer round trip), so that the compiler keeps these as
    // shared-space accesses; dynamic shared memory starts on the declared alignment
    extern __shared__ __align__(128) uint8_t smem_raw[];
    Smem<TPW, NSTAGE> &s = *reinterpret_cast<Smem<TPW, NSTAGE> *>(smem_raw);
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t n_ent = a.n_act ? min(*a.n_act, a.n_entries) : a.n_entries;

    // code table, replicated per lane: entry i for lane l at tab[32 i + l]
    for (uint32_t i = tid; i < 32u * 512u; i += NT) s.tab[i] = __ldg(a.codes + (i >> 5));
    if (tid == 0) {
        for (uint32_t i = 0; i < NSTAGE; i++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&s.full[i])), "r"(1u));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&s.empty[i])),
                         "r"(NCW));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // live entries, in order: ballot per warp, then a prefix over the warps
    uint32_t base_live = 0;
    for (uint32_t e0 = 0; e0 < n_ent; e0 += NT) {
        const uint32_t e = e0 + tid;
        const int32_t nr = e < n_ent ? a.bounds[e + 1] - a.bounds[e] : 0;
        const bool lv = nr > 0 && (uint32_t)nr <= a.max_rows;
        const uint32_t bal = __ballot_sync(0xffffffffu, lv);
        if (lane == 0) s.wcount[warp] = __popc(bal);
        __syncthreads();
        uint32_t off = base_live, tot = 0;
        for (uint32_t wv = 0; wv < NT / 32u; wv++) {
            if (wv < warp) off += s.wcount[wv];
            tot += s.wcount[wv];
        }
        if (lv) {
            const uint32_t pos = off + __popc(bal & ((1u << lane) - 1u));
            if (pos < MAX_ENTRIES) s.live[pos] = e;
        }
        base_live += tot;
        __syncthreads();
    }
    if (tid == 0) s.n_live = min(base_live, MAX_ENTRIES);
    __syncthreads();
    const uint32_t n_live = s.n_live;
    if (n_live == 0) return;
    constexpr uint32_t B = BB;
    const uint32_t n_tiles = (a.w_rows * B) >> 3;
    const uint32_t cpe = (n_tiles + CT - 1u) / CT;             // chunks per entry (the last may be short)
    // split by cost, not by chunk count: entries differ in rows
    {
        uint32_t v[2];
#pragma unroll
        for (uint32_t h = 0; h < 2; h++) {
            const uint32_t i = 2u * tid + h;
            v[h] = 0;
            if (i < n_live) {
                const uint32_t e = s.live[i];
                v[h] = cpe * chunk_cost((uint32_t)(a.bounds[e + 1] - a.bounds[e]));
            }
        }
        const uint32_t sum = v[0] + v[1];
        uint32_t inc = sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= (uint32_t)o) inc += t;
        }
        if (lane == 31u) s.wcount[warp] = inc;
        __syncthreads();
        uint32_t off = 0;
        for (uint32_t wv = 0; wv < warp; wv++) off += s.wcount[wv];
        const uint32_t excl = off + inc - sum;
        if (2u * tid <= n_live) s.cost[2u * tid] = excl;
        if (2u * tid + 1u <= n_live) s.cost[2u * tid + 1u] = excl + v[0];
    }
    __syncthreads();
    auto chunk_at = [&](uint64_t target) -> uint32_t {   // first chunk whose start cost >= target
        uint32_t lo = 0, hi = n_live;                    // entry with cost[lo] <= target < cost[lo+1]
        if (target >= s.cost[n_live]) return n_live * cpe;
        while (hi - lo > 1u) {
            const uint32_t mid = (lo + hi) >> 1;
            if (s.cost[mid] <= target) lo = mid; else hi = mid;
        }
        const uint32_t per = (s.cost[lo + 1] - s.cost[lo]) / cpe;
        const uint32_t within = (uint32_t)((target - s.cost[lo] + per - 1u) / per);
        return lo * cpe + min(within, cpe);
    };
    const uint64_t total_cost = s.cost[n_live];
    const uint32_t c_lo = chunk_at(total_cost * blockIdx.x / gridDim.x);
    const uint32_t c_hi = blockIdx.x + 1u == gridDim.x ? n_live * cpe
                                                        : chunk_at(total_cost * (blockIdx.x + 1ull) / gridDim.x);
    if (c_lo >= c_hi) return;

    // ---- producer duty: lane 0 of warp 0 keeps the ring NSTAGE - 1 chunks ahead ----
    auto produce = [&](uint32_t k) {
        const uint32_t c = c_lo + k;
        if (c >= c_hi) return;
        const uint32_t st = k % NSTAGE;
        if (k >= NSTAGE && !mbar_wait(&s.empty[st], ((k / NSTAGE) - 1u) & 1u, WAIT_LIMIT, a.err))
            return;  // not issued: the consumers' wait for this stage runs out in turn
        const uint32_t li = c / cpe, ch = c - li * cpe;
        const uint32_t e = s.live[li];
        const uint8_t *src = a.w + (uint64_t)(a.act ? a.act[e] : (int32_t)e) * a.expert_stride +
                             (uint64_t)ch * CHUNK_BYTES;
        const uint32_t bytes = min(CT, n_tiles - ch * CT) * Q4B_TILE_BYTES;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&s.full[st])),
                     "r"(bytes)
                     : "memory");
        asm volatile(
            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                smem_u32(s.stage[st])),
            "l"(src), "r"(bytes), "r"(smem_u32(&s.full[st]))
            : "memory");
    };
    if (tid == 0)
        for (uint32_t k = 0; k + 1u < NSTAGE; k++) produce(k);

    // ---- consumers ----
    const uint32_t *tab = s.tab + lane;
    const uint32_t p = lane & 3u, blk = lane >> 2;
    constexpr uint32_t lanes_per_row = 4u * B;
    const uint32_t brow = blk & (B - 1u);                // block within the weight row
    const uint32_t gcol = brow * 8u + 2u * p;            // first of the lane's two 32-groups
    const uint32_t ngr = a.cols >> 5;
    constexpr uint32_t rows_per_tile = 8u / B;
    int q[RB][16];
    float dx[RB][2];
    int bs[RB][2];
    float *orow[RB];               // the rows' places in dst
    uint32_t have_e = 0xffffffffu;
    int32_t r0 = 0, r1 = 0;
    uint32_t nr = 0;               // rows held in registers: min(r1 - r0, RB)
    uint32_t limit = WAIT_LIMIT;   // after a wait gave up the rest run through with short waits
    uint32_t li = c_lo / cpe, ch = c_lo - li * cpe, st = 0, ph = 0;
    // sum over the lanes of a weight row, then one lane stores
    auto finish = [&](float v, float *o) {
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        if (B >= 2) v += __shfl_xor_sync(0xffffffffu, v, 4);
        if (B >= 4) v += __shfl_xor_sync(0xffffffffu, v, 8);
        if (B >= 8) v += __shfl_xor_sync(0xffffffffu, v, 16);
        if ((lane & (lanes_per_row - 1u)) == 0) *o = v;
    };
    for (uint32_t c = c_lo, k = 0; c < c_hi; c++, k++) {
        if (tid == 0) produce(k + NSTAGE - 1u);
        __syncwarp();
        const uint32_t e = s.live[li];
        if (e != have_e) {   // next expert: its first RB rows' bytes for this lane's 64 columns
            have_e = e;
            r0 = a.bounds[e];
            r1 = a.bounds[e + 1];
            nr = min((uint32_t)(r1 - r0), RB);
#pragma unroll
            for (uint32_t i = 0; i < RB; i++) {
                if (i < nr) {
                    const uint64_t r = (uint64_t)(r0 + (int32_t)i);
                    const int4 *qp = reinterpret_cast<const int4 *>(a.xq + r * a.cols + gcol * 32u);
                    const int4 v0 = __ldg(qp), v1 = __ldg(qp + 1), v2 = __ldg(qp + 2), v3 = __ldg(qp + 3);
                    q[i][0] = v0.x, q[i][1] = v0.y, q[i][2] = v0.z, q[i][3] = v0.w;
                    q[i][4] = v1.x, q[i][5] = v1.y, q[i][6] = v1.z, q[i][7] = v1.w;
                    q[i][8] = v2.x, q[i][9] = v2.y, q[i][10] = v2.z, q[i][11] = v2.w;
                    q[i][12] = v3.x, q[i][13] = v3.y, q[i][14] = v3.z, q[i][15] = v3.w;
                    const float2 dv = __ldg(reinterpret_cast<const float2 *>(a.xd + r * ngr + gcol));
                    const int2 bv = __ldg(reinterpret_cast<const int2 *>(a.xbs + r * ngr + gcol));
                    dx[i][0] = dv.x, dx[i][1] = dv.y;
                    bs[i][0] = bv.x, bs[i][1] = bv.y;
                    orow[i] = a.dst + r * a.ld_dst;
                }
            }
        }
        if (!mbar_wait(&s.full[st], ph, limit, a.err)) limit = 1024u;
#pragma unroll 1   // one copy of the body: unrolled it was 1 % slower (four times the code to fetch)
        for (uint32_t sub = 0; sub < TPW; sub++) {
            // decode this warp's tile into registers; after the last one, give the stage back
            const uint32_t tc = sub * NCW + warp;                      // tile within the chunk
            const uint8_t *tile = s.stage[st] + tc * Q4B_TILE_BYTES;
            const uint4 qs = *reinterpret_cast<const uint4 *>(tile + Q4B_TILE_OFF_QS + 16u * lane);
            const uint2 sg = *reinterpret_cast<const uint2 *>(tile + Q4B_TILE_OFF_SG + 8u * lane);
            const uint32_t qh = *reinterpret_cast<const uint16_t *>(tile + Q4B_TILE_OFF_QH + 2u * lane);
            const uint32_t sc = tile[Q4B_TILE_OFF_SC + lane];
            const float d = __half2float(*reinterpret_cast<const __half *>(tile + 2u * blk));
            if (sub + 1u == TPW) {
                __syncwarp();
                if (lane == 0)
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&s.empty[st])) : "memory");
            }
            uint32_t cw[16];
            {
                const uint32_t h0 = ((qh & 0xfu) * 0x00204081u) & 0x01010101u;
                const uint32_t h1 = (((qh >> 4) & 0xfu) * 0x00204081u) & 0x01010101u;
                const uint32_t h2 = (((qh >> 8) & 0xfu) * 0x00204081u) & 0x01010101u;
                const uint32_t h3 = ((qh >> 12) * 0x00204081u) & 0x01010101u;
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const uint32_t wq = j < 4 ? qs.x : j < 8 ? qs.y : j < 12 ? qs.z : qs.w;
                    const uint32_t hh = j < 4 ? h0 : j < 8 ? h1 : j < 12 ? h2 : h3;
                    const uint32_t b = (uint32_t)j & 3u;
                    const uint32_t sel = b | ((4u + b) << 4) | ((12u + b) << 8) | ((12u + b) << 12);
                    const uint32_t idx = q4b_prmt(wq, hh, sel);
                    const uint32_t t = (j < 8 ? sg.x : sg.y) << (j & 7);
                    cw[j] = tab[idx * 32u] ^ q4b_prmt(t, t, 0xba98u);
                }
            }
            const int ls0 = (int)(2u * (sc & 15u) + 1u), ls1 = (int)(2u * (sc >> 4) + 1u);
            const uint32_t ti = ch * CT + tc;                          // tile within the matrix
            const uint32_t wrow = ti * rows_per_tile + blk / B;        // this lane's weight row
            if (ti < n_tiles) {                                        // a short last chunk leaves warps idle
                // one row held in registers: same expression as grouped_rows_k
                auto row_reg = [&](uint32_t i) {
                    int a0 = 0, a1 = 0;
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        a0 = __dp4a((int)cw[j], q[i][j], a0);
                        a1 = __dp4a((int)cw[8 + j], q[i][8 + j], a1);
                    }
                    // sum sign*(2c+1)*q = 2 sum c'q + sum q
                    const int I0 = 2 * a0 + bs[i][0], I1 = 2 * a1 + bs[i][1];
                    finish(d * ((float)(I0 * ls0) * dx[i][0] + (float)(I1 * ls1) * dx[i][1]), orow[i] + wrow);
                };
                // straight-line code per row count: no per-row guards
                row_reg(0);
                if (nr >= 2u) {
                    row_reg(1);
                    if constexpr (RB >= 3) {
                        if (nr == 3u) row_reg(2);
                    }
                }
                for (int32_t r = r0 + (int32_t)RB; r < r1; r++) {      // further rows: straight from memory
                    const int4 *qp = reinterpret_cast<const int4 *>(a.xq + (uint64_t)r * a.cols + gcol * 32u);
                    int a0 = 0, a1 = 0;
                    {
                        const int4 v0 = __ldg(qp), v1 = __ldg(qp + 1);
                        a0 = __dp4a((int)cw[0], v0.x, a0), a0 = __dp4a((int)cw[1], v0.y, a0);
                        a0 = __dp4a((int)cw[2], v0.z, a0), a0 = __dp4a((int)cw[3], v0.w, a0);
                        a0 = __dp4a((int)cw[4], v1.x, a0), a0 = __dp4a((int)cw[5], v1.y, a0);
                        a0 = __dp4a((int)cw[6], v1.z, a0), a0 = __dp4a((int)cw[7], v1.w, a0);
                    }
                    {
                        const int4 v2 = __ldg(qp + 2), v3 = __ldg(qp + 3);
                        a1 = __dp4a((int)cw[8], v2.x, a1), a1 = __dp4a((int)cw[9], v2.y, a1);
                        a1 = __dp4a((int)cw[10], v2.z, a1), a1 = __dp4a((int)cw[11], v2.w, a1);
                        a1 = __dp4a((int)cw[12], v3.x, a1), a1 = __dp4a((int)cw[13], v3.y, a1);
                        a1 = __dp4a((int)cw[14], v3.z, a1), a1 = __dp4a((int)cw[15], v3.w, a1);
                    }
                    const float2 dv = __ldg(reinterpret_cast<const float2 *>(a.xd + (uint64_t)r * ngr + gcol));
                    const int2 bv = __ldg(reinterpret_cast<const int2 *>(a.xbs + (uint64_t)r * ngr + gcol));
                    const int I0 = 2 * a0 + bv.x, I1 = 2 * a1 + bv.y;
                    finish(d * ((float)(I0 * ls0) * dv.x + (float)(I1 * ls1) * dv.y),
                           a.dst + (uint64_t)r * a.ld_dst + wrow);
                }
            }
        }
        if (++ch == cpe) ch = 0, li++;
        if (++st == NSTAGE) st = 0, ph ^= 1u;
    }
}

static bool g_ready = false;
template <uint32_t TPW, uint32_t NSTAGE> static bool warm_shape() {
    const int bytes = (int)smem_bytes<TPW, NSTAGE>();
    return cudaFuncSetAttribute(grouped_few_k<1, TPW, NSTAGE>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) ==
               cudaSuccess &&
           cudaFuncSetAttribute(grouped_few_k<2, TPW, NSTAGE>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) ==
               cudaSuccess &&
           cudaFuncSetAttribute(grouped_few_k<4, TPW, NSTAGE>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) ==
               cudaSuccess &&
           cudaFuncSetAttribute(grouped_few_k<8, TPW, NSTAGE>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) ==
               cudaSuccess;
}
bool warm() {
    if (!warm_shape<4, 2>() || !warm_shape<2, 4>()) {
        cudaGetLastError();
        return false;
    }
    g_ready = true;
    return true;
}

bool shape_ok(uint64_t w_rows, uint64_t w_cols, uint32_t n_entries) {
    if (!g_ready || w_cols == 0 || (w_cols % 256u) || n_entries > MAX_ENTRIES) return false;
    const uint64_t B = w_cols / 256u;
    if (!(B == 1 || B == 2 || B == 4 || B == 8)) return false;
    const uint64_t blocks = w_rows * B;
    return blocks != 0 && (blocks % 8u) == 0;
}

template <uint32_t TPW, uint32_t NSTAGE> static bool launch_shape(const Args &a) {
    const size_t sm = smem_bytes<TPW, NSTAGE>();
    switch (a.cols >> 8) {
    case 1: grouped_few_k<1, TPW, NSTAGE><<<g_q4b.n_sm, NT, sm, g_q4b.stream>>>(a); break;
    case 2: grouped_few_k<2, TPW, NSTAGE><<<g_q4b.n_sm, NT, sm, g_q4b.stream>>>(a); break;
    case 4: grouped_few_k<4, TPW, NSTAGE><<<g_q4b.n_sm, NT, sm, g_q4b.stream>>>(a); break;
    case 8: grouped_few_k<8, TPW, NSTAGE><<<g_q4b.n_sm, NT, sm, g_q4b.stream>>>(a); break;
    default: return false;
    }
    return true;
}
// Large chunks pay the loop and ring tests once per four tiles, but a CTA wants a few dozen of them to
// fill its pipeline and to balance against the others: with little work (an expert-parallel rank's 64
// experts, a verify window's 40) the smaller chunks win.  The entry count is the caller's upper bound
// on the live entries.
bool launch(const Args &a) {
    const uint64_t tiles = ((uint64_t)a.w_rows * (a.cols >> 8)) >> 3;
    const uint64_t big_chunks_per_cta = (uint64_t)a.n_entries * ((tiles + 63u) / 64u) / (uint64_t)g_q4b.n_sm;
    return big_chunks_per_cta >= 20u ? launch_shape<4, 2>(a) : launch_shape<2, 4>(a);
}

}  // namespace few
