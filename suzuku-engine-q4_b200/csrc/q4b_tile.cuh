// The library's resident expert format ("tiled IQ3_S") and the warp-level dot
// product on it.
//
// An expert pack arrives in the engine's layout: matrices of rows of 110-byte
// IQ3_S super-blocks (fp16 d | qs[64] | qh[8] | signs[32] | scales[4]; reference
// src/q4_quant.c:384-394).  110-byte records are only 2-byte aligned, which
// rules out wide loads.  When a pack is put into an arena the library rewrites
// every run of eight consecutive super-blocks (880 bytes, always 16-byte
// aligned) in place as one TILE with the same bytes regrouped by field:
//
//   offset   0  d[8]        fp16 scale of block b at 2b
//           16  scales[8]   the 4 sub-scale bytes of block b at 16 + 4b
//           48  qh[8]       the 8 high-bit bytes of block b at 48 + 8b
//          112  signs[8]    32 bytes of block b at 112 + 32b, each 32-bit group
//                           word bit-permuted (see q4b_sign_permute)
//          368  qs[8]       the 64 index bytes of block b at 368 + 64b
//
// Same size, same position, a pure permutation of bits: row r of a matrix with
// eight blocks per row (2048 columns) is still the 880 bytes at r*880, and a
// matrix with two blocks per row (512 columns) has four rows per tile.  Lane l
// of a warp working on a tile owns block l/4, sub-block pair l%4, i.e. the
// byte-contiguous chunks qs[16l..), signs[8l..), qh[2l..), scales[l]: every
// load is aligned and conflict-free.
#pragma once

#include "q4b_internal.cuh"

#define Q4B_TILE_BYTES 880u
#define Q4B_TILE_OFF_D 0u
#define Q4B_TILE_OFF_SC 16u
#define Q4B_TILE_OFF_QH 48u
#define Q4B_TILE_OFF_SG 112u
#define Q4B_TILE_OFF_QS 368u

// Sign word of one 32-weight group: engine order has element e at bit e.  The
// tiled order puts element 4k+j (quad k, byte j) at bit 8j+7-k, so that
// (word << k) carries quad k's four sign bits in the top bit of each byte and
// one byte-permute turns them into a 0x00/0xFF mask.
__host__ __device__ inline uint32_t q4b_sign_permute(uint32_t w) {
    uint32_t o = 0;
    for (int k = 0; k < 8; k++)
        for (int j = 0; j < 4; j++) o |= ((w >> (4 * k + j)) & 1u) << (8 * j + 7 - k);
    return o;
}
__host__ __device__ inline uint32_t q4b_sign_unpermute(uint32_t w) {
    uint32_t o = 0;
    for (int k = 0; k < 8; k++)
        for (int j = 0; j < 4; j++) o |= ((w >> (8 * j + 7 - k)) & 1u) << (4 * k + j);
    return o;
}

#ifdef __CUDACC__

__device__ __forceinline__ uint32_t q4b_prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// Integer dot of one 32-weight group held in tiled form.
//   qs_lo/qs_hi: eight index bytes; qh: eight high bits (bit k for index k)
//   sgp: permuted sign word; tab: this lane's column of the replicated code
//   table (entry i at tab[TS i]; TS = 32 for the per-lane replicated table, 1 for a
//   plain 512-word table); q: eight int8x4 activation words; qsum: their sum.
template <int TS>
__device__ __forceinline__ int32_t q4b_tile_group_idot(uint32_t qs_lo, uint32_t qs_hi,
                                                       uint32_t qh, uint32_t sgp,
                                                       const uint32_t *tab, const int *q,
                                                       int32_t qsum) {
    int32_t acc0 = 0, acc1 = 0;
    // high bits spread to one byte each (0 or 1): bit i of a nibble -> bit 8i
    const uint32_t h_lo = ((qh & 0xfu) * 0x00204081u) & 0x01010101u;
    const uint32_t h_hi = (((qh >> 4) & 0xfu) * 0x00204081u) & 0x01010101u;
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const uint32_t w = k < 4 ? qs_lo : qs_hi;
        const uint32_t h = k < 4 ? h_lo : h_hi;
        const int b = k & 3;
        // byte0 = index byte, byte1 = its high bit, bytes 2,3 = 0 (top bit of a 0/1 byte)
        const uint32_t sel = (uint32_t)b | ((4u + b) << 4) | ((12u + b) << 8) | ((12u + b) << 12);
        const uint32_t idx = q4b_prmt(w, h, sel);
        const uint32_t c = tab[idx * TS];
        const uint32_t t = sgp << k;
        const uint32_t m = q4b_prmt(t, t, 0xba98u);
        if (k & 1)
            acc1 = __dp4a((int)(c ^ m), q[k], acc1);
        else
            acc0 = __dp4a((int)(c ^ m), q[k], acc0);
    }
    return 2 * (acc0 + acc1) + qsum;
}

// One lane's share of a tile: block l/4, groups 2(l%4) and 2(l%4)+1.
// q: 16 activation words of those 64 columns; dx/bs: their two group scales and
// sums.  Returns d * sum_g (1+2 s_g) * I_g * dx_g (the lane's part of the row dot).
__device__ __forceinline__ float q4b_tile_lane_dot(const uint8_t *tile, uint32_t lane,
                                                   const uint32_t *tab, const int *q, float dx0,
                                                   float dx1, int bs0, int bs1) {
    const uint4 qs = *reinterpret_cast<const uint4 *>(tile + Q4B_TILE_OFF_QS + 16u * lane);
    const uint2 sg = *reinterpret_cast<const uint2 *>(tile + Q4B_TILE_OFF_SG + 8u * lane);
    const uint32_t qh = *reinterpret_cast<const uint16_t *>(tile + Q4B_TILE_OFF_QH + 2u * lane);
    const uint32_t sc = tile[Q4B_TILE_OFF_SC + lane];
    const float d = __half2float(*reinterpret_cast<const __half *>(tile + 2u * (lane >> 2)));
    const int I0 = q4b_tile_group_idot<32>(qs.x, qs.y, qh & 0xffu, sg.x, tab, q, bs0);
    const int I1 = q4b_tile_group_idot<32>(qs.z, qs.w, qh >> 8, sg.y, tab, q + 8, bs1);
    const float f = (float)(I0 * (int)(2u * (sc & 15u) + 1u)) * dx0 +
                    (float)(I1 * (int)(2u * (sc >> 4) + 1u)) * dx1;
    return d * f;
}

#endif  // __CUDACC__
