// Seeded synthetic tensors generated on the device, for benchmarks and smoke
// runs at sizes where generating on the host and uploading would dominate the
// run (one MoE layer at the benchmark shapes is 693 MB of expert weights).
// Distributions follow the benchmark definition: per IQ3_S super-block
// fp16 d = |N(0,1)| * 2^-6, every other byte uniform random; fp32 tensors
// N(mean, std).  A counter-based generator (splitmix64 of seed and index), so
// the content does not depend on the launch geometry.
#include "q4b_internal.cuh"

#include <atomic>

#include "../../include/q4cuda.h"

extern std::atomic<uint64_t> g_q4b_launches;

namespace {

__device__ __forceinline__ uint64_t synth_mix(uint64_t z) {
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}
__device__ __forceinline__ float synth_normal(uint64_t seed, uint64_t i) {
    const uint64_t a = synth_mix(seed ^ synth_mix(2 * i));
    const uint64_t b = synth_mix(seed ^ synth_mix(2 * i + 1));
    const float u1 = ((float)(a >> 40) + 1.0f) * (1.0f / 16777217.0f);  // (0,1)
    const float u2 = (float)(b >> 40) * (1.0f / 16777216.0f);           // [0,1)
    return sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
}

__global__ void synth_iq3s_k(uint8_t *out, uint64_t n_blocks, uint64_t seed, uint64_t first) {
    const uint64_t bl = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (bl >= n_blocks) return;
    uint8_t *p = out + bl * Q4B_IQ3S_BYTES;
    const uint64_t b = first + bl;  // index in the whole tensor: a shard equals the same range of the full run
    const __half d = __float2half_rn(fabsf(synth_normal(seed, b)) * 0.015625f);
    const unsigned short db = __half_as_ushort(d);
    p[0] = (uint8_t)(db & 0xff);
    p[1] = (uint8_t)(db >> 8);
    for (uint32_t j = 0; j < 14; j++) {  // 108 payload bytes
        uint64_t r = synth_mix((seed + 0x51ed27ull) ^ synth_mix(b * 16 + j));
        const uint32_t nb = j < 13 ? 8u : 4u;
        for (uint32_t t = 0; t < nb; t++) {
            p[2 + 8 * j + t] = (uint8_t)(r & 0xff);
            r >>= 8;
        }
    }
}

__global__ void synth_normal_k(float *out, uint64_t n, uint64_t seed, float mean, float std) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t step = (uint64_t)gridDim.x * blockDim.x;
    for (; i < n; i += step) out[i] = mean + std * synth_normal(seed, i);
}

}  // namespace

extern "C" bool q4_cuda_synth_iq3s_at(uint8_t *d_out, uint64_t n_blocks, uint64_t seed,
                                      uint64_t first_block) {
    if (!g_q4b.ok || !d_out || n_blocks == 0) return false;
    synth_iq3s_k<<<(unsigned)((n_blocks + 255) / 256), 256, 0, g_q4b.stream>>>(d_out, n_blocks, seed,
                                                                                 first_block);
    g_q4b_launches++;
    return q4b_launch_ok("synth_iq3s");
}

extern "C" bool q4_cuda_synth_iq3s(uint8_t *d_out, uint64_t n_blocks, uint64_t seed) {
    return q4_cuda_synth_iq3s_at(d_out, n_blocks, seed, 0);
}

extern "C" bool q4_cuda_synth_normal(float *d_out, uint64_t n, uint64_t seed, float mean,
                                     float std) {
    if (!g_q4b.ok || !d_out || n == 0) return false;
    uint64_t nb = (n + 255) / 256;
    if (nb > 65535) nb = 65535;
    synth_normal_k<<<(unsigned)nb, 256, 0, g_q4b.stream>>>(d_out, n, seed, mean, std);
    g_q4b_launches++;
    return q4b_launch_ok("synth_normal");
}
