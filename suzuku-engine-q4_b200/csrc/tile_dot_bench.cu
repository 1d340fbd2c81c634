// Micro-benchmark of the warp-level tile dot (q4b_tile.cuh) with the tiles already in shared
// memory: what the IQ3_S decode costs by itself, away from copies and exchanges.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o tile_dot_bench tile_dot_bench.cu
//   ./tile_dot_bench
//
// Part 1 (throughput): 148 CTAs, every warp walks the CTA's 96 tiles round robin, 20 times;
// prints cycles per tile and SM for 8, 16, 24 and 32 warps per CTA.
// Part 2 (latency): a hidden unit = gate tile + up tile interleaved, both warp sums, SwiGLU and
// one store, repeated 16 times by warp 0; prints cycles per unit with 1, 4 and 16 warps at work.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "q4b_tile.cuh"

__device__ __forceinline__ float bench_swiglu(float g, float u) { return g / (1.f + expf(-g)) * u; }

template <int NT>
__global__ void __launch_bounds__(NT, 1) throughput_k(const uint32_t *codes, const uint8_t *tiles_g, int n_tiles,
                                                      int reps, float *out, long long *cycles) {
    extern __shared__ __align__(1024) uint8_t sm[];
    uint32_t *tab = (uint32_t *)sm;
    uint8_t *tiles = sm + 65536;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (uint32_t i = tid; i < 512 * 32; i += NT) tab[i] = codes[i >> 5];
    for (uint32_t i = tid; i < (uint32_t)n_tiles * 880 / 4; i += NT) ((uint32_t *)tiles)[i] = ((const uint32_t *)tiles_g)[i];
    int q[16];
    for (int i = 0; i < 16; i++) q[i] = (int)(0x01020304u * (lane + 1) + i * 0x11111111u);
    __syncthreads();
    const long long t0 = clock64();
    float acc = 0.f;
    const uint32_t *tl = tab + lane;
    for (int r = 0; r < reps; r++)
        for (int t = warp; t < n_tiles; t += NT / 32)
            acc += q4b_warp_sum(q4b_tile_lane_dot(tiles + (size_t)t * 880, lane, tl, q, 0.01f, 0.02f, 3 + r, 5));
    __syncthreads();
    const long long t1 = clock64();
    if (tid == 0) cycles[blockIdx.x] = t1 - t0;
    out[blockIdx.x * NT + tid] = acc;
}

__global__ void __launch_bounds__(512, 1) latency_k(const uint32_t *codes, const uint8_t *tiles_g, int n_tiles, int reps,
                                                    int active, float *out, long long *cycles) {
    extern __shared__ __align__(1024) uint8_t sm[];
    uint32_t *tab = (uint32_t *)sm;
    uint8_t *tiles = sm + 65536;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (uint32_t i = tid; i < 512 * 32; i += 512) tab[i] = codes[i >> 5];
    for (uint32_t i = tid; i < (uint32_t)n_tiles * 880 / 4; i += 512) ((uint32_t *)tiles)[i] = ((const uint32_t *)tiles_g)[i];
    int q[16];
    for (int i = 0; i < 16; i++) q[i] = (int)(0x01020304u * (lane + 1) + i * 0x11111111u);
    __syncthreads();
    const uint32_t *tl = tab + lane;
    const long long t0 = clock64();
    if ((int)warp < active) {
#pragma unroll 1
        for (int r = 0; r < reps; r++) {
            const uint32_t t = (warp * 2 + r * 6) % (n_tiles - 1);
            float g = q4b_tile_lane_dot(tiles + (size_t)t * 880, lane, tl, q, 0.01f, 0.02f, 3 + r, 5);
            float u = q4b_tile_lane_dot(tiles + (size_t)(t + 1) * 880, lane, tl, q, 0.01f, 0.02f, 3 + r, 5);
#pragma unroll
            for (int o = 16; o; o >>= 1) {
                g += __shfl_xor_sync(0xffffffffu, g, o);
                u += __shfl_xor_sync(0xffffffffu, u, o);
            }
            if (lane == 0) out[blockIdx.x * 512 + warp * 32 + (r & 31)] = bench_swiglu(g, u);
        }
    }
    const long long t1 = clock64();
    if (lane == 0 && warp == 0) cycles[blockIdx.x] = t1 - t0;
}

static double mean_cycles(const long long *d_cyc) {
    long long h[148];
    cudaMemcpy(h, d_cyc, sizeof(h), cudaMemcpyDeviceToHost);
    double avg = 0;
    for (int i = 0; i < 148; i++) avg += (double)h[i];
    return avg / 148;
}

template <int NT>
static void run_throughput(const uint32_t *d_codes, const uint8_t *d_tiles, int n_tiles, int reps, float *out,
                           long long *cyc) {
    const size_t smem = 65536 + (size_t)n_tiles * 880;
    cudaFuncSetAttribute(throughput_k<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    for (int it = 0; it < 2; it++) throughput_k<NT><<<148, NT, smem>>>(d_codes, d_tiles, n_tiles, reps, out, cyc);
    const cudaError_t e = cudaDeviceSynchronize();
    const double avg = mean_cycles(cyc);
    printf("throughput: %2d warps per CTA: %s, %.1f cycles per tile and SM\n", NT / 32, cudaGetErrorString(e),
           avg / (n_tiles * (double)reps));
}

static void run_latency(const uint32_t *d_codes, const uint8_t *d_tiles, int n_tiles, int reps, int active, float *out,
                        long long *cyc) {
    const size_t smem = 65536 + (size_t)n_tiles * 880;
    cudaFuncSetAttribute(latency_k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    for (int it = 0; it < 2; it++) latency_k<<<148, 512, smem>>>(d_codes, d_tiles, n_tiles, reps, active, out, cyc);
    const cudaError_t e = cudaDeviceSynchronize();
    printf("latency: %2d of 16 warps at work: %s, %.0f cycles per hidden unit (warp 0)\n", active, cudaGetErrorString(e),
           mean_cycles(cyc) / reps);
}

int main() {
    std::vector<uint32_t> codes(512);
    for (int i = 0; i < 512; i++) codes[i] = (i * 2654435761u) & 0x07070707u;
    const int n_tiles = 96;
    std::vector<uint8_t> tiles((size_t)n_tiles * 880);
    srand(1);
    for (auto &b : tiles) b = (uint8_t)(rand() & 0xff);
    uint32_t *d_codes;
    uint8_t *d_tiles;
    float *out;
    long long *cyc;
    cudaMalloc(&d_codes, 2048);
    cudaMalloc(&d_tiles, tiles.size());
    cudaMalloc(&out, 148 * 1024 * 4);
    cudaMalloc(&cyc, 148 * 8);
    cudaMemcpy(d_codes, codes.data(), 2048, cudaMemcpyHostToDevice);
    cudaMemcpy(d_tiles, tiles.data(), tiles.size(), cudaMemcpyHostToDevice);
    run_throughput<256>(d_codes, d_tiles, n_tiles, 20, out, cyc);
    run_throughput<512>(d_codes, d_tiles, n_tiles, 20, out, cyc);
    run_throughput<768>(d_codes, d_tiles, n_tiles, 20, out, cyc);
    run_throughput<1024>(d_codes, d_tiles, n_tiles, 20, out, cyc);
    run_latency(d_codes, d_tiles, n_tiles, 16, 1, out, cyc);
    run_latency(d_codes, d_tiles, n_tiles, 16, 4, out, cyc);
    run_latency(d_codes, d_tiles, n_tiles, 16, 16, out, cyc);
    return 0;
}
