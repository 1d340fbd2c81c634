/* GPU test of the C host mirror (suzuku-engine-q4_b200/host/q4_moe_b200.c): a C program, like
 * the reference engine, that loads one synthetic MoE layer through the device C ABI and runs
 * it (a) by the reference's fine-grained call sequence, (b) by the fused call, (c) as a batch,
 * and checks all three against the CPU oracle (oracle/q4_oracle.c, test infrastructure).
 * Prints "PASS" and exits 0, or says what differed and exits 1.  Exit 2: no usable GPU. */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/q4cuda.h"
#include "../../oracle/q4_oracle.h"
#include "../../suzuku-engine-q4_b200/host/q4_moe_b200.h"

static uint64_t rng_state = 0x243f6a8885a308d3ull;
static uint64_t next_u64(void) {
    uint64_t z = (rng_state += 0x9e3779b97f4a7c15ull);
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}
static float next_normal(void) {
    const double u1 = ((double)(next_u64() >> 11) + 1.0) / 9007199254740993.0;
    const double u2 = (double)(next_u64() >> 11) / 9007199254740992.0;
    return (float)(sqrt(-2.0 * log(u1)) * cos(6.283185307179586 * u2));
}
/* fp32 -> fp16 bits, round to nearest even, for small positive normal values */
static uint16_t f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    int32_t e = (int32_t)((x >> 23) & 0xff) - 127 + 15;
    uint32_t m = x & 0x7fffffu;
    if (e <= 0) return (uint16_t)sign;                 /* flush tiny values to zero */
    uint32_t h = ((uint32_t)e << 10) | (m >> 13);
    const uint32_t rem = m & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++;
    return (uint16_t)(sign | h);
}
/* one IQ3_S super-block: fp16 d = |N(0,1)| * 2^-6, every other byte uniform random */
static void synth_block(uint8_t *b) {
    const uint16_t d = f32_to_f16(fabsf(next_normal()) * 0.015625f);
    b[0] = (uint8_t)(d & 0xff);
    b[1] = (uint8_t)(d >> 8);
    for (int i = 2; i < 110; i++) b[i] = (uint8_t)(next_u64() & 0xff);
}
static double rel_l2(const float *a, const float *b, uint32_t n) {
    double num = 0, den = 0;
    for (uint32_t i = 0; i < n; i++) {
        num += ((double)a[i] - b[i]) * ((double)a[i] - b[i]);
        den += (double)b[i] * b[i];
    }
    return sqrt(num / (den > 0 ? den : 1e-30));
}

#define CHECK(c, msg)                                   \
    do {                                                \
        if (!(c)) {                                     \
            fprintf(stderr, "FAIL: %s (line %d)\n", msg, __LINE__); \
            return 1;                                   \
        }                                               \
    } while (0)

int main(void) {
    enum { H = 2048, F = 512, E = 32, K = 6, T = 5 };
    if (!q4_hip_init()) {
        fprintf(stderr, "no usable sm_100 GPU: q4_hip_init refused (there is no CPU path)\n");
        return 2;
    }
    const uint64_t pb = q4b_expert_pack_bytes(H, F);
    uint8_t *packs = malloc((size_t)(E + 1) * pb);
    float *router = malloc(sizeof(float) * E * H), *norm_w = malloc(sizeof(float) * H);
    float *x = malloc(sizeof(float) * T * H);
    CHECK(packs && router && norm_w && x, "host allocation");
    for (uint64_t b = 0; b < (uint64_t)(E + 1) * pb / 110; b++) synth_block(packs + b * 110);
    for (int i = 0; i < E * H; i++) router[i] = 0.02f * next_normal();
    for (int i = 0; i < H; i++) norm_w[i] = 1.0f + 0.1f * next_normal();
    for (int i = 0; i < T * H; i++) x[i] = next_normal();

    q4b_moe_layer L;
    memset(&L, 0, sizeof L);
    CHECK(q4b_moe_layer_load(&L, 0, packs, packs + (uint64_t)E * pb, E, H, F), "layer load");
    L.topk = K;
    L.eps = 1e-6f;
    float *d_router = q4_hip_malloc(sizeof(float) * E * H), *d_norm = q4_hip_malloc(sizeof(float) * H);
    float *d_x = q4_hip_malloc(sizeof(float) * T * H), *d_y = q4_hip_malloc(sizeof(float) * T * H);
    float *d_ws1 = q4_hip_malloc(sizeof(float) * q4_moe_layer_dev_ws_floats(&L));
    const uint64_t wsn = q4_cuda_moe_layer_n_ws_bytes(T, K, E, H, F);
    void *d_wsn = q4_hip_malloc(wsn);
    int32_t *d_ids = q4_hip_malloc(sizeof(int32_t) * 64);
    float *d_wts = q4_hip_malloc(sizeof(float) * 64);
    CHECK(d_router && d_norm && d_x && d_y && d_ws1 && d_wsn && d_ids && d_wts, "device allocation");
    CHECK(q4_hip_h2d(d_router, router, sizeof(float) * E * H) && q4_hip_h2d(d_norm, norm_w, sizeof(float) * H) &&
              q4_hip_h2d(d_x, x, sizeof(float) * T * H),
          "upload");
    L.d_router = d_router;
    L.d_norm_w = d_norm;

    float *want = malloc(sizeof(float) * T * H), *got = malloc(sizeof(float) * T * H);
    int32_t ids0[T][64], ids1[64];
    for (int t = 0; t < T; t++)
        q4o_moe_layer(x + t * H, norm_w, 1e-6f, router, E, K, packs, pb, packs + (uint64_t)E * pb, H, F,
                      want + t * H, ids0[t], NULL, NULL);

    /* (a) the reference's fine-grained sequence, token by token */
    for (int t = 0; t < T; t++) {
        CHECK(q4_moe_layer_dev(&L, d_x + t * H, d_y + t * H, d_ws1), "q4_moe_layer_dev");
    }
    CHECK(q4_hip_d2h(got, d_y, sizeof(float) * T * H), "download");
    for (int t = 0; t < T; t++) {
        const double r = rel_l2(got + t * H, want + t * H, H);
        if (r > 1e-3) fprintf(stderr, "chain token %d rel-L2 %.3g\n", t, r);
        CHECK(r <= 1e-3, "fine-grained sequence vs oracle");
    }
    /* (b) the fused call: same picks, same numbers as (a) up to the summation order */
    float *got_b = malloc(sizeof(float) * T * H);
    for (int t = 0; t < T; t++) {
        CHECK(q4_moe_layer_dev_fused(&L, d_x + t * H, d_y + t * H, d_ids, d_wts), "q4_moe_layer_dev_fused");
        CHECK(q4_hip_d2h(ids1, d_ids, sizeof(int32_t) * K), "ids download");
        for (int k = 0; k < K; k++) CHECK(ids1[k] == ids0[t][k], "picks differ from the oracle's");
    }
    CHECK(q4_hip_d2h(got_b, d_y, sizeof(float) * T * H), "download");
    for (int t = 0; t < T; t++) {
        CHECK(rel_l2(got_b + t * H, want + t * H, H) <= 1e-3, "fused call vs oracle");
        CHECK(rel_l2(got_b + t * H, got + t * H, H) <= 1e-5, "fused call vs fine-grained sequence");
    }
    /* (c) all tokens in one call */
    CHECK(q4_moe_layer_dev_n(&L, d_x, d_y, T, d_wsn, wsn), "q4_moe_layer_dev_n");
    CHECK(q4_hip_d2h(got_b, d_y, sizeof(float) * T * H), "download");
    for (int t = 0; t < T; t++) CHECK(rel_l2(got_b + t * H, want + t * H, H) <= 1e-3, "batched call vs oracle");
    /* (d) the loader from stacked tensors (one tensor per matrix kind, experts back to back)
     * builds the same packs: read them back in the engine's byte order and compare */
    {
        const uint64_t sg = (uint64_t)F * q4b_iq3s_row_bytes(H), sd = (uint64_t)H * q4b_iq3s_row_bytes(F);
        uint8_t *gate = malloc((size_t)E * sg), *up = malloc((size_t)E * sg), *down = malloc((size_t)E * sd);
        uint8_t *back = malloc((size_t)pb);
        CHECK(gate && up && down && back, "host allocation");
        for (int e = 0; e < E; e++) {
            memcpy(gate + (uint64_t)e * sg, packs + (uint64_t)e * pb, sg);
            memcpy(up + (uint64_t)e * sg, packs + (uint64_t)e * pb + sg, sg);
            memcpy(down + (uint64_t)e * sd, packs + (uint64_t)e * pb + 2 * sg, sd);
        }
        const uint8_t *shp = packs + (uint64_t)E * pb;
        q4b_moe_layer L2;
        memset(&L2, 0, sizeof L2);
        CHECK(q4b_moe_layer_load_stacked(&L2, 1, gate, up, down, shp, shp + sg, shp + 2 * sg, E, H, F),
              "stacked load");
        CHECK(L2.shared_slot == E && L2.ou == sg && L2.od == 2 * sg, "stacked layer geometry");
        for (int e = 0; e <= E; e += 7) {
            CHECK(q4_cuda_experts_get_a(1, (uint32_t)e, back, pb), "pack read-back");
            CHECK(memcmp(back, packs + (uint64_t)e * pb, pb) == 0, "stacked loader built a different pack");
        }
        CHECK(q4_cuda_experts_get_a(1, E, back, pb) && memcmp(back, shp, pb) == 0, "shared pack differs");
        CHECK(!q4b_moe_layer_load_stacked(&L2, 2, gate, up, down, shp, NULL, NULL, E, H, F),
              "half-given shared expert must be refused");
        q4_hip_experts_free_a(1);
        free(gate), free(up), free(down), free(back);
    }
    /* refusals: nothing is enqueued for a shape the path does not take */
    q4b_moe_layer bad = L;
    bad.topk = 0;
    CHECK(!q4_moe_layer_dev(&bad, d_x, d_y, d_ws1), "topk 0 must be refused");
    CHECK(!q4_moe_layer_dev_n(&L, d_x, d_y, T, d_wsn, wsn - 1), "short workspace must be refused");
    CHECK(q4_cuda_device_error() == 0, "device error word");
    q4_hip_shutdown();
    printf("PASS\n");
    return 0;
}
