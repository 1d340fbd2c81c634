"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (no model file or dataset is involved).

IQ3_S super-block (110 bytes, 256 weights; reference layout src/q4_quant.c:384-394):
fp16 d = |N(0,1)| * 2^-6; qs / qh / sign bytes uniform random; the four scale
bytes uniform random (two uniform 4-bit sub-scales each).  This mirrors the
reference tests' rule "random payload, sane scale" (src/q4_test.c:250-262).
"""
import numpy as np

IQ3S_BLOCK = 110
QK_K = 256


def iq3s_row_bytes(ncols):
    assert ncols % QK_K == 0
    return ncols // QK_K * IQ3S_BLOCK


def expert_pack_bytes(n_embd, n_ff):
    """gate [n_ff x n_embd] | up [n_ff x n_embd] | down [n_embd x n_ff]
    (reference pack order: src/q4_expert.c:962-982)."""
    return 2 * n_ff * iq3s_row_bytes(n_embd) + n_embd * iq3s_row_bytes(n_ff)


def iq3s_blocks(rng, n_blocks):
    """n_blocks random super-blocks -> uint8 [n_blocks, 110]."""
    b = rng.integers(0, 256, size=(n_blocks, IQ3S_BLOCK), dtype=np.uint8)
    d = (np.abs(rng.standard_normal(n_blocks)) * 2.0 ** -6).astype(np.float16)
    b[:, 0:2] = d.view(np.uint8).reshape(n_blocks, 2)
    return b


IQ4NL_BLOCK = 18


def iq4nl_blocks(rng, n_blocks):
    """n_blocks random IQ4_NL blocks (fp16 d = |N(0,1)| * 2^-6, 16 bytes of 4-bit codes)."""
    b = rng.integers(0, 256, size=(n_blocks, IQ4NL_BLOCK), dtype=np.uint8)
    d = (np.abs(rng.standard_normal(n_blocks)) * 2.0 ** -6).astype(np.float16)
    b[:, 0:2] = d.view(np.uint8).reshape(n_blocks, 2)
    return b


def expert_pack_bytes_mixed(n_embd, n_ff):
    """gate, up IQ3_S; down IQ4_NL (one of the mixes the engine's call sites accept,
    src/q4_rocm.cu:4926-4944)."""
    return 2 * n_ff * iq3s_row_bytes(n_embd) + n_embd * (n_ff // 32) * IQ4NL_BLOCK


def expert_packs_mixed(rng, n, n_embd, n_ff):
    """n packed experts with an IQ4_NL down projection -> uint8 [n, pack_bytes]."""
    gu = 2 * n_ff * iq3s_row_bytes(n_embd)
    dn = n_embd * (n_ff // 32) * IQ4NL_BLOCK
    out = np.empty((n, gu + dn), np.uint8)
    for e in range(n):
        out[e, :gu] = iq3s_blocks(rng, gu // IQ3S_BLOCK).reshape(-1)
        out[e, gu:] = iq4nl_blocks(rng, dn // IQ4NL_BLOCK).reshape(-1)
    return out


IQ4XS_BLOCK = 136


def iq4xs_blocks(rng, n_blocks):
    """n_blocks random IQ4_XS super-blocks (fp16 d = |N(0,1)| * 2^-6, everything else uniform)."""
    b = rng.integers(0, 256, size=(n_blocks, IQ4XS_BLOCK), dtype=np.uint8)
    d = (np.abs(rng.standard_normal(n_blocks)) * 2.0 ** -6).astype(np.float16)
    b[:, 0:2] = d.view(np.uint8).reshape(n_blocks, 2)
    return b


# K-quant super-blocks (public ggml formats): {bytes per 256 values, offsets of the fp16 d and dmin}
KQUANT = {12: (144, 0, 2), 13: (176, 0, 2), 14: (210, 208, None)}


def kquant_blocks(rng, type_id, n_blocks):
    """n_blocks random Q4_K (12), Q5_K (13) or Q6_K (14) super-blocks: uniform bytes, fp16
    d = |N(0,1)| * 2^-8 and (Q4_K, Q5_K) dmin = |N(0,1)| * 2^-9, the magnitudes of the
    reference's own test of this product (src/q4_test.c:2678-2682)."""
    bs, od, om = KQUANT[type_id]
    b = rng.integers(0, 256, size=(n_blocks, bs), dtype=np.uint8)
    d = (np.abs(rng.standard_normal(n_blocks)) * 2.0 ** -8).astype(np.float16)
    b[:, od:od + 2] = d.view(np.uint8).reshape(n_blocks, 2)
    if om is not None:
        m = (np.abs(rng.standard_normal(n_blocks)) * 2.0 ** -9).astype(np.float16)
        b[:, om:om + 2] = m.view(np.uint8).reshape(n_blocks, 2)
    return b


# the remaining routed-expert formats: {bytes per block, values per block}; all byte patterns are valid
SMALL_FORMATS = {18: (98, 256), 22: (82, 256), 42: (18, 64)}      # IQ3_XXS, IQ2_S, Q2_0


def small_format_blocks(rng, type_id, n_blocks):
    """n_blocks random IQ3_XXS (18), IQ2_S (22) or Q2_0 (42) blocks: uniform bytes, fp16 d = |N(0,1)| * 2^-6."""
    bs = SMALL_FORMATS[type_id][0]
    b = rng.integers(0, 256, size=(n_blocks, bs), dtype=np.uint8)
    d = (np.abs(rng.standard_normal(n_blocks)) * 2.0 ** -6).astype(np.float16)
    b[:, 0:2] = d.view(np.uint8).reshape(n_blocks, 2)
    return b


def row_bytes(type_id, ncols):
    if type_id in SMALL_FORMATS:
        return ncols // SMALL_FORMATS[type_id][1] * SMALL_FORMATS[type_id][0]
    if type_id in KQUANT:
        return ncols // 256 * KQUANT[type_id][0]
    return {21: ncols // 256 * IQ3S_BLOCK, 20: ncols // 32 * IQ4NL_BLOCK, 23: ncols // 256 * IQ4XS_BLOCK}[type_id]


def blocks_of(rng, type_id, nbytes):
    if type_id in SMALL_FORMATS:
        return small_format_blocks(rng, type_id, nbytes // SMALL_FORMATS[type_id][0]).reshape(-1)
    if type_id in KQUANT:
        return kquant_blocks(rng, type_id, nbytes // KQUANT[type_id][0]).reshape(-1)
    make, bs = {21: (iq3s_blocks, IQ3S_BLOCK), 20: (iq4nl_blocks, IQ4NL_BLOCK), 23: (iq4xs_blocks, IQ4XS_BLOCK)}[type_id]
    return make(rng, nbytes // bs).reshape(-1)


def expert_packs_typed(rng, n, n_embd, n_ff, gu_type, down_type):
    """n packed experts, gate and up of one format, down of another -> uint8 [n, pack_bytes]."""
    gu = 2 * n_ff * row_bytes(gu_type, n_embd)
    dn = n_embd * row_bytes(down_type, n_ff)
    out = np.empty((n, gu + dn), np.uint8)
    for e in range(n):
        out[e, :gu] = blocks_of(rng, gu_type, gu)
        out[e, gu:] = blocks_of(rng, down_type, dn)
    return out


def expert_packs(rng, n, n_embd, n_ff):
    """n packed experts -> uint8 [n, pack_bytes]."""
    pb = expert_pack_bytes(n_embd, n_ff)
    assert pb % IQ3S_BLOCK == 0
    return iq3s_blocks(rng, n * (pb // IQ3S_BLOCK)).reshape(n, pb)


def layer(seed, n_expert, n_embd, n_ff):
    """One MoE layer: routed packs, shared pack, router, norm weight."""
    rng = np.random.default_rng(seed)
    return {
        "experts": expert_packs(rng, n_expert, n_embd, n_ff),
        "shared": expert_packs(rng, 1, n_embd, n_ff)[0],
        "router": (rng.standard_normal((n_expert, n_embd)) * 0.02).astype(np.float32),
        "norm_w": (1.0 + 0.1 * rng.standard_normal(n_embd)).astype(np.float32),
    }


def hidden(seed, n_tok, n_embd):
    rng = np.random.default_rng(seed)
    return rng.standard_normal((n_tok, n_embd)).astype(np.float32)


def zipf_bias(n_expert, s=1.1):
    """Additive router-logit bias that skews expert popularity: the log of a
    Zipf(s) probability mass over expert rank (expert 0 the most popular)."""
    r = np.arange(1, n_expert + 1, dtype=np.float64)
    p = r ** -s
    p /= p.sum()
    return np.log(p).astype(np.float32)


class XorShift64:
    """The generator the reference's tests use for weight bytes
    (src/q4_test.c:250-254): x ^= x<<13; x ^= x>>7; x ^= x<<17."""

    def __init__(self, seed):
        self.s = seed & 0xFFFFFFFFFFFFFFFF

    def next(self):
        s = self.s
        s ^= (s << 13) & 0xFFFFFFFFFFFFFFFF
        s ^= s >> 7
        s ^= (s << 17) & 0xFFFFFFFFFFFFFFFF
        self.s = s
        return s

    def bytes(self, n):
        out = np.empty(n, np.uint8)
        for i in range(n):
            out[i] = self.next() & 0xFF
        return out
