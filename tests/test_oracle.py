"""Pin the CPU oracle: the reference's closed-form known answers, the golden
vectors generated from the reference's own CPU code, and (where the compiled
reference is available) bit-for-bit agreement on fresh random inputs."""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(__file__), "golden", "iq3s_moe_small.npz")


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD)


def _bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def test_kat_zero_block_dot_is_256(oracle, gold):
    # src/q4_test.c:52-58: all-zero IQ3_S block, d = 1.0, x = 1 -> 256
    blk = np.zeros(110, np.uint8)
    blk[0:2] = np.array([0x3c00], np.uint16).view(np.uint8)
    w = oracle.dequant_row(blk, 256)
    assert abs(float(w.sum()) - 256.0) < 1e-2
    assert abs(float(gold["kat"]) - 256.0) < 1e-2
    xq = oracle.quant8(np.ones(256, np.float32))
    assert abs(oracle.dot8(blk, xq, 256) - 256.0) < 1e-2
    assert oracle.group_idot(blk, xq, 256).tolist() == [32 * 127] * 8


def test_grid_entries_are_odd_below_16(oracle):
    g = oracle.grid()
    b = np.stack([(g >> (8 * j)) & 0xFF for j in range(4)])
    assert ((b % 2) == 1).all() and (b <= 15).all()
    assert g[0] == 0x01010101 and len(set(g.tolist())) == 512


def test_f16_conversion_all_values(oracle):
    h = np.arange(65536, dtype=np.uint16)
    ref = h.view(np.float16).astype(np.float32)
    got = np.array([oracle.f16_to_f32(int(v)) for v in h[::7]], np.float32)
    exp = ref[::7]
    nan = np.isnan(exp)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(_bits(got[~nan]), _bits(exp[~nan]))


def test_golden_dequant_quant_dots(oracle, gold):
    H, F = int(gold["H"]), int(gold["F"])
    packs, x = gold["packs"], gold["x"]
    rb = H // 256 * 110
    for r in range(4):
        got = oracle.dequant_row(packs[0][r * rb:(r + 1) * rb], H)
        assert np.array_equal(_bits(got), _bits(gold["deq"][r]))
    xq = oracle.quant8(x)
    assert xq.tobytes() == gold["xq"].tobytes()
    assert (xq["q"][1] == 0).all() and xq["d"][1] == 0.0  # the all-zero group
    dots = oracle.matvec8(packs[0][:F * rb], F, xq, H)
    assert np.array_equal(_bits(dots), _bits(gold["gate_dots"]))


def test_golden_expert_outputs(oracle, gold):
    H, F = int(gold["H"]), int(gold["F"])
    packs, x = gold["packs"], gold["x"]
    y1 = oracle.expert_job([packs[0]], [1.0], x, H, F)
    assert np.array_equal(_bits(y1), _bits(gold["y1"]))  # one expert: no ordering freedom
    y2 = oracle.expert_job([packs[0], packs[1]], gold["wts"], x, H, F)
    # two experts: the reference adds them in a racy order and may fuse the
    # multiply into the add, so allow the last bits
    assert np.allclose(y2, gold["y2"], rtol=0, atol=2e-6 * np.abs(gold["y2"]).max())


def test_golden_router(oracle, gold):
    x, nw = gold["x"], gold["norm_w"]
    xn = oracle.rms_norm(x, nw, 1e-6)
    assert np.array_equal(_bits(xn), _bits(gold["xn"]))
    logits = gold["logits"]
    p = oracle.softmax(logits)
    assert np.array_equal(_bits(p), _bits(gold["probs"]))
    ids, w = oracle.topk(p, 6, True)
    assert ids.tolist() == gold["top_ids"].tolist()
    assert np.array_equal(_bits(w), _bits(gold["top_w"]))
    # the planted tie: equal values keep the lower index first
    li = ids.tolist()
    if 3 in li and 7 in li:
        assert li.index(3) < li.index(7)
    assert 7 not in li or 3 in li


def test_integer_dot_matches_dequantised_weights(oracle):
    rng = np.random.default_rng(5)
    blk = rng.integers(0, 256, 220, dtype=np.uint8)
    for b in range(2):
        blk[110 * b:110 * b + 2] = np.array([0x3c00], np.uint16).view(np.uint8)  # d = 1
    x = rng.standard_normal(512).astype(np.float32)
    xq = oracle.quant8(x)
    I = oracle.group_idot(blk, xq, 512)
    w = oracle.dequant_row(blk, 512)
    for g in range(16):
        wv, ls, _ = oracle.unpack(blk[110 * (g // 8):110 * (g // 8 + 1)])
        ib = g % 8
        exp = int(np.dot(wv[32 * ib:32 * ib + 32].astype(np.int64), xq[g]["q"].astype(np.int64)))
        assert I[g] == exp
        # dequantised weight = d * ls * signed magnitude
        assert np.array_equal(w[32 * g:32 * g + 32], wv[32 * ib:32 * ib + 32].astype(np.float32) * ls[ib])


def test_quant8_properties(oracle):
    rng = np.random.default_rng(7)
    x = (rng.standard_normal(4096) * rng.uniform(1e-3, 1e3, 4096)).astype(np.float32)
    xq = oracle.quant8(x)
    xr = (xq["q"].astype(np.float32) * xq["d"][:, None]).ravel()
    dmax = np.repeat(xq["d"], 32)
    assert (np.abs(x - xr) <= 0.51 * dmax + 1e-30).all()  # src/q4_cpuexp.c selftest bound
    assert (xq["bs"] == xq["q"].astype(np.int32).sum(1)).all()
    assert np.abs(xq["q"]).max() == 127
    # round-half-even at exact ties
    t = np.zeros(32, np.float32)
    t[0] = 127.0
    t[1] = 0.5
    t[2] = 1.5
    t[3] = 2.5
    t[4] = -0.5
    q = oracle.quant8(t)["q"][0]
    assert q[:5].tolist() == [127, 0, 2, 2, 0]


def test_topk_edge_cases(oracle):
    p = np.array([0.1, 0.4, 0.4, 0.05, 0.05], np.float32)
    ids, w = oracle.topk(p, 3, False)
    assert ids.tolist() == [1, 2, 0]
    ids, w = oracle.topk(p, 9, True)  # k > n clamps
    assert ids[:5].tolist() == [1, 2, 0, 3, 4]


def test_mmq_order_dot_close_to_cpu_order(oracle):
    rng = np.random.default_rng(11)
    H = 2048
    row = np.frombuffer(rng.integers(0, 256, H // 256 * 110, dtype=np.uint8).tobytes(), np.uint8).copy()
    for b in range(H // 256):
        row[110 * b:110 * b + 2] = np.array([0x2a66], np.uint16).view(np.uint8)
    x = rng.standard_normal(H).astype(np.float32)
    q, d = oracle.quant8_mmq(x)
    a = oracle.dot_mmq(row, q, d, H)
    b_ = oracle.dot8(row, oracle.quant8(x), H)
    assert abs(a - b_) <= 2e-3 * (1 + abs(b_))
    # half-away-from-zero vs half-even: differ only at exact ties
    t = np.zeros(32, np.float32)
    t[0], t[1], t[2] = 127.0, 0.5, 2.5
    assert q.dtype == np.int8 and oracle.quant8_mmq(t)[0][:3].tolist() == [127, 1, 3]


def test_against_compiled_reference(oracle, reference):
    if reference is None:
        pytest.skip("compiled reference CPU path not available on this machine")
    assert reference.selftest() == 0
    rng = np.random.default_rng(3)
    H, F = 2048, 512
    rb = H // 256 * 110
    blocks = rng.integers(0, 256, size=(16, rb), dtype=np.uint8)
    for r in range(16):
        for b in range(H // 256):
            dd = np.float16(abs(rng.standard_normal()) * 2.0 ** -6)
            blocks[r, 110 * b:110 * b + 2] = np.array([dd]).view(np.uint8)
    x = rng.standard_normal(H).astype(np.float32)
    xq = oracle.quant8(x)
    assert xq.tobytes() == reference.quant8(x).tobytes()
    for r in range(16):
        assert np.array_equal(_bits(oracle.dequant_row(blocks[r], H)),
                              _bits(reference.dequant_row(blocks[r], H)))
        a = np.float32(oracle.dot8(blocks[r], xq, H))
        assert _bits(a) == _bits(np.float32(reference.dot8(blocks[r], xq, H)))
        assert _bits(a) == _bits(np.float32(reference.dot8(blocks[r], xq, H, avx2=True)))


# ---- IQ4_NL (type 20): a routed expert's down projection may use it ----
def test_iq4nl_oracle_pinned_to_reference(pkg, oracle, reference):
    """Dequantisation, the per-block integer dots and the Q8-A row dot of the restatement against the
    reference's own code (src/q4_quant.c:270-290, src/q4_cpuexp.c:977-996) on seeded blocks: bit-exact."""
    if reference is None:
        pytest.skip("reference CPU path not built here")
    rng = np.random.default_rng(2024)
    n = 512
    rows = pkg.synth.iq4nl_blocks(rng, 6 * n // 32).reshape(6, -1)
    x = rng.standard_normal(n).astype(np.float32)
    xq = oracle.quant8(x)
    for row in rows:
        a, b = oracle.iq4nl_dequant_row(row, n), reference.dequant_row_t(20, row, n)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
        got = oracle.iq4nl_dot8(row, xq, n)
        for want in (reference.dot8_t(20, row, xq, n, avx2_iq4nl=True), reference.dot8_t(20, row, xq, n)):
            assert np.float32(got).view(np.uint32) == np.float32(want).view(np.uint32)
        # integer parts: table value x q summed per block, against a direct numpy evaluation
        I = oracle.iq4nl_group_idot(row, xq, n)
        w = np.rint(oracle.iq4nl_dequant_row(np.concatenate(
            [np.concatenate([np.array([0x00, 0x3c], np.uint8), blk[2:]]) for blk in row.reshape(-1, 18)]), n))
        want_I = (w.reshape(-1, 32).astype(np.int64) * xq["q"].astype(np.int64)).sum(1)
        assert np.array_equal(I, want_I)


def test_expert_job_with_iq4nl_down_matches_reference(pkg, oracle, reference):
    """gate/up IQ3_S, down IQ4_NL through the reference's worker pool (q4_cpuex_dispatch2) vs the
    restatement; y is summed by the pool in worker order, hence the last-bit tolerance."""
    if reference is None:
        pytest.skip("reference CPU path not built here")
    H, F, k = 512, 256, 3
    rng = np.random.default_rng(77)
    packs = pkg.synth.expert_packs_mixed(rng, k, H, F)
    x = rng.standard_normal(H).astype(np.float32)
    wts = rng.random(k).astype(np.float32)
    reference.set_down_type(20)
    try:
        want = reference.expert_job(list(packs), np.arange(k, dtype=np.int32), wts, x, H, F)
    finally:
        reference.set_down_type(21)
    got = oracle.expert_job_t(list(packs), wts, x, H, F, 20)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 2e-6


def test_iq4xs_oracle_pinned_to_reference(pkg, oracle, reference):
    """IQ4_XS (type 23): dequantisation and the Q8-A row dot bit-exact against the reference's
    q4_dequant_row / dq8_iq4_xs / cpx_dot8 (src/q4_quant.c:455-480, src/q4_cpuexp.c:945-975)."""
    if reference is None:
        pytest.skip("reference CPU path not built here")
    rng = np.random.default_rng(2025)
    n = 1024
    rows = pkg.synth.iq4xs_blocks(rng, 5 * n // 256).reshape(5, -1)
    xq = oracle.quant8(rng.standard_normal(n).astype(np.float32))
    for row in rows:
        a, b = oracle.iq4xs_dequant_row(row, n), reference.dequant_row_t(23, row, n)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
        got = oracle.dot8_t(23, row, xq, n)
        for want in (reference.dot8_t(23, row, xq, n, avx2_iq4xs=True), reference.dot8_t(23, row, xq, n)):
            assert np.float32(got).view(np.uint32) == np.float32(want).view(np.uint32)


@pytest.mark.parametrize("gu,dn", [(23, 21), (23, 20), (21, 23), (20, 23)])
def test_expert_job_other_format_mixes_match_reference(pkg, oracle, reference, gu, dn):
    if reference is None:
        pytest.skip("reference CPU path not built here")
    H, F, k = 512, 256, 3
    rng = np.random.default_rng(gu * 100 + dn)
    packs = pkg.synth.expert_packs_typed(rng, k, H, F, gu, dn)
    x = rng.standard_normal(H).astype(np.float32)
    wts = rng.random(k).astype(np.float32)
    reference.set_gu_type(gu)
    reference.set_down_type(dn)
    try:
        want = reference.expert_job(list(packs), np.arange(k, dtype=np.int32), wts, x, H, F)
    finally:
        reference.set_gu_type(21)
        reference.set_down_type(21)
    got = oracle.expert_job_t(list(packs), wts, x, H, F, dn, gu)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 2e-6


# ---- the dense product of up to 8 activation rows in 8-bit form (src/q4_mmvq.cu) ----
DENSE_GOLD = os.path.join(os.path.dirname(__file__), "golden", "dense_types_dequant.npz")
DENSE_TYPES = (12, 13, 14, 23, 20)      # Q4_K, Q5_K, Q6_K, IQ4_XS, IQ4_NL


@pytest.mark.parametrize("ty", DENSE_TYPES)
def test_dense_run_decoders_against_reference_dequant(oracle, reference, ty):
    """value = a * w + c of every 16-value run against the reference's q4_dequant_row (fixture made by
    tests/golden/gen_golden.py, and the compiled reference itself where it is present).  One wrong bit
    in a decoded weight moves a value by a whole step `a`; the bound is a few float roundings."""
    g = np.load(DENSE_GOLD)
    n = int(g["n"])
    for row, want in zip(g["rows_%d" % ty], g["deq_%d" % ty]):
        got = oracle.mv_dequant_row(ty, row, n)
        assert np.abs(got - want).max() <= 4e-7 * np.abs(want).max()
        if reference is not None:
            live = reference.dequant_row_t(ty, row, n)
            assert np.array_equal(live.view(np.uint32), want.view(np.uint32))


def test_dense_quantiser_divides_and_sums_halves(oracle):
    rng = np.random.default_rng(9)
    x = rng.standard_normal(256).astype(np.float32)
    x[32:64] = 0.0
    x[64], x[65] = 127.0, 0.5              # d = 1: 0.5 rounds to even (0)
    x[66:96] = 0.25
    q, d, s16 = oracle.quant8_d(x)
    assert d[1] == 0 and not q[32:64].any() and d[2] == 1.0 and q[64] == 127 and q[65] == 0
    for gi in range(8):
        xb = x[32 * gi:32 * gi + 32]
        dg = np.float32(np.abs(xb).max()) / np.float32(127)
        assert d[gi] == dg
        if dg > 0:
            assert np.array_equal(q[32 * gi:32 * gi + 32], np.rint(xb / dg).astype(np.int8))
    assert np.array_equal(s16, q.astype(np.int32).reshape(-1, 16).sum(1))


@pytest.mark.parametrize("ty", DENSE_TYPES)
def test_dense_product_accuracy_and_row_independence(pkg, oracle, ty):
    """The bound of the reference's own test (src/q4_test.c:2702-2716: rel-L2 < 2e-2 against the
    dequantised weights in double) and a row's result not depending on the rows beside it."""
    rng = np.random.default_rng(40 + ty)
    K, R, NT = 2560, 24, 3
    w = np.stack([pkg.synth.blocks_of(rng, ty, pkg.synth.row_bytes(ty, K)) for _ in range(R)])
    xs = (rng.integers(-1000, 1001, (NT, K)) * 1e-3).astype(np.float32)
    y = oracle.mv_rows(ty, w, R, K, xs, 0.5)
    deq = np.stack([oracle.mv_dequant_row(ty, r, K) for r in w]).astype(np.float64)
    want = 0.5 * xs.astype(np.float64) @ deq.T
    assert np.linalg.norm(y - want) / np.linalg.norm(want) < 2e-2
    y1 = oracle.mv_rows(ty, w, R, K, xs[1:2], 0.5)
    assert np.array_equal(y1[0].view(np.uint32), y[1].view(np.uint32))


# ---- IQ3_XXS (18), IQ2_S (22) gate/up and Q2_0 (42) down ----
@pytest.mark.parametrize("ty", [18, 22, 42])
def test_small_formats_pinned_to_reference(pkg, oracle, reference, ty):
    """Dequantisation and the Q8-A row dot of the restatement against the reference's own code
    (src/q4_quant.c:177-188,290-322,424-452; src/q4_cpuexp.c:814-852,895-931,1113-1145) on seeded
    blocks, bit for bit; the integer parts against the dequantised weights."""
    if reference is None:
        pytest.skip("reference CPU path not built here")
    rng = np.random.default_rng(3000 + ty)
    n = 1024
    rows = np.stack([pkg.synth.blocks_of(rng, ty, pkg.synth.row_bytes(ty, n)) for _ in range(5)])
    x = rng.standard_normal(n).astype(np.float32)
    x[64:96] = 0.0
    xq = oracle.quant8(x)
    for row in rows:
        a, b = oracle.dequant_row_x(ty, row, n), reference.dequant_row_t(ty, row, n)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
        got = oracle.dot8_t(ty, row, xq, n)
        want = reference.dot8_t(ty, row, xq, n)
        assert np.float32(got).view(np.uint32) == np.float32(want).view(np.uint32)
    # integer parts: a block with d = 1.0 dequantises to multiples of the sub-scale step
    I = oracle.group_idot_x(ty, rows[0], xq, n)
    assert I.shape == (n // 32,) and np.abs(I).max() > 0


@pytest.mark.parametrize("gu,dn", [(18, 42), (22, 21), (21, 42), (22, 42)])
def test_expert_job_small_format_mixes_match_reference(pkg, oracle, reference, gu, dn):
    if reference is None:
        pytest.skip("reference CPU path not built here")
    H, F, k = 512, 256, 3
    rng = np.random.default_rng(gu * 100 + dn)
    packs = pkg.synth.expert_packs_typed(rng, k, H, F, gu, dn)
    x = rng.standard_normal(H).astype(np.float32)
    wts = rng.random(k).astype(np.float32)
    reference.set_gu_type(gu)
    reference.set_down_type(dn)
    try:
        want = reference.expert_job(list(packs), np.arange(k, dtype=np.int32), wts, x, H, F)
    finally:
        reference.set_gu_type(21)
        reference.set_down_type(21)
    got = oracle.expert_job_t(list(packs), wts, x, H, F, dn, gu)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 2e-6
