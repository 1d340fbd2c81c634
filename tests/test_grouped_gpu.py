"""The many-token path (prefill chunks, verify windows, batches): routing,
assignment, grouped IQ3_S x int8 product, combine -- against the CPU oracle and
with the fixtures of the reference's own tests."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

IQ3_S = 21


def _rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b), 1e-30))


def test_route_pf_matches_host_softmax_topk(dev, oracle):
    rng = np.random.default_rng(1)
    n_tok, n_exp, topk = 17, 512, 10
    logits = rng.standard_normal((n_tok, n_exp)).astype(np.float32)
    logits[3, 100] = logits[3, 7]                      # planted tie
    d_ids, d_w = dev.malloc(n_tok * topk * 4), dev.malloc(n_tok * topk * 4)
    assert dev.lib.q4_hip_route_pf(dev.upload(logits), d_ids, d_w, n_tok, n_exp, topk)
    ids = dev.download(d_ids, (n_tok, topk), np.int32)
    w = dev.download(d_w, (n_tok, topk), np.float32)
    for t in range(n_tok):
        i0, w0 = oracle.topk(oracle.softmax(logits[t]), topk, True)
        assert ids[t].tolist() == i0.tolist()
        assert (np.abs(w[t] - w0) <= 1e-6 * (1 + np.abs(w0))).all()   # src/q4_test.c:1927-2145
    assert not dev.lib.q4_hip_route_pf(dev.upload(logits), d_ids, d_w, n_tok, n_exp, 65)
    assert not dev.lib.q4_hip_route_pf(dev.upload(logits), d_ids, d_w, n_tok, n_exp, 0)


@pytest.mark.parametrize("n_tok", [1, 4, 8, 9, 37, 64, 256])
def test_one_launch_routing_is_the_three_launches_bit_for_bit(dev, n_tok):
    """q4_cuda_route_small (norm + router product + top-k in one launch, a counter per group of eight
    tokens) against q4_hip_grouped_rms_n + q4_hip_gemv_dd_n + q4_hip_route_pf on the same rows, twice in
    a row (the counters must be back at zero); a batch beyond its limit is refused with nothing queued."""
    lib = dev.lib
    rng = np.random.default_rng(100 + n_tok)
    n_exp, topk, n = 512, 10, 2048
    x = (rng.standard_normal((n_tok, n)) * rng.uniform(0.1, 30.0, (n_tok, 1))).astype(np.float32)
    nw = rng.uniform(0.5, 1.5, n).astype(np.float32)
    router = (rng.standard_normal((n_exp, n)) * 0.02).astype(np.float32)
    d_x, d_nw, d_r = dev.upload(x), dev.upload(nw), dev.upload(router)
    d_xn0, d_lg0 = dev.malloc(n_tok * n * 4), dev.malloc(n_tok * n_exp * 4)
    d_i0, d_w0 = dev.malloc(n_tok * topk * 4), dev.malloc(n_tok * topk * 4)
    assert lib.q4_hip_grouped_rms_n(d_x, d_nw, d_xn0, n, 1, 1e-6, n_tok)
    assert lib.q4_hip_gemv_dd_n(0, d_r, n_exp, n, d_xn0, d_lg0, 1.0, n_tok)
    assert lib.q4_hip_route_pf(d_lg0, d_i0, d_w0, n_tok, n_exp, topk)
    ref = (dev.download(d_xn0, (n_tok, n), np.uint32), dev.download(d_lg0, (n_tok, n_exp), np.uint32),
           dev.download(d_i0, (n_tok, topk), np.int32), dev.download(d_w0, (n_tok, topk), np.uint32))
    for nw_ptr in (d_nw, None):
        if nw_ptr is None:
            assert lib.q4_hip_grouped_rms_n(d_x, None, d_xn0, n, 1, 1e-6, n_tok)
            assert lib.q4_hip_gemv_dd_n(0, d_r, n_exp, n, d_xn0, d_lg0, 1.0, n_tok)
            assert lib.q4_hip_route_pf(d_lg0, d_i0, d_w0, n_tok, n_exp, topk)
            ref = (dev.download(d_xn0, (n_tok, n), np.uint32), dev.download(d_lg0, (n_tok, n_exp), np.uint32),
                   dev.download(d_i0, (n_tok, topk), np.int32), dev.download(d_w0, (n_tok, topk), np.uint32))
        for rep in range(2):
            d_xn, d_lg = dev.malloc(n_tok * n * 4), dev.malloc(n_tok * n_exp * 4)
            d_i, d_w = dev.malloc(n_tok * topk * 4), dev.malloc(n_tok * topk * 4)
            assert lib.q4_cuda_route_small(d_x, nw_ptr, 1e-6, d_r, n_exp, topk, n, n_tok, d_xn, d_lg, d_i, d_w)
            got = (dev.download(d_xn, (n_tok, n), np.uint32), dev.download(d_lg, (n_tok, n_exp), np.uint32),
                   dev.download(d_i, (n_tok, topk), np.int32), dev.download(d_w, (n_tok, topk), np.uint32))
            for a, b, what in zip(got, ref, ("xn", "logits", "ids", "weights")):
                assert (a == b).all(), (what, rep)
    assert not lib.q4_cuda_route_small(d_x, d_nw, 1e-6, d_r, n_exp, topk, n, 257, d_xn, d_lg, d_i, d_w)
    assert not lib.q4_cuda_route_small(d_x, d_nw, 1e-6, d_r, n_exp, topk, 1024, n_tok, d_xn, d_lg, d_i, d_w)
    assert lib.q4_cuda_device_error() == 0


def test_assign_pf_invariants(dev):
    """17 tokens in groups of 8 (src/q4_test.c:1927-2145): every row placed once,
    back-map consistent, rows of an expert contiguous and hole-free."""
    rng = np.random.default_rng(2)
    n_tok, n_exp, topk, gsz = 17, 64, 6, 8
    ids = np.stack([rng.choice(n_exp, topk, replace=False) for _ in range(n_tok)]).astype(np.int32)
    ids[5, 2] = -1                                      # poisoned picks are skipped
    ids[9, 0] = n_exp + 3
    wts = rng.random((n_tok, topk)).astype(np.float32)
    n_g = (n_tok + gsz - 1) // gsz
    d = {k: dev.malloc(4 * max(n_g * gsz * topk, n_g * 512)) for k in
         ("atok", "rsrc", "rw", "stg", "stgn", "ek")}
    assert dev.lib.q4_hip_assign_pf(dev.upload(ids), dev.upload(wts), d["atok"], d["rsrc"], d["rw"],
                                    d["stg"], d["stgn"], d["ek"], gsz, topk, n_exp, n_tok)
    atok = dev.download(d["atok"], (n_g, gsz * topk), np.int32)
    rsrc = dev.download(d["rsrc"], (n_tok, topk), np.int32)
    rw = dev.download(d["rw"], (n_tok, topk), np.float32)
    stg = dev.download(d["stg"], (n_g, 512), np.int32)
    stgn = dev.download(d["stgn"], (n_g,), np.uint32)
    ek = dev.download(d["ek"], (n_g, 512), np.uint32)
    for g in range(n_g):
        t0, t1 = g * gsz, min(n_tok, (g + 1) * gsz)
        valid = [(t, k) for t in range(t0, t1) for k in range(topk) if 0 <= ids[t, k] < n_exp]
        counts = np.bincount([ids[t, k] for t, k in valid], minlength=n_exp)
        assert np.array_equal(ek[g, :n_exp], counts)
        used = np.nonzero(counts)[0]
        assert stgn[g] == used.size and stg[g, :used.size].tolist() == used.tolist()
        base = np.concatenate([[0], np.cumsum(counts)])
        seen = set()
        for t, k in valid:
            p = rsrc[t, k]
            e = ids[t, k]
            assert base[e] <= p < base[e + 1]           # inside its expert's range
            assert atok[g, p] == t and p not in seen    # back-map, no duplicate
            seen.add(p)
            assert rw[t, k] == wts[t, k]
        assert seen == set(range(len(valid)))           # hole-free
        # rows of one expert keep (token, pick) order
        for e in used:
            toks = atok[g, base[e]:base[e + 1]]
            assert (np.diff(toks) >= 0).all()
    assert rsrc[5, 2] == -1 and rw[5, 2] == 0 and rsrc[9, 0] == -1


@pytest.mark.parametrize("wr,wc,tc", [(1280, 2560, 0), (2560, 512, 0), (1024, 2048, 0), (64, 256, 0),
                                        (32, 1024, 0), (1280, 2560, 1), (2560, 512, 1), (1024, 2048, 1),
                                        (128, 256, 1)])
def test_grouped_product_reference_fixture(dev, pkg, oracle, wr, wc, tc):
    """The reference's grouped-GEMM fixture (src/q4_test.c:206-307): 8 experts with
    ragged bounds {100,0,1,40,60,30,50,19}, 300 rows gathered by ids[r]=(r*37+e*11)%320,
    xorshift weight bytes with block scales from {0x2a66,0x2e66,0x30a3}, x in steps of
    .025.  Checked against the fp64 dequantised dot (the reference's bound, rel-L2 <
    1e-2) and, much tighter, against the CPU path's int8 dot on the same rows.  tc = 0
    runs the CUDA-core kernel, tc = 1 the tensor-core kernel (100 rows = two passes of 64,
    1 row = the smallest MMA tile)."""
    assert dev.lib.q4_cuda_mmq_tc_mode(tc)
    try:
        _grouped_fixture(dev, pkg, oracle, wr, wc)
    finally:
        assert dev.lib.q4_cuda_mmq_tc_mode(-1)


def _grouped_fixture(dev, pkg, oracle, wr, wc):
    n_exp, rows, nsrc = 8, 300, 320
    per = [100, 0, 1, 40, 60, 30, 50, 19]
    bounds = np.concatenate([[0], np.cumsum(per)]).astype(np.int32)
    ids = np.zeros(rows, np.int32)
    for r in range(rows):
        e = int(np.searchsorted(bounds, r, side="right") - 1)
        ids[r] = (r * 37 + e * 11) % nsrc
    rb = wc // 256 * 110
    eb = wr * rb
    rng = np.random.default_rng(88172645463325252 % (2 ** 32) + wr)
    w = rng.integers(0, 256, size=(n_exp, wr, wc // 256, 110), dtype=np.uint8)
    ds = np.array([0x2a66, 0x2e66, 0x30a3], np.uint16)
    e_i, r_i, b_i = np.meshgrid(np.arange(n_exp), np.arange(wr), np.arange(wc // 256), indexing="ij")
    w[..., 0:2] = ds[(e_i + r_i + b_i) % 3].view(np.uint8).reshape(n_exp, wr, wc // 256, 2)
    w = w.reshape(n_exp, eb)
    x = ((rng.integers(0, 41, size=(nsrc, wc)) - 20) * 0.025).astype(np.float32)
    lib = dev.lib
    d_w = dev.upload(w)
    d_xq = dev.malloc(lib.q4_mmq_q8_bytes(rows, wc))
    d_dst = dev.malloc(rows * wr * 4)
    assert lib.q4_mmq_supported(IQ3_S, wr)
    assert lib.q4_mmq_quantize(dev.upload(x), dev.upload(ids), d_xq, IQ3_S, wc, rows)
    assert lib.q4_mmq_mul_id(d_w, IQ3_S, wr, wc, eb, n_exp, d_xq, dev.upload(bounds), max(per), rows,
                             d_dst, wr)
    got = dev.download(d_dst, (rows, wr), np.float32)
    num = den = 0.0
    num8 = den8 = 0.0
    check_rows = list(range(0, rows, 7)) + [100, 101, 299]
    for r in check_rows:
        e = int(np.searchsorted(bounds, r, side="right") - 1)
        xr = x[ids[r]]
        xq = oracle.quant8(xr)
        for j in range(0, wr, max(1, wr // 16)):
            row = w[e][j * rb:(j + 1) * rb]
            acc = float(np.dot(oracle.dequant_row(row, wc).astype(np.float64), xr))
            num += (acc - got[r, j]) ** 2
            den += acc ** 2
            a8 = oracle.dot8(row, xq, wc)
            num8 += (a8 - got[r, j]) ** 2
            den8 += a8 ** 2
    assert np.sqrt(num / den) < 1e-2
    assert np.sqrt(num8 / den8) < 1e-5
    # rows of the empty expert's neighbours are untouched by it; unsupported shapes refuse
    assert not lib.q4_mmq_mul_id(d_w, 12, wr, wc, eb, n_exp, d_xq, dev.upload(bounds), 100, rows, d_dst, wr)
    assert not lib.q4_mmq_mul_id(d_w, IQ3_S, wr, wc, eb, n_exp, d_xq, dev.upload(bounds), 100, rows, d_dst, wr - 1)


def test_tensor_core_integer_parts_exact(dev):
    """With unit scales the float result IS the integer sum: block scale d = 1, activations
    integer-valued with a 127 in every group (so q = x and the group scale is 1), K = 256 so
    every partial sum stays below 2^24.  The tensor-core product must then equal
    sum_g (1 + 2 s_g) * sum_k w_k x_k computed in integers, exactly."""
    rng = np.random.default_rng(11)
    wr, wc, n_exp = 256, 256, 3
    per = [70, 5, 17]
    rows = sum(per)
    bounds = np.concatenate([[0], np.cumsum(per)]).astype(np.int32)
    w = rng.integers(0, 256, size=(n_exp, wr, 110), dtype=np.uint8)
    w[..., 0:2] = np.array([0x3c00], np.uint16).view(np.uint8)          # d = 1.0
    x = rng.integers(-127, 128, size=(rows, wc)).astype(np.float32)
    x[:, ::32] = 127.0
    lib = dev.lib
    d_xq = dev.malloc(lib.q4_mmq_q8_bytes(rows, wc))
    d_dst = dev.malloc(rows * wr * 4)
    assert lib.q4_mmq_quantize(dev.upload(x), None, d_xq, IQ3_S, wc, rows)
    assert lib.q4_cuda_mmq_tc_mode(1)
    try:
        assert lib.q4_mmq_mul_id(dev.upload(w.reshape(n_exp, -1)), IQ3_S, wr, wc, wr * 110, n_exp, d_xq,
                                 dev.upload(bounds), max(per), rows, d_dst, wr)
    finally:
        assert lib.q4_cuda_mmq_tc_mode(-1)
    got = dev.download(d_dst, (rows, wr), np.float32)
    # integer model of the block (src/q4_quant.c:397-409): the library's own dequantiser
    # gives d * ls * sign * grid, integer-valued here
    d_deq = dev.malloc(n_exp * wr * wc * 4)
    assert lib.q4_cuda_iq3s_dequant(dev.upload(w.reshape(-1)), n_exp * wr, wc, d_deq)
    wi = dev.download(d_deq, (n_exp, wr, wc), np.float32).astype(np.int64)
    xi = x.astype(np.int64)
    for e in range(n_exp):
        want = xi[bounds[e]:bounds[e + 1]] @ wi[e].T
        assert np.abs(want).max() < 2 ** 24
        assert np.array_equal(got[bounds[e]:bounds[e + 1]].astype(np.int64), want)
        assert np.array_equal(got[bounds[e]:bounds[e + 1]], want.astype(np.float32))
    assert lib.q4_cuda_device_error() == 0


def test_verify_window_matches_single_token_path(dev, pkg, oracle):
    """4 tokens with 3/5/7/9 picks over 16 slots (src/q4_test.c:2527-2619)."""
    H, F, n_slots = 2048, 512, 16
    rng = np.random.default_rng(5)
    packs = pkg.synth.expert_packs(rng, n_slots, H, F)
    layer = pkg.MoeLayer(dev, packs, None, np.zeros((n_slots, H), np.float32), None, H, F, 1, arena=1)
    lib = dev.lib
    try:
        n_tok, counts = 4, [3, 5, 7, 9]
        xs = rng.standard_normal((n_tok, H)).astype(np.float32)
        es = np.full((n_tok, 64), -7, np.int32)
        ew = np.zeros((n_tok, 64), np.float32)
        for t, c in enumerate(counts):
            es[t, :c] = rng.choice(n_slots, c, replace=False)
            ew[t, :c] = rng.random(c).astype(np.float32)
        d_y = dev.malloc(n_tok * H * 4)
        assert lib.q4_hip_fill(d_y, 0.0, n_tok * H)
        assert lib.q4_hip_moe_win_ok(IQ3_S, IQ3_S, IQ3_S, H, F, n_tok)
        assert lib.q4_hip_moe_exec_win(layer.base, layer.stride, dev.upload(es), dev.upload(ew),
                                       dev.upload(np.array(counts, np.int32)), n_tok, IQ3_S, layer.og,
                                       IQ3_S, layer.ou, IQ3_S, layer.od, dev.upload(xs), None, d_y,
                                       F, H, H)
        y = dev.download(d_y, (n_tok, H), np.float32)
        for t, c in enumerate(counts):
            y1, _ = layer.exec_experts(xs[t], es[t, :c], ew[t, :c])
            assert _rel(y[t], y1) < 1e-5                        # same integers, same row dots
            y0 = oracle.expert_job([packs[i] for i in es[t, :c]], ew[t, :c], xs[t], H, F)
            assert _rel(y[t], y0) <= 1e-3
        assert not lib.q4_hip_moe_win_ok(IQ3_S, IQ3_S, IQ3_S, H, F, 9)
        assert not lib.q4_hip_moe_win_ok(IQ3_S, 20, IQ3_S, H, F, 4)
    finally:
        lib.q4_cuda_mmq_tc_mode(-1)
        layer.close()


@pytest.mark.parametrize("n_tok,n_expert,topk,tiled", [(4, 64, 10, True), (4, 64, 10, False),
                                                         (1, 32, 4, True), (33, 48, 6, True)])
def test_layer_n_matches_oracle_per_token(dev, pkg, oracle, n_tok, n_expert, topk, tiled):
    H, F = 2048, 512
    L = pkg.synth.layer(40 + n_tok, n_expert, H, F)
    xs = pkg.synth.hidden(41, n_tok, H)
    lib = dev.lib
    lib.q4_cuda_set_tiled_default(1 if tiled else 0)
    try:
        layer = pkg.MoeLayer(dev, L["experts"], L["shared"], L["router"], L["norm_w"], H, F, topk, arena=1)
    finally:
        lib.q4_cuda_set_tiled_default(1)
    # the CUDA-core kernels first: with them a token's result does not depend on the batch
    assert lib.q4_cuda_mmq_tc_mode(0)
    try:
        ws = lib.q4_cuda_moe_layer_n_ws_bytes(n_tok, topk, n_expert, H, F)
        d_ws = dev.malloc(ws)
        d_y = dev.malloc(n_tok * H * 4)
        d_ids, d_w = dev.malloc(n_tok * topk * 4), dev.malloc(n_tok * topk * 4)
        assert lib.q4_cuda_moe_layer_n(layer.base, layer.stride, layer.og, layer.ou, layer.od,
                                       layer.shared_slot, dev.upload(xs), layer.d_norm, 1e-6,
                                       layer.d_router, n_expert, topk, H, F, n_tok, d_y, d_ids, d_w,
                                       d_ws, ws)
        y = dev.download(d_y, (n_tok, H), np.float32)
        ids = dev.download(d_ids, (n_tok, topk), np.int32)
        for t in range(n_tok):
            y0, ids0, w0, _ = oracle.moe_layer(xs[t], L["norm_w"], 1e-6, L["router"], topk,
                                               L["experts"], L["shared"], H, F)
            assert ids[t].tolist() == ids0.tolist()
            assert _rel(y[t], y0) <= 1e-3
        # batch invariance: a token's row does not depend on who else is in the batch
        if n_tok > 1:
            d_y1 = dev.malloc(H * 4)
            assert lib.q4_cuda_moe_layer_n(layer.base, layer.stride, layer.og, layer.ou, layer.od,
                                           layer.shared_slot, dev.upload(xs[2:3]), layer.d_norm, 1e-6,
                                           layer.d_router, n_expert, topk, H, F, 1, d_y1, None, None,
                                           d_ws, ws)
            y1 = dev.download(d_y1, (H,), np.float32)
            assert np.array_equal(y1.view(np.uint32), y[2].view(np.uint32))
        # the streaming kernel (tiled arenas) and the general kernel do the same sums
        assert lib.q4_cuda_mmq_tc_mode(2)
        try:
            assert lib.q4_cuda_moe_layer_n(layer.base, layer.stride, layer.og, layer.ou, layer.od,
                                           layer.shared_slot, dev.upload(xs), layer.d_norm, 1e-6,
                                           layer.d_router, n_expert, topk, H, F, n_tok, d_y, d_ids, d_w,
                                           d_ws, ws)
        finally:
            assert lib.q4_cuda_mmq_tc_mode(-1)
        y2 = dev.download(d_y, (n_tok, H), np.float32)
        assert np.array_equal(y2.view(np.uint32), y.view(np.uint32))
        # the tensor-core kernel, alone (1) or taking the entries with many rows (-1, the
        # default), agrees to rounding: another order of the same products
        for mode in (1, -1):
            assert lib.q4_cuda_mmq_tc_mode(mode)
            try:
                assert lib.q4_cuda_moe_layer_n(layer.base, layer.stride, layer.og, layer.ou, layer.od,
                                               layer.shared_slot, dev.upload(xs), layer.d_norm, 1e-6,
                                               layer.d_router, n_expert, topk, H, F, n_tok, d_y, d_ids,
                                               d_w, d_ws, ws)
            finally:
                assert lib.q4_cuda_mmq_tc_mode(-1)
            y3 = dev.download(d_y, (n_tok, H), np.float32)
            for t in range(n_tok):
                assert _rel(y3[t], y[t]) < 1e-5
        assert lib.q4_cuda_device_error() == 0
        assert not lib.q4_cuda_moe_layer_n(layer.base, layer.stride, layer.og, layer.ou, layer.od,
                                           layer.shared_slot, dev.upload(xs), layer.d_norm, 1e-6,
                                           layer.d_router, n_expert, topk, H, F, n_tok, d_y, d_ids,
                                           d_w, d_ws, ws - 1)
    finally:
        lib.q4_cuda_mmq_tc_mode(-1)
        layer.close()


@pytest.mark.parametrize("per", [[0, 0, 0, 0], [2100, 11, 12, 5], [64, 0, 65, 1], [3, 0, 0, 129]])
def test_grouped_product_edge_row_counts(dev, pkg, oracle, per):
    """Row counts at the edges of the kernels' ranges, on a tiled arena: no rows at all (nothing may
    be written), 11 / 12 rows either side of the tensor-core threshold next to an expert with
    2100 rows (one call, two kernels), 64 / 65 (one pass / two passes), 129 (three passes, the last
    with one row).
    Every kernel choice must agree with the CPU path's int8 dot."""
    H, F, n_exp = 2048, 512, 4
    rng = np.random.default_rng(7 + sum(per))
    packs = pkg.synth.expert_packs(rng, n_exp, H, F)
    layer = pkg.MoeLayer(dev, packs, None, np.zeros((n_exp, H), np.float32), None, H, F, 1, arena=1)
    lib = dev.lib
    try:
        rows = sum(per)
        bounds = np.concatenate([[0], np.cumsum(per)]).astype(np.int32)
        nr = max(rows, 1)
        x = rng.standard_normal((nr, H)).astype(np.float32)
        d_xq = dev.malloc(lib.q4_mmq_q8_bytes(nr, H))
        d_dst = dev.malloc(nr * 2 * F * 4)
        sentinel = np.full((nr, 2 * F), 7.5, np.float32)
        assert lib.q4_mmq_quantize(dev.upload(x), None, d_xq, IQ3_S, H, nr)
        rb = pkg.synth.iq3s_row_bytes(H)
        for mode in (-1, 0, 1, 2):
            dev.write(d_dst, sentinel)
            assert lib.q4_cuda_mmq_tc_mode(mode)
            try:
                ok = lib.q4_mmq_mul_id(layer.base + layer.og, IQ3_S, 2 * F, H, layer.stride, n_exp, d_xq,
                                       dev.upload(bounds), max(per), nr if rows else 1, d_dst, 2 * F)
            finally:
                assert lib.q4_cuda_mmq_tc_mode(-1)
            assert ok
            got = dev.download(d_dst, (nr, 2 * F), np.float32)
            if rows == 0:
                assert np.array_equal(got, sentinel)        # no rows: nothing written
                continue
            for r in sorted({0, rows - 1, rows // 2, min(rows - 1, 64), min(rows - 1, 11), max(0, rows - 6),
                             max(0, rows - 30), max(0, rows - 40)}):
                e = int(np.searchsorted(bounds, r, side="right") - 1)
                xq = oracle.quant8(x[r])
                for j in (0, 1, 511, 512, 1023):
                    row = packs[e][j * rb:(j + 1) * rb]
                    want = oracle.dot8(row, xq, H)
                    # fp32 sums of the same terms in different orders (64 group terms on the CUDA cores,
                    # 16-term steps inside the tensor cores): a few units in the last place of the partial
                    # sums, whose size is that of a random walk over the terms, not of the (possibly
                    # cancelling) result
                    terms = oracle.dequant_row(row, H).astype(np.float64) * \
                        (np.repeat(np.asarray(xq["d"], np.float64), 32) * np.asarray(xq["q"], np.float64).ravel())
                    walk = float(np.sqrt((terms * terms).sum()))
                    assert abs(got[r, j] - want) <= 1e-5 * abs(want) + 5e-6 * walk + 2e-5, \
                        (mode, r, j, got[r, j], want, walk)
        assert lib.q4_cuda_device_error() == 0
    finally:
        layer.close()


def test_tensor_core_product_with_an_outlier_channel(dev, pkg, oracle):
    """The tensor-core product carries an activation row as two fp16 planes scaled by one power
    of two per row, so its error is small against the row's largest group, not against every
    group.  Rows with one group 1000 times the rest (hidden states have such channels) must
    still agree with the CUDA-core kernels, which form the exact integer sums, and with the CPU
    int8 dot."""
    H, F, n_exp, rows = 2048, 512, 2, 40
    rng = np.random.default_rng(31)
    packs = pkg.synth.expert_packs(rng, n_exp, H, F)
    layer = pkg.MoeLayer(dev, packs, None, np.zeros((n_exp, H), np.float32), None, H, F, 1, arena=1)
    lib = dev.lib
    try:
        x = rng.standard_normal((rows, H)).astype(np.float32)
        x[:, 96:128] *= 1000.0                                   # one 32-group per row
        bounds = np.array([0, rows // 2, rows], np.int32)
        d_xq = dev.malloc(lib.q4_mmq_q8_bytes(rows, H))
        d_dst = dev.malloc(rows * 2 * F * 4)
        assert lib.q4_mmq_quantize(dev.upload(x), None, d_xq, IQ3_S, H, rows)
        out = {}
        for mode in (0, 1):
            assert lib.q4_cuda_mmq_tc_mode(mode)
            try:
                assert lib.q4_mmq_mul_id(layer.base + layer.og, IQ3_S, 2 * F, H, layer.stride, n_exp, d_xq,
                                         dev.upload(bounds), rows // 2, rows, d_dst, 2 * F)
            finally:
                assert lib.q4_cuda_mmq_tc_mode(-1)
            out[mode] = dev.download(d_dst, (rows, 2 * F), np.float32)
        worst = max(_rel(out[1][r], out[0][r]) for r in range(rows))
        print("outlier rows: tensor-core vs CUDA-core product, worst rel-L2 %.3g" % worst)
        assert worst < 1e-4
        rb = pkg.synth.iq3s_row_bytes(H)
        for r in (0, rows - 1):
            xq = oracle.quant8(x[r])
            e = 0 if r < rows // 2 else 1
            want = np.array([oracle.dot8(packs[e][j * rb:(j + 1) * rb], xq, H) for j in range(0, 2 * F, 37)])
            assert _rel(out[1][r, ::37], want) <= 1e-3
        assert lib.q4_cuda_device_error() == 0
    finally:
        lib.q4_cuda_mmq_tc_mode(-1)
        layer.close()


def test_q8_compat_quantiser_is_ggml_q8_1(dev, pkg, oracle):
    """q4_cuda_mmq_q8_compat(1): the row buffers are filled with ggml's q8_1 rounding (what the
    reference's grouped device product uses, restated as q4o_quant8_mmq) instead of Q8-A: q and d bit for
    bit, on rows with exact halves planted; the grouped product on those rows against the oracle's
    dot in the grouped order."""
    import ctypes as C
    lib = dev.lib
    rng = np.random.default_rng(33)
    rows, K, R = 6, 512, 64
    x = rng.standard_normal((rows, K)).astype(np.float32)
    x[0, :32] = 0.0
    x[1, 32:64] = np.array([127.0, 0.5, -0.5, 2.5, -2.5, 1.5] + [0.25] * 26, np.float32)   # d_inv = 1: halves
    w = pkg.synth.iq3s_blocks(rng, R * K // 256).reshape(R, -1)
    d_x = dev.upload(x)
    d_xq = dev.malloc(lib.q4_mmq_q8_bytes(rows, K))
    d_dst = dev.malloc(rows * R * 4)
    bounds = dev.upload(np.array([0, rows], np.int32))
    got = {}
    try:
        for mode in (1, 0):
            lib.q4_cuda_mmq_q8_compat(mode)
            assert lib.q4_mmq_quantize(d_x, None, d_xq, IQ3_S, K, rows)
            pq, pd, ps = C.c_void_p(), C.c_void_p(), C.c_void_p()
            assert lib.q4_cuda_mmq_q8_sections(d_xq, rows, K, C.byref(pq), C.byref(pd), C.byref(ps))
            q = dev.download(pq.value, (rows, K), np.int8)
            d = dev.download(pd.value, (rows, K // 32), np.float32)
            s = dev.download(ps.value, (rows, K // 32), np.int32)
            assert np.array_equal(s, q.astype(np.int32).reshape(rows, K // 32, 32).sum(2))
            assert lib.q4_cuda_mmq_tc_mode(0)
            assert lib.q4_mmq_mul_id(dev.upload(w), IQ3_S, R, K, 0, 1, d_xq, bounds, rows, rows, d_dst, R)
            got[mode] = (q, d, dev.download(d_dst, (rows, R), np.float32))
    finally:
        lib.q4_cuda_mmq_q8_compat(0)
        lib.q4_cuda_mmq_tc_mode(-1)
    qc, dc, yc = got[1]
    qa, da, _ = got[0]
    for r in range(rows):
        q0, d0 = oracle.quant8_mmq(x[r])
        assert np.array_equal(qc[r], q0) and np.array_equal(dc[r].view(np.uint32), d0.view(np.uint32)), r
        xa = oracle.quant8(x[r])
        assert np.array_equal(qa[r], xa["q"].ravel()) and np.array_equal(da[r].view(np.uint32), xa["d"].view(np.uint32))
        want = np.array([oracle.dot_mmq(w[i], q0, d0, K) for i in range(R)], np.float64)
        assert np.linalg.norm(yc[r] - want) / np.linalg.norm(want) < 1e-5, r
    assert qc[1, 33] == 1 and qa[1, 33] == 0 and qc[1, 34] == -1 and qa[1, 34] == 0      # 0.5: away / to even
    assert qc[1, 35] == 3 and qa[1, 35] == 2 and qc[1, 37] == 2 and qa[1, 37] == 2      # 2.5, 1.5
    assert not qc[0, :32].any() and dc[0, 0] == 0
