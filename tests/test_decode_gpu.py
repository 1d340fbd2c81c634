"""Parity of the CUDA decode path with the CPU oracle, through the C ABI.

Integer stages (dequantisation, activation quantiser, per-32-group integer dots)
are compared bit for bit; floating-point outputs within rel-L2 <= 1e-3 (the
tolerance the task states for expert outputs), routing ids exactly."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(__file__), "golden", "iq3s_moe_small.npz")
REL_TOL = 1e-3


def _bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def _rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b), 1e-30))


def test_dequant_bit_exact(dev, pkg, oracle):
    rng = np.random.default_rng(1)
    rows, cols = 24, 1024
    w = pkg.synth.iq3s_blocks(rng, rows * cols // 256).reshape(-1)
    d_w = dev.upload(w)
    d_o = dev.malloc(rows * cols * 4)
    assert dev.lib.q4_cuda_iq3s_dequant(d_w, rows, cols, d_o)
    got = dev.download(d_o, (rows, cols), np.float32)
    rb = cols // 256 * 110
    for r in range(rows):
        exp = oracle.dequant_row(w[r * rb:(r + 1) * rb], cols)
        assert np.array_equal(_bits(got[r]), _bits(exp))


@pytest.mark.parametrize("n", [32, 2048, 16384])
def test_quant8_bit_exact(dev, oracle, n):
    rng = np.random.default_rng(n)
    x = (rng.standard_normal(n) * rng.uniform(1e-3, 1e3, n)).astype(np.float32)
    x[:32] = 0.0
    if n >= 64:
        x[32:37] = [127.0, 0.5, 1.5, 2.5, -0.5]   # exact ties: round half to even
        x[37:64] = 0.0
    d_x = dev.upload(x)
    d_q, d_d, d_b = dev.malloc(n), dev.malloc(n // 8), dev.malloc(n // 8)
    assert dev.lib.q4_cuda_quant8(d_x, n, d_q, d_d, d_b)
    q = dev.download(d_q, (n // 32, 32), np.int8)
    d = dev.download(d_d, (n // 32,), np.float32)
    bs = dev.download(d_b, (n // 32,), np.int32)
    ref = oracle.quant8(x)
    assert np.array_equal(q, ref["q"])
    assert np.array_equal(_bits(d), _bits(ref["d"]))
    assert np.array_equal(bs, ref["bs"])


def test_quant8_rejects_ragged(dev):
    assert not dev.lib.q4_cuda_quant8(dev.malloc(256), 33, dev.malloc(64), dev.malloc(64), None)
    assert not dev.lib.q4_cuda_quant8(dev.malloc(256), 0, dev.malloc(64), dev.malloc(64), None)


def test_group_integer_dots_bit_exact(dev, pkg, oracle):
    rng = np.random.default_rng(2)
    rows, cols = 40, 2048
    w = pkg.synth.iq3s_blocks(rng, rows * cols // 256).reshape(-1)
    x = rng.standard_normal(cols).astype(np.float32)
    xq = oracle.quant8(x)
    d_w = dev.upload(w)
    d_q = dev.upload(np.ascontiguousarray(xq["q"]))
    d_I = dev.malloc(rows * cols // 32 * 4)
    assert dev.lib.q4_cuda_iq3s_idot(d_w, rows, cols, d_q, d_I)
    got = dev.download(d_I, (rows, cols // 32), np.int32)
    rb = cols // 256 * 110
    for r in range(rows):
        assert np.array_equal(got[r], oracle.group_idot(w[r * rb:(r + 1) * rb], xq, cols))


def test_kat_zero_block(dev, oracle):
    # src/q4_test.c:52-58 restated for the int8 path: zero block, d = 1, x = 1
    blk = np.zeros(110, np.uint8)
    blk[0:2] = np.array([0x3c00], np.uint16).view(np.uint8)
    d_w = dev.upload(blk)
    d_o = dev.malloc(1024)
    assert dev.lib.q4_cuda_iq3s_dequant(d_w, 1, 256, d_o)
    assert dev.download(d_o, (256,), np.float32).sum() == 256.0
    xq = oracle.quant8(np.ones(256, np.float32))
    d_I = dev.malloc(32)
    assert dev.lib.q4_cuda_iq3s_idot(d_w, 1, 256, dev.upload(np.ascontiguousarray(xq["q"])), d_I)
    assert dev.download(d_I, (8,), np.int32).tolist() == [32 * 127] * 8


def test_rms_norm_bit_exact(dev, oracle):
    rng = np.random.default_rng(4)
    n, hc, ntok = 2048, 2, 3
    x = rng.standard_normal((ntok, hc, n)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal((hc, n))).astype(np.float32)
    d_x, d_w, d_y = dev.upload(x), dev.upload(w), dev.malloc(x.nbytes)
    assert dev.lib.q4_hip_grouped_rms_n(d_x, d_w, d_y, n, hc, 1e-6, ntok)
    got = dev.download(d_y, x.shape, np.float32)
    for t in range(ntok):
        for c in range(hc):
            assert np.array_equal(_bits(got[t, c]), _bits(oracle.rms_norm(x[t, c], w[c], 1e-6)))


def test_softmax_topk_ids_exact_with_ties(dev, oracle):
    rng = np.random.default_rng(6)
    n, k = 512, 10
    for trial in range(8):
        logits = rng.standard_normal(n).astype(np.float32)
        if trial % 2:
            top = np.argsort(-logits)[:3]
            logits[top[1]] = logits[top[0]]          # tie inside the top-k
            j = np.argsort(-logits)[k - 1]
            logits[(j + 17) % n] = logits[j]         # tie at the cut
        ids = np.zeros(k, np.int32)
        wts = np.zeros(k, np.float32)
        assert dev.lib.q4_hip_softmax_topk(dev.upload(logits), n, k, ids.ctypes.data, wts.ctypes.data)
        ids0, w0 = oracle.topk(oracle.softmax(logits), k, True)
        assert ids.tolist() == ids0.tolist()
        assert np.abs(wts - w0).max() <= 1e-6       # the reference's own bound (src/q4_test.c:1597-1926)
        assert abs(float(wts.sum()) - 1.0) < 1e-5
    assert not dev.lib.q4_hip_softmax_topk(dev.upload(logits), n, 0, ids.ctypes.data, wts.ctypes.data)
    assert not dev.lib.q4_hip_softmax_topk(dev.upload(logits), n, 65, ids.ctypes.data, wts.ctypes.data)


def test_router_gemv(dev, oracle):
    rng = np.random.default_rng(8)
    W = (rng.standard_normal((512, 2048)) * 0.02).astype(np.float32)
    x = rng.standard_normal(2048).astype(np.float32)
    d_y = dev.malloc(512 * 4)
    assert dev.lib.q4_hip_gemv_dd(0, dev.upload(W), 512, 2048, dev.upload(x), d_y, 1.0)
    got = dev.download(d_y, (512,), np.float32)
    assert _rel(got, oracle.gemv_f32(W, x)) < 1e-6


def test_gemv_iq3s_float_activations(dev, pkg, oracle):
    rng = np.random.default_rng(9)
    rows, cols = 64, 1024
    w = pkg.synth.iq3s_blocks(rng, rows * cols // 256).reshape(-1)
    x = rng.standard_normal(cols).astype(np.float32)
    d_y = dev.malloc(rows * 4)
    assert dev.lib.q4_hip_gemv_dd(21, dev.upload(w), rows, cols, dev.upload(x), d_y, 0.5)
    got = dev.download(d_y, (rows,), np.float32)
    rb = cols // 256 * 110
    exp = np.array([0.5 * np.dot(oracle.dequant_row(w[r * rb:(r + 1) * rb], cols).astype(np.float64), x)
                    for r in range(rows)])
    assert np.abs(got - exp).max() <= 2e-3 * (1 + np.abs(exp).max())   # src/q4_test.c:75-135


def test_golden_single_expert(dev, pkg, oracle):
    g = np.load(GOLD)
    H, F = int(g["H"]), int(g["F"])
    layer = pkg.MoeLayer(dev, g["packs"], None, np.zeros((2, H), np.float32), None, H, F, 1, arena=1)
    try:
        y, h = layer.exec_experts(g["x"], [0], [1.0])
        assert _rel(y, g["y1"]) <= REL_TOL
        y2, _ = layer.exec_experts(g["x"], [0, 1], g["wts"])
        assert _rel(y2, g["y2"]) <= REL_TOL
    finally:
        layer.close()


def test_config0_single_expert_full_shape(dev, pkg, oracle):
    """hidden 2048, intermediate 512, one token, one expert."""
    H, F = 2048, 512
    rng = np.random.default_rng(10)
    packs = pkg.synth.expert_packs(rng, 3, H, F)
    x = rng.standard_normal(H).astype(np.float32)
    layer = pkg.MoeLayer(dev, packs, None, np.zeros((3, H), np.float32), None, H, F, 1, arena=1)
    try:
        y, h = layer.exec_experts(x, [2], [1.0])
        xq = oracle.quant8(x)
        y0 = np.zeros(H, np.float32)
        h0, hq0 = oracle.expert_ffn(packs[2], xq, H, F, 1.0, y0)
        assert _rel(h[0], h0) <= 1e-5         # same integers, fp32 order differs
        assert _rel(y, y0) <= REL_TOL
        # accumulate semantics: running again without clearing doubles y
        lib = dev.lib
        slots = np.array([2], np.int32)
        w = np.array([1.0], np.float32)
        assert lib.q4_hip_moe_exec(layer.base, layer.stride, slots.ctypes.data, w.ctypes.data, 1,
                                   21, layer.og, 21, layer.ou, 21, layer.od, layer.d_x, layer.d_h,
                                   None, None, layer.d_y, F, H, H)
        y_twice = dev.download(layer.d_y, (H,), np.float32)
        assert _rel(y_twice, 2 * y0) <= REL_TOL
        # unsupported types and shapes are refused before anything is queued
        assert not lib.q4_hip_moe_exec(layer.base, layer.stride, slots.ctypes.data, w.ctypes.data, 1,
                                       20, layer.og, 21, layer.ou, 21, layer.od, layer.d_x,
                                       layer.d_h, None, None, layer.d_y, F, H, H)
        assert not lib.q4_hip_moe_exec(layer.base, layer.stride, slots.ctypes.data, w.ctypes.data, 65,
                                       21, layer.og, 21, layer.ou, 21, layer.od, layer.d_x,
                                       layer.d_h, None, None, layer.d_y, F, H, H)
        assert not lib.q4_hip_moe_tok_ok(21, 21, 21, 2048 + 32, 512)
        assert np.array_equal(dev.download(layer.d_y, (H,), np.float32), y_twice)
    finally:
        layer.close()


def test_exec_staged_and_dev_lists(dev, pkg, oracle):
    H, F = 1024, 256
    rng = np.random.default_rng(12)
    packs = pkg.synth.expert_packs(rng, 6, H, F)
    x = rng.standard_normal(H).astype(np.float32)
    layer = pkg.MoeLayer(dev, packs, None, np.zeros((6, H), np.float32), None, H, F, 1, arena=1)
    lib = dev.lib
    try:
        slots = np.array([5, 0, 3], np.int32)
        wts = np.array([0.5, 0.25, 0.25], np.float32)
        y0 = oracle.expert_job([packs[i] for i in slots], wts, x, H, F)
        dev.write(layer.d_x, x)
        # staged list (graph-replayable form)
        assert lib.q4_hip_fill(layer.d_y, 0.0, H)
        assert lib.q4_hip_moe_stage(slots.ctypes.data, wts.ctypes.data, 3)
        assert lib.q4_hip_moe_exec_staged(layer.base, layer.stride, 21, layer.og, 21, layer.ou, 21,
                                          layer.od, layer.d_x, layer.d_h, None, None, layer.d_y,
                                          F, H, H)
        assert _rel(dev.download(layer.d_y, (H,), np.float32), y0) <= REL_TOL
        # device list + device count
        d_es, d_ew = dev.upload(slots), dev.upload(wts)
        d_n = dev.upload(np.array([3], np.int32))
        assert lib.q4_hip_fill(layer.d_y, 0.0, H)
        assert lib.q4_hip_moe_exec_dev(layer.base, layer.stride, d_es, d_ew, d_n, 21, layer.og, 21,
                                       layer.ou, 21, layer.od, layer.d_x, layer.d_h, None, None,
                                       layer.d_y, F, H, H)
        y_dev = dev.download(layer.d_y, (H,), np.float32)
        assert _rel(y_dev, y0) <= REL_TOL
        # graph capture and replay with a new list
        assert lib.q4_hip_fill(layer.d_y, 0.0, H)
        assert lib.q4_hip_graph_begin() == 1
        assert lib.q4_hip_moe_exec_staged(layer.base, layer.stride, 21, layer.og, 21, layer.ou, 21,
                                          layer.od, layer.d_x, layer.d_h, None, None, layer.d_y,
                                          F, H, H)
        ex = lib.q4_hip_graph_end()
        assert ex
        slots2 = np.array([1, 2], np.int32)
        wts2 = np.array([0.75, 0.25], np.float32)
        assert lib.q4_hip_moe_stage(slots2.ctypes.data, wts2.ctypes.data, 2)
        assert lib.q4_hip_graph_launch(ex)
        y_g = dev.download(layer.d_y, (H,), np.float32)
        lib.q4_hip_graph_free(ex)
        assert _rel(y_g, oracle.expert_job([packs[1], packs[2]], wts2, x, H, F)) <= REL_TOL
    finally:
        layer.close()


def _check_layer(dev, pkg, oracle, seed, n_expert, H, F, topk, n_tok=2):
    L = pkg.synth.layer(seed, n_expert, H, F)
    xs = pkg.synth.hidden(seed + 1, n_tok, H)
    layer = pkg.MoeLayer(dev, L["experts"], L["shared"], L["router"], L["norm_w"], H, F, topk, arena=1)
    try:
        for t in range(n_tok):
            y, ids, wts = layer.decode(xs[t])
            y0, ids0, w0, xn0 = oracle.moe_layer(xs[t], L["norm_w"], 1e-6, L["router"], topk,
                                                 L["experts"], L["shared"], H, F)
            assert ids.tolist() == ids0.tolist()
            assert np.abs(wts - w0).max() <= 1e-6
            assert _rel(y, y0) <= REL_TOL
        assert dev.lib.q4_cuda_device_error() == 0
    finally:
        layer.close()


def test_moe_layer_small(dev, pkg, oracle):
    _check_layer(dev, pkg, oracle, 21, 32, 512, 256, 4)


def test_config1_moe_layer_full_shape(dev, pkg, oracle):
    """hidden 2048, intermediate 512, 512 experts top-10 + shared, one token."""
    _check_layer(dev, pkg, oracle, 22, 512, 2048, 512, 10, n_tok=2)


def test_decode_host_buffers_match_device_call(dev, pkg):
    """q4_cuda_moe_decode_host: pinned + mapped result buffer (the kernel writes y into host
    memory and raises a flag the host spins on) and an ordinary pageable buffer (copy + sync)
    both return exactly what the device-pointer call computes; repeated calls do not
    interfere (the flag carries an epoch)."""
    import ctypes
    H, F, E, K = 2048, 512, 64, 8
    L = pkg.synth.layer(91, E, H, F)
    xs = pkg.synth.hidden(92, 3, H)
    layer = pkg.MoeLayer(dev, L["experts"], L["shared"], L["router"], L["norm_w"], H, F, K, arena=2)
    lib = dev.lib
    try:
        h_x = lib.q4_hip_host_alloc_coh(H * 4)
        h_y = lib.q4_hip_host_alloc_coh(H * 4)
        assert h_x and h_y
        y_page = np.zeros(H, np.float32)
        for x in xs:
            want, _, _ = layer.decode(x)
            ctypes.memmove(h_x, x.ctypes.data, H * 4)
            ctypes.memset(h_y, 0, H * 4)
            assert lib.q4_cuda_moe_decode_host(layer.base, layer.stride, layer.og, layer.ou, layer.od,
                                               layer.shared_slot, h_x, layer.d_norm, 1e-6, layer.d_router,
                                               E, K, H, F, h_y)
            got = np.ctypeslib.as_array(ctypes.cast(h_y, ctypes.POINTER(ctypes.c_float)), (H,)).copy()
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
            assert lib.q4_cuda_moe_decode_host(layer.base, layer.stride, layer.og, layer.ou, layer.od,
                                               layer.shared_slot, x.ctypes.data, layer.d_norm, 1e-6,
                                               layer.d_router, E, K, H, F, y_page.ctypes.data)
            assert np.array_equal(y_page.view(np.uint32), want.view(np.uint32))
        # the same layer with its arguments bound once
        plan = lib.q4_cuda_decode_plan(layer.base, layer.stride, layer.og, layer.ou, layer.od,
                                       layer.shared_slot, layer.d_norm, 1e-6, layer.d_router, E, K, H, F)
        assert plan
        want, _, _ = layer.decode(xs[1])
        ctypes.memmove(h_x, xs[1].ctypes.data, H * 4)
        ctypes.memset(h_y, 0, H * 4)
        assert lib.q4_cuda_decode_plan_host(plan, h_x, h_y)
        got = np.ctypeslib.as_array(ctypes.cast(h_y, ctypes.POINTER(ctypes.c_float)), (H,)).copy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        d_y2 = dev.malloc(H * 4)
        assert lib.q4_cuda_decode_plan_dev(plan, dev.upload(xs[1]), d_y2, None, None)
        assert np.array_equal(dev.download(d_y2, (H,), np.float32).view(np.uint32), want.view(np.uint32))
        lib.q4_cuda_decode_plan_free(plan)
        assert not lib.q4_cuda_decode_plan(layer.base, layer.stride, layer.og, layer.ou, layer.od,
                                           layer.shared_slot, layer.d_norm, 1e-6, layer.d_router, E, 0, H, F)
        lib.q4_hip_host_free_coh(h_x)
        lib.q4_hip_host_free_coh(h_y)
        assert lib.q4_cuda_device_error() == 0
    finally:
        layer.close()
