"""The small device routines the engine's MoE layer code issues around the expert products
(src/q4_moe.c:1404-1435, 1853-1884, 2095-2186, 2795-2845): elementwise updates, reductions,
the shared expert's gate, the pack/final pair, the multi-segment GEMV, the per-token exec over
packed device lists, the 2..8-row GEMV on 8-bit activations and the expert gather."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
IQ3_S, F32 = 21, 0


def _rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b), 1e-30))


def _sig(v):
    return 1.0 / (1.0 + np.exp(-v.astype(np.float64)))


@pytest.mark.parametrize("n", [1, 7, 1000, 4099, 1 << 20])
def test_elementwise_updates(dev, n):
    rng = np.random.default_rng(n)
    lib = dev.lib
    y0, a, b = (rng.standard_normal(n).astype(np.float32) for _ in range(3))
    d_a, d_b = dev.upload(a), dev.upload(b)
    alpha = dev.upload(np.array([0.375], np.float32))

    def run(call, want, tol=2e-6):
        d_y = dev.upload(y0)
        assert call(d_y)
        got = dev.download(d_y, (n,), np.float32)
        np.testing.assert_allclose(got, want, rtol=tol, atol=tol)

    y64, a64, b64 = y0.astype(np.float64), a.astype(np.float64), b.astype(np.float64)
    run(lambda y: lib.q4_hip_silu(y, n), y64 * _sig(y0))
    run(lambda y: lib.q4_hip_sigmoid(y, n), _sig(y0))
    run(lambda y: lib.q4_hip_scale(y, 0.25, n), y64 * 0.25, 0)
    run(lambda y: lib.q4_hip_scale_silu(y, 0.5, n), 0.5 * y64 * _sig(0.5 * y0))
    run(lambda y: lib.q4_hip_mul(y, d_a, d_b, n), (a * b).astype(np.float64), 0)
    run(lambda y: lib.q4_hip_add(y, d_a, d_b, n), (a + b).astype(np.float64), 0)
    run(lambda y: lib.q4_hip_add(y, y, d_b, n), (y0 + b).astype(np.float64), 0)      # in place
    run(lambda y: lib.q4_hip_mul_sig(y, d_a, d_b, n), a64 * _sig(b))
    run(lambda y: lib.q4_hip_silu_mul(y, d_a, n), y64 * _sig(y0) * a64)
    run(lambda y: lib.q4_hip_axpy(y, d_a, -1.5, n), y64 - 1.5 * a64, 1e-6)
    run(lambda y: lib.q4_hip_axpy_dalpha(y, d_a, alpha, n), y64 + 0.375 * a64, 1e-6)
    assert not lib.q4_hip_silu(None, n) and not lib.q4_hip_axpy(d_a, d_b, 1.0, 0)
    lib.q4_hip_clear()
    assert lib.q4_cuda_device_error() == 0


def test_reductions_and_shared_gate(dev):
    rng = np.random.default_rng(3)
    lib = dev.lib
    n, n_tok = 2048, 5
    a, w = (rng.standard_normal(n).astype(np.float32) * 0.05 for _ in range(2))
    d_out = dev.malloc(4)
    assert lib.q4_hip_dot(dev.upload(a), dev.upload(w), d_out, n)
    dot = dev.download(d_out, (1,), np.float32)[0]
    want = float(a.astype(np.float64) @ w)
    assert abs(dot - want) <= 1e-5 * max(1.0, abs(want))
    assert lib.q4_hip_dot_sigmoid(dev.upload(a), dev.upload(w), d_out, n)
    assert abs(dev.download(d_out, (1,), np.float32)[0] - 1 / (1 + np.exp(-want))) < 1e-6
    # d_y[t] += sigmoid(w . x[t]) * sh[t]   and the unfused form   d_y[t] += sg[t] * sh[t]
    x = rng.standard_normal((n_tok, n)).astype(np.float32)
    sh, y0 = (rng.standard_normal((n_tok, n)).astype(np.float32) for _ in range(2))
    sg = _sig(x.astype(np.float64) @ w.astype(np.float64))
    want = y0 + sg[:, None] * sh
    d_y = dev.upload(y0)
    assert lib.q4_hip_sgate_axpy(d_y, dev.upload(sh), dev.upload(w), dev.upload(x), n, n_tok)
    np.testing.assert_allclose(dev.download(d_y, (n_tok, n), np.float32), want, rtol=1e-5, atol=1e-5)
    d_y = dev.upload(y0)
    assert lib.q4_hip_axpy_rows(d_y, dev.upload(sh), dev.upload(sg.astype(np.float32)), n, n_tok)
    np.testing.assert_allclose(dev.download(d_y, (n_tok, n), np.float32), want, rtol=1e-5, atol=1e-5)


def test_pack_and_final(dev):
    """Head and tail of a decode layer (src/q4_rocm.cu:15920-16024)."""
    rng = np.random.default_rng(4)
    lib = dev.lib
    H, F, hc = 2048, 512, 4
    x, sgate = (rng.standard_normal(H).astype(np.float32) * 0.05 for _ in range(2))
    sm, sm2 = (rng.standard_normal(F).astype(np.float32) for _ in range(2))
    d_y = dev.upload(rng.standard_normal(H).astype(np.float32))
    d_dot, d_flag, d_sm = dev.malloc(4), dev.upload(np.array([41], np.uint32)), dev.upload(sm)
    assert lib.q4_hip_moe_pack(d_y, dev.upload(x), dev.upload(sgate), d_dot, d_flag, H, True, d_sm,
                               dev.upload(sm2), F)
    assert not dev.download(d_y, (H,), np.float32).any()
    g = 1 / (1 + np.exp(-float(x.astype(np.float64) @ sgate)))
    assert abs(dev.download(d_dot, (1,), np.float32)[0] - g) < 1e-6
    assert dev.download(d_flag, (1,), np.uint32)[0] == 42
    np.testing.assert_allclose(dev.download(d_sm, (F,), np.float32),
                               sm.astype(np.float64) * _sig(sm) * sm2, rtol=2e-6, atol=2e-6)
    # without a gate, a counter or shared projections the call only zeroes y
    d_y2 = dev.upload(np.ones(H, np.float32))
    assert lib.q4_hip_moe_pack(d_y2, dev.upload(x), None, None, None, H, False, None, None, 0)
    assert not dev.download(d_y2, (H,), np.float32).any()
    assert not lib.q4_hip_moe_pack(d_y2, dev.upload(x), dev.upload(sgate), None, None, H, False, None, None, 0)
    y, hy, sh = (rng.standard_normal(H).astype(np.float32) for _ in range(3))
    inj = rng.standard_normal(hc).astype(np.float32)
    res0 = rng.standard_normal((hc, H)).astype(np.float32)
    for dot in (d_dot, None):
        d_res = dev.upload(res0)
        assert lib.q4_hip_moe_final(d_res, dev.upload(y), dev.upload(hy), dev.upload(sh), dot,
                                    dev.upload(inj), H, hc)
        v = y.astype(np.float64) + hy + sh * (g if dot else 1.0)
        want = res0 + v[None, :] * (2 * _sig(inj / np.float32(hc)))[:, None]
        np.testing.assert_allclose(dev.download(d_res, (hc, H), np.float32), want, rtol=1e-5, atol=1e-5)


class _Seg(C.Structure):
    _fields_ = [("w", C.c_void_p), ("out", C.c_void_p), ("rows", C.c_uint32), ("ty", C.c_uint32),
                ("act", C.c_float)]


def test_multi_segment_gemv(dev, pkg, oracle):
    """Shared-expert gate and up rows plus an fp32 gate row in one launch (src/q4_moe.c:1404-1410)."""
    rng = np.random.default_rng(8)
    lib = dev.lib
    H, F = 2048, 256
    x = rng.standard_normal(H).astype(np.float32)
    wg, wu = (pkg.synth.iq3s_blocks(rng, F * H // 256).reshape(F, -1) for _ in range(2))
    wf = rng.standard_normal((3, H)).astype(np.float32) * 0.02
    outs = [dev.malloc(F * 4), dev.malloc(F * 4), dev.malloc(3 * 4)]
    segs = (_Seg * 3)(_Seg(dev.upload(wg), outs[0], F, IQ3_S, 0.5), _Seg(dev.upload(wu), outs[1], F, IQ3_S, 0.0),
                      _Seg(dev.upload(wf), outs[2], 3, F32, 0.0))
    assert lib.q4_hip_gemv_m(C.cast(segs, C.c_void_p), 3, dev.upload(x), H)
    dq = lambda w: np.stack([oracle.dequant_row(w[r], H) for r in range(F)]).astype(np.float64)
    g = 0.5 * (dq(wg) @ x)
    assert _rel(dev.download(outs[0], (F,), np.float32), g * _sig(g)) < 1e-5
    assert _rel(dev.download(outs[1], (F,), np.float32), dq(wu) @ x) < 1e-5
    assert _rel(dev.download(outs[2], (3,), np.float32), wf.astype(np.float64) @ x) < 1e-5
    segs[1].ty = 12                                   # a type this path does not take: nothing runs
    assert not lib.q4_hip_gemv_m(C.cast(segs, C.c_void_p), 3, dev.upload(x), H)
    assert not lib.q4_hip_gemv_m(C.cast(segs, C.c_void_p), 9, dev.upload(x), H)


@pytest.mark.parametrize("counts", [[3, 5, 7, 9], [4], [0, 6, 0], [64, 1]])
def test_exec_tok_matches_single_token_exec(dev, pkg, oracle, counts):
    """Per-token exec over packed device lists (src/q4_rocm.cu:5619-5660)."""
    H, F, n_slots = 2048, 512, 70
    rng = np.random.default_rng(sum(counts))
    packs = pkg.synth.expert_packs(rng, n_slots, H, F)
    layer = pkg.MoeLayer(dev, packs, None, np.zeros((n_slots, H), np.float32), None, H, F, 1, arena=1)
    lib = dev.lib
    try:
        n_tok = len(counts)
        xs = rng.standard_normal((n_tok, H)).astype(np.float32)
        off = np.concatenate([[0], np.cumsum(counts)]).astype(np.uint32)
        slots = np.concatenate([rng.choice(n_slots, c, replace=False) for c in counts]).astype(np.int32)
        wts = rng.random(off[-1]).astype(np.float32)
        y0 = rng.standard_normal((n_tok, H)).astype(np.float32)     # the call adds into y
        d_y = dev.upload(y0)
        d_h = dev.malloc(max(1, int(off[-1])) * F * 4)
        assert lib.q4_hip_moe_tok_ok(IQ3_S, IQ3_S, IQ3_S, H, F)
        assert lib.q4_hip_moe_exec_tok(layer.base, layer.stride, dev.upload(slots), dev.upload(wts),
                                       off.ctypes.data_as(C.c_void_p), n_tok, IQ3_S, layer.og, IQ3_S,
                                       layer.ou, IQ3_S, layer.od, dev.upload(xs), d_h, None, d_y, F, H, H)
        y = dev.download(d_y, (n_tok, H), np.float32)
        for t, c in enumerate(counts):
            if c == 0:
                assert np.array_equal(y[t], y0[t])
                continue
            s, w = slots[off[t]:off[t + 1]], wts[off[t]:off[t + 1]]
            y1, _ = layer.exec_experts(xs[t], s, w)
            assert _rel(y[t] - y0[t], y1) < 1e-5
            if c <= 9:
                assert _rel(y[t] - y0[t], oracle.expert_job([packs[i] for i in s], w, xs[t], H, F)) <= 1e-3
        bad = off.copy()
        bad[-1] = bad[-2] + 65                                      # more than 64 entries for a token
        assert not lib.q4_hip_moe_exec_tok(layer.base, layer.stride, dev.upload(slots), dev.upload(wts),
                                           bad.ctypes.data_as(C.c_void_p), n_tok, IQ3_S, layer.og, IQ3_S,
                                           layer.ou, IQ3_S, layer.od, dev.upload(xs), d_h, None, d_y, F, H, H)
        assert lib.q4_cuda_device_error() == 0
    finally:
        layer.close()


@pytest.mark.parametrize("n", [2, 5, 8])
def test_mmvq_rows_match_oracle_dots(dev, pkg, oracle, n):
    """2..8-row GEMV on 8-bit activations: the shared expert's projections in a verify window
    (src/q4_moe.c:2151-2170)."""
    rng = np.random.default_rng(20 + n)
    lib = dev.lib
    nrows, ncols = 512, 2048
    w = pkg.synth.iq3s_blocks(rng, nrows * ncols // 256).reshape(nrows, -1)
    x = rng.standard_normal((n, ncols)).astype(np.float32)
    d_w, d_x = dev.upload(w), dev.upload(x)
    d_y = dev.malloc(n * nrows * 4)
    lib.q4_mmvq_warm()
    assert lib.q4_mmvq_on() == 1
    assert lib.q4_mmvq_n(IQ3_S, d_w, nrows, ncols, d_x, d_y, 0.5, n)
    y = dev.download(d_y, (n, nrows), np.float32)
    for t in range(n):
        xq = oracle.quant8(x[t])
        want = np.array([oracle.dot8(w[r], xq, ncols) for r in range(0, nrows, 37)], np.float64) * 0.5
        assert _rel(y[t, ::37], want) < 1e-5
    # hold: a second matrix against the same rows reuses their quantisation
    w2 = pkg.synth.iq3s_blocks(rng, nrows * ncols // 256).reshape(nrows, -1)
    launches = lib.q4_cuda_launch_count()
    lib.q4_mmvq_hold(d_x)
    assert lib.q4_mmvq_n(IQ3_S, d_w, nrows, ncols, d_x, d_y, 1.0, n)
    mid = lib.q4_cuda_launch_count()
    d_y2 = dev.malloc(n * nrows * 4)
    assert lib.q4_mmvq_n(IQ3_S, dev.upload(w2), nrows, ncols, d_x, d_y2, 1.0, n)
    lib.q4_mmvq_release()
    assert lib.q4_cuda_launch_count() - mid == (mid - launches) - 1      # no second quantise
    y2 = dev.download(d_y2, (n, nrows), np.float32)
    xq = oracle.quant8(x[n - 1])
    assert _rel(y2[n - 1, :8], np.array([oracle.dot8(w2[r], xq, ncols) for r in range(8)])) < 1e-5
    assert not lib.q4_mmvq_n(IQ3_S, d_w, nrows, ncols, d_x, d_y, 1.0, 9)
    assert not lib.q4_mmvq_n(IQ3_S, d_w, nrows, ncols, d_x, d_y, 1.0, 1)
    lib.q4_mmvq_set(0)
    assert lib.q4_mmvq_on() == 0 and not lib.q4_mmvq_n(IQ3_S, d_w, nrows, ncols, d_x, d_y, 1.0, n)
    lib.q4_mmvq_set(1)
    assert lib.q4_xg_on() == 0


@pytest.mark.parametrize("tiled", [True, False])
def test_gather_into_expert_indexed_buffers(dev, pkg, tiled):
    """q4_mmq_wbuf + q4_mmq_gather (src/q4_moe.c:3641-3675): slots in any order -> buffers indexed by
    expert id; the grouped product over the copy equals the product over the arena."""
    H, F, n_exp = 2048, 512, 6
    rng = np.random.default_rng(9)
    packs = pkg.synth.expert_packs(rng, n_exp, H, F)
    lib = dev.lib
    perm = rng.permutation(n_exp)                       # expert e lives in slot perm[e]
    lib.q4_cuda_set_tiled_default(1 if tiled else 0)
    try:
        layer = pkg.MoeLayer(dev, packs[np.argsort(perm)], None, np.zeros((n_exp, H), np.float32), None, H, F, 1,
                             arena=2)
    finally:
        lib.q4_cuda_set_tiled_default(1)
    try:
        gu_bytes, d_bytes = 2 * F * (H // 256) * 110, H * (F // 256) * 110
        p_gu, p_d = C.c_void_p(), C.c_void_p()
        assert lib.q4_mmq_wbuf(gu_bytes, d_bytes, n_exp, C.byref(p_gu), C.byref(p_d))
        eid = np.arange(n_exp, dtype=np.int32)
        assert lib.q4_mmq_gather(layer.base, layer.stride, layer.og, gu_bytes, layer.od, d_bytes, gu_bytes,
                                 d_bytes, dev.upload(eid), dev.upload(perm.astype(np.int32)), n_exp,
                                 p_gu, p_d)
        rows = 3 * n_exp
        bounds = (3 * np.arange(n_exp + 1)).astype(np.int32)
        x = rng.standard_normal((rows, H)).astype(np.float32)
        d_xq = dev.malloc(lib.q4_mmq_q8_bytes(rows, H))
        assert lib.q4_mmq_quantize(dev.upload(x), None, d_xq, IQ3_S, H, rows)
        d_a, d_b = dev.malloc(rows * 2 * F * 4), dev.malloc(rows * 2 * F * 4)
        assert lib.q4_mmq_mul_id(p_gu, IQ3_S, 2 * F, H, gu_bytes, n_exp, d_xq, dev.upload(bounds), 3, rows,
                                 d_a, 2 * F)
        # the same product straight from the arena, expert e = slot perm[e]: one call per expert
        for e in range(n_exp):
            b2 = np.array([3 * e, 3 * e + 3], np.int32)
            assert lib.q4_mmq_mul_id(layer.base + int(perm[e]) * layer.stride + layer.og, IQ3_S, 2 * F, H, 0, 1,
                                     d_xq, dev.upload(b2), 3, rows, d_b, 2 * F)
        a, b = dev.download(d_a, (rows, 2 * F), np.float32), dev.download(d_b, (rows, 2 * F), np.float32)
        # the copy holds the same bytes: the same kernel gives the same floats; in the engine's byte order
        # a one-expert call may take another kernel, whose row sums differ in the last bits
        assert np.array_equal(a, b) if tiled else _rel(a, b) < 1e-6
        assert lib.q4_cuda_device_error() == 0
    finally:
        layer.close()


def test_gemv_forms_with_host_operands_and_row_gather(dev, pkg, oracle):
    """q4_hip_gemv (host W), q4_hip_gemv_dev (device W, host x and y), q4_hip_gemv_dd_n_which
    (token i reads row which[i]) (src/q4.h:1061-1077)."""
    rng = np.random.default_rng(12)
    lib = dev.lib
    nrows, ncols, n_tok = 40, 1024, 6
    x = rng.standard_normal((n_tok, ncols)).astype(np.float32)
    wf = (rng.standard_normal((nrows, ncols)) * 0.05).astype(np.float32)
    wq = pkg.synth.iq3s_blocks(rng, nrows * ncols // 256).reshape(nrows, -1)
    deq = np.stack([oracle.dequant_row(wq[r], ncols) for r in range(nrows)]).astype(np.float64)
    y = np.zeros(nrows, np.float32)
    for ty, w, ref in ((F32, wf, wf.astype(np.float64)), (IQ3_S, wq, deq)):
        w = np.ascontiguousarray(w)
        assert lib.q4_hip_gemv(ty, w.ctypes.data, nrows, ncols, x[0].ctypes.data, y.ctypes.data, 2.0)
        assert _rel(y, 2.0 * (ref @ x[0])) < 1e-5
        d_w = dev.upload(w)
        assert lib.q4_hip_gemv_dev(ty, d_w, nrows, ncols, x[1].ctypes.data, y.ctypes.data, 1.0)
        assert _rel(y, ref @ x[1]) < 1e-5
        which = np.array([5, 0, 0, 3], np.int32)
        d_y = dev.malloc(4 * nrows * 4)
        assert lib.q4_hip_gemv_dd_n_which(ty, d_w, nrows, ncols, dev.upload(x), d_y, 0.5, 4, dev.upload(which))
        got = dev.download(d_y, (4, nrows), np.float32)
        assert _rel(got, 0.5 * (x[which].astype(np.float64) @ ref.T)) < 1e-5
        assert lib.q4_hip_gemv_dd_n_which(ty, d_w, nrows, ncols, dev.upload(x), d_y, 0.5, 4, None)
        assert _rel(dev.download(d_y, (4, nrows), np.float32), 0.5 * (x[:4].astype(np.float64) @ ref.T)) < 1e-5
    assert not lib.q4_hip_gemv(12, wf.ctypes.data, nrows, ncols, x[0].ctypes.data, y.ctypes.data, 1.0)


def test_host_memory_helpers_and_declined_calls(dev):
    lib = dev.lib
    buf = np.zeros(4096, np.uint8)
    if lib.q4_hip_host_register(buf.ctypes.data, buf.nbytes):
        alias = lib.q4_hip_host_devptr(buf.ctypes.data)
        assert alias
        assert lib.q4_hip_copy_memset(alias, 0x5a, 1024)     # on the copy stream, into the host page
        lib.q4_hip_copy_wait()
        lib.q4_hip_sync()
        assert (buf[:1024] == 0x5a).all() and not buf[1024:].any()
        lib.q4_hip_host_unregister(buf.ctypes.data)
    d = dev.malloc(256)
    assert lib.q4_hip_copy_memset(d, 7, 256)
    lib.q4_hip_copy_wait()
    assert (dev.download(d, (256,), np.uint8) == 7).all()
    g, u = np.linspace(-3, 3, 64, dtype=np.float32), np.full(64, 2.0, np.float32)
    d_g = dev.upload(g)
    assert lib.q4_hip_moe_act(d_g, dev.upload(u), 64)
    np.testing.assert_allclose(dev.download(d_g, (64,), np.float32), g * _sig(g) * 2.0, rtol=2e-6, atol=2e-6)
    # alternates and offload machinery answer "nothing enqueued"
    n0 = lib.q4_cuda_launch_count()
    assert not lib.q4_hip_moe_pf(IQ3_S, None, 0, 0, None, None, None, None, None, None, 8, 256, 1)
    assert not lib.q4_hip_moe_wmma2(IQ3_S, None, 0, 0, 0, None, None, None, None, None, None, 8, 256, 1)
    assert not lib.q4_hip_route_dev_n(None, None, None, None, None, None, None, None, None, 512, 10, 4)
    assert not lib.q4_hip_cpx_spin_init() and not lib.q4_hip_vtl_init()
    assert lib.q4_hip_cpx_wait_timeouts() == 0 and lib.q4_hip_pred_size() == 152
    assert not lib.q4_xg_gu_type(IQ3_S) and lib.q4_xg_tile_cap(64, 512) == 0
    assert lib.q4_cuda_launch_count() == n0
    # lend mode of the expert-indexed buffers: borrowed memory, never an allocation
    a, b = dev.malloc(1 << 20), dev.malloc(1 << 20)
    p_gu, p_d = C.c_void_p(), C.c_void_p()
    assert lib.q4_mmq_wbuf_lend(a, 1 << 20, b, 1 << 20)
    assert lib.q4_mmq_wbuf(1 << 18, 1 << 18, 4, C.byref(p_gu), C.byref(p_d)) and p_gu.value == a and p_d.value == b
    assert not lib.q4_mmq_wbuf(1 << 18, 1 << 18, 5, C.byref(p_gu), C.byref(p_d))       # too small: refused
    assert lib.q4_mmq_wbuf_lend(None, 0, None, 0)
    assert not lib.q4_mmq_wbuf(16, 16, 1, C.byref(p_gu), C.byref(p_d))                 # dropped: refused


@pytest.mark.parametrize("n_batch", [1, 5, 64, 600])
def test_batched_fp32_gemv_all_kernel_paths(dev, n_batch):
    """q4_hip_gemv_dd_n on the router's shape (src/q4.h:1069-1071): one vector per launch row, 16 vectors
    per weight row held in registers, and from 512 vectors on a tiled product (the last token tile ragged)."""
    rng = np.random.default_rng(n_batch)
    lib = dev.lib
    nrows, ncols = 512, 2048
    w = (rng.standard_normal((nrows, ncols)) * 0.02).astype(np.float32)
    x = rng.standard_normal((n_batch, ncols)).astype(np.float32)
    d_y = dev.malloc(n_batch * nrows * 4)
    assert lib.q4_hip_gemv_dd_n(F32, dev.upload(w), nrows, ncols, dev.upload(x), d_y, 0.5, n_batch)
    y = dev.download(d_y, (n_batch, nrows), np.float32)
    want = 0.5 * (x.astype(np.float64) @ w.astype(np.float64).T)
    assert _rel(y, want) < 2e-6
    assert np.abs(y - want).max() <= 1e-5 * np.abs(want).max()
    # a vector's logits do not depend on the batch it came in, beyond the summation order
    d_y1 = dev.malloc(nrows * 4)
    assert lib.q4_hip_gemv_dd_n(F32, dev.upload(w), nrows, ncols, dev.upload(x[n_batch - 1]), d_y1, 0.5, 1)
    assert _rel(dev.download(d_y1, (nrows,), np.float32), y[n_batch - 1]) < 2e-6


def test_hyper_connection_update_and_norm_in_one_launch(dev):
    """The reference's own check (src/q4_test.c:1400-1430): stream update + grouped RMSNorm in one
    launch is bit for bit the two separate calls, for the residual streams and for the normalised
    rows; the inputs are that test's closed-form patterns.  Then several tokens, with a second
    block row merged in, against numpy."""
    lib = dev.lib
    hc, ne = 4, 512
    tot = hc * ne
    i = np.arange(tot)
    hres = ((i * 37 % 101) - 50).astype(np.float32) * np.float32(0.01171875)
    hblk = ((np.arange(ne) * 53 % 89) - 44).astype(np.float32) * np.float32(0.0078125)
    hinj = ((np.arange(hc) * 29 % 41) - 20).astype(np.float32) * np.float32(0.0625)
    hwn = np.float32(0.75) + ((i * 7) % 19).astype(np.float32) * np.float32(0.015625)
    d_ra, d_rb = dev.upload(hres), dev.upload(hres)
    d_b, d_i, d_w = dev.upload(hblk), dev.upload(hinj), dev.upload(hwn)
    d_ya, d_yb = dev.malloc(tot * 4), dev.malloc(tot * 4)
    assert lib.q4_hip_hc_combine(d_ra, d_b, d_i, ne, hc)
    assert lib.q4_hip_grouped_rms(d_ra, d_w, d_ya, ne, hc, 1e-6)
    assert lib.q4_hip_hc_comb_rms(d_rb, d_b, d_i, d_w, d_yb, ne, hc, 1e-6)
    ra, rb = dev.download(d_ra, (tot,), np.float32), dev.download(d_rb, (tot,), np.float32)
    ya, yb = dev.download(d_ya, (tot,), np.float32), dev.download(d_yb, (tot,), np.float32)
    assert np.array_equal(ra.view(np.uint32), rb.view(np.uint32))
    assert np.array_equal(ya.view(np.uint32), yb.view(np.uint32))
    f = 2.0 / (1.0 + np.exp(-hinj.astype(np.float64) / hc))
    want_r = hres.reshape(hc, ne) + hblk[None, :] * f[:, None]
    np.testing.assert_allclose(ra.reshape(hc, ne), want_r, rtol=1e-6, atol=1e-6)
    want_y = want_r / np.sqrt((want_r ** 2).mean(axis=1, keepdims=True) + 1e-6) * hwn.reshape(hc, ne)
    np.testing.assert_allclose(ya.reshape(hc, ne), want_y, rtol=1e-5, atol=1e-6)
    # n tokens, a second block row merged in; and the update-only form (y == NULL)
    rng = np.random.default_rng(12)
    T, H = 3, 2048
    res0 = rng.standard_normal((T, hc, H)).astype(np.float32)
    blk, hy = (rng.standard_normal((T, H)).astype(np.float32) for _ in range(2))
    inj = rng.standard_normal((T, hc)).astype(np.float32)
    wn = (1 + 0.1 * rng.standard_normal((hc, H))).astype(np.float32)
    d_r, d_y = dev.upload(res0), dev.malloc(T * hc * H * 4)
    assert lib.q4_hip_hc_comb_rms_n(d_r, dev.upload(blk), dev.upload(hy), dev.upload(inj), dev.upload(wn), d_y, H,
                                    hc, 1e-6, T)
    f = 2.0 / (1.0 + np.exp(-inj.astype(np.float64) / hc))
    want_r = res0 + (blk.astype(np.float64) + hy)[:, None, :] * f[:, :, None]
    want_y = want_r / np.sqrt((want_r ** 2).mean(axis=2, keepdims=True) + 1e-6) * wn[None]
    np.testing.assert_allclose(dev.download(d_r, (T, hc, H), np.float32), want_r, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(dev.download(d_y, (T, hc, H), np.float32), want_y, rtol=1e-5, atol=1e-5)
    d_r2 = dev.upload(res0)
    assert lib.q4_hip_hc_comb_rms_n(d_r2, dev.upload(blk), dev.upload(hy), dev.upload(inj), None, None, H, hc,
                                    1e-6, T)
    assert np.array_equal(dev.download(d_r2, (T, hc, H), np.float32).view(np.uint32),
                          dev.download(d_r, (T, hc, H), np.float32).view(np.uint32))
    assert not lib.q4_hip_hc_comb_rms(d_r, dev.upload(blk), dev.upload(inj), None, None, H, hc, 1e-6)
    assert lib.q4_cuda_device_error() == 0
