"""The first two of the other routed-expert formats the engine's call sites accept
(src/q4_rocm.cu:4926-4944): IQ4_NL and IQ4_XS, for gate+up and/or down.  Stage tests bit for bit,
then the one-token exec calls on packs of mixed formats against the CPU oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
IQ3_S, IQ4_NL, IQ4_XS = 21, 20, 23
IQ3_XXS, IQ2_S, Q2_0 = 18, 22, 42


def test_iq4nl_dequant_and_integer_dots_bit_exact(dev, pkg, oracle):
    rng = np.random.default_rng(5)
    nrows, n = 9, 512
    w = pkg.synth.iq4nl_blocks(rng, nrows * n // 32).reshape(nrows, -1)
    lib = dev.lib
    d_w = dev.upload(w)
    d_out = dev.malloc(nrows * n * 4)
    assert lib.q4_cuda_iq4nl_dequant(d_w, nrows, n, d_out)
    got = dev.download(d_out, (nrows, n), np.float32)
    x = rng.standard_normal(n).astype(np.float32)
    xq = oracle.quant8(x)
    d_q = dev.upload(np.ascontiguousarray(xq["q"]))
    d_I = dev.malloc(nrows * (n // 32) * 4)
    assert lib.q4_cuda_iq4nl_idot(d_w, nrows, n, d_q, d_I)
    I = dev.download(d_I, (nrows, n // 32), np.int32)
    for r in range(nrows):
        want = oracle.iq4nl_dequant_row(w[r], n)
        assert np.array_equal(got[r].view(np.uint32), want.view(np.uint32))
        assert np.array_equal(I[r], oracle.iq4nl_group_idot(w[r], xq, n))
    assert not lib.q4_cuda_iq4nl_dequant(d_w, nrows, 500, d_out)     # not a multiple of 32


def test_iq4xs_dequant_and_integer_dots_bit_exact(dev, pkg, oracle):
    rng = np.random.default_rng(6)
    nrows, n = 7, 1024
    w = pkg.synth.iq4xs_blocks(rng, nrows * n // 256).reshape(nrows, -1)
    lib = dev.lib
    d_w = dev.upload(w)
    d_out = dev.malloc(nrows * n * 4)
    assert lib.q4_cuda_iq4_dequant(IQ4_XS, d_w, nrows, n, d_out)
    got = dev.download(d_out, (nrows, n), np.float32)
    xq = oracle.quant8(rng.standard_normal(n).astype(np.float32))
    d_I = dev.malloc(nrows * (n // 32) * 4)
    assert lib.q4_cuda_iq4_idot(IQ4_XS, d_w, nrows, n, dev.upload(np.ascontiguousarray(xq["q"])), d_I)
    I = dev.download(d_I, (nrows, n // 32), np.int32)
    for r in range(nrows):
        assert np.array_equal(got[r].view(np.uint32), oracle.iq4xs_dequant_row(w[r], n).view(np.uint32))
        assert np.array_equal(I[r], oracle.iq4xs_group_idot(w[r], xq, n))
    assert not lib.q4_cuda_iq4_dequant(IQ4_XS, d_w, nrows, 1000, d_out)   # not a multiple of 256
    assert not lib.q4_cuda_iq4_dequant(IQ3_S, d_w, nrows, n, d_out)       # not a 4-bit format


@pytest.mark.parametrize("ty", [IQ3_XXS, IQ2_S, Q2_0])
def test_small_formats_dequant_and_integer_dots_bit_exact(dev, pkg, oracle, ty):
    rng = np.random.default_rng(50 + ty)
    nrows, n = 6, 1024
    w = np.stack([pkg.synth.blocks_of(rng, ty, pkg.synth.row_bytes(ty, n)) for _ in range(nrows)])
    lib = dev.lib
    d_w = dev.upload(w)
    d_out = dev.malloc(nrows * n * 4)
    assert lib.q4_cuda_fmt_dequant(ty, d_w, nrows, n, d_out)
    got = dev.download(d_out, (nrows, n), np.float32)
    xq = oracle.quant8(rng.standard_normal(n).astype(np.float32))
    d_I = dev.malloc(nrows * (n // 32) * 4)
    assert lib.q4_cuda_fmt_idot(ty, d_w, nrows, n, dev.upload(np.ascontiguousarray(xq["q"])), d_I)
    I = dev.download(d_I, (nrows, n // 32), np.int32)
    for r in range(nrows):
        assert np.array_equal(got[r].view(np.uint32), oracle.dequant_row_x(ty, w[r], n).view(np.uint32)), r
        assert np.array_equal(I[r], oracle.group_idot_x(ty, w[r], xq, n)), r
    assert not lib.q4_cuda_fmt_dequant(ty, d_w, nrows, n - 32, d_out)
    assert not lib.q4_cuda_fmt_dequant(IQ3_S, d_w, nrows, n, d_out)


@pytest.mark.parametrize("H,F,gu,dn", [(512, 256, IQ3_S, IQ4_NL), (2048, 512, IQ3_S, IQ4_NL),
                                       (512, 256, IQ3_S, IQ4_XS), (512, 256, IQ4_XS, IQ3_S),
                                       (2048, 512, IQ4_XS, IQ4_XS), (512, 256, IQ4_NL, IQ4_NL),
                                       (512, 256, IQ4_XS, IQ4_NL), (2048, 512, IQ3_XXS, Q2_0),
                                       (512, 256, IQ2_S, IQ3_S), (2048, 512, IQ2_S, Q2_0),
                                       (512, 256, IQ3_XXS, IQ4_NL), (512, 256, IQ3_S, Q2_0)])
def test_exec_with_other_formats_matches_oracle(dev, pkg, oracle, H, F, gu, dn):
    rng = np.random.default_rng(H + 7 * gu + dn)
    n_slots, k = 6, 4
    packs = pkg.synth.expert_packs_typed(rng, n_slots, H, F, gu, dn)
    pb = packs.shape[1]
    lib = dev.lib
    lib.q4_cuda_set_tiled_default(0)          # mixed packs stay in the engine's byte order
    try:
        assert lib.q4_hip_experts_alloc_a(3, n_slots, pb)
    finally:
        lib.q4_cuda_set_tiled_default(1)
    try:
        for e in range(n_slots):
            row = np.ascontiguousarray(packs[e])
            assert lib.q4_hip_experts_put_a(3, e, row.ctypes.data, pb)
        base, stride = lib.q4_hip_experts_base_a(3), lib.q4_hip_experts_stride_a(3)
        rb = pkg.synth.row_bytes(gu, H)
        og, ou, od = 0, F * rb, 2 * F * rb
        assert lib.q4_hip_moe_tok_ok(gu, gu, dn, H, F)
        assert not lib.q4_hip_moe_tok_ok(IQ4_NL, IQ3_S, IQ3_S, H, F)      # gate and up share a type
        assert not lib.q4_hip_moe_tok_ok(IQ3_S, IQ3_S, 12, H, F)          # a type this path does not take
        assert not lib.q4_hip_moe_tok_ok(Q2_0, Q2_0, IQ3_S, H, F)         # Q2_0 is a down format only
        assert not lib.q4_hip_moe_tok_ok(IQ3_S, IQ3_S, IQ2_S, H, F)       # IQ2_S a gate/up format only
        x = rng.standard_normal(H).astype(np.float32)
        slots = rng.choice(n_slots, k, replace=False).astype(np.int32)
        wts = rng.random(k).astype(np.float32)
        d_x, d_y, d_h = dev.upload(x), dev.malloc(H * 4), dev.malloc(64 * F * 4)
        assert lib.q4_hip_fill(d_y, 0.0, H)
        assert lib.q4_hip_moe_exec(base, stride, slots.ctypes.data, wts.ctypes.data, k, gu, og, gu, ou,
                                   dn, od, d_x, d_h, None, None, d_y, F, H, H)
        y = dev.download(d_y, (H,), np.float32)
        want = oracle.expert_job_t([packs[s] for s in slots], wts, x, H, F, dn, gu)
        assert np.linalg.norm(y - want) / np.linalg.norm(want) <= 1e-3
        # device-side list form, same result bit for bit
        assert lib.q4_hip_fill(d_y, 0.0, H)
        assert lib.q4_hip_moe_exec_dev(base, stride, dev.upload(slots), dev.upload(wts),
                                       dev.upload(np.array([k], np.int32)), gu, og, gu, ou, dn, od,
                                       d_x, d_h, None, None, d_y, F, H, H)
        y2 = dev.download(d_y, (H,), np.float32)
        assert np.array_equal(y2.view(np.uint32), y.view(np.uint32))
        assert lib.q4_cuda_device_error() == 0
    finally:
        lib.q4_hip_experts_free_a(3)


def test_iq4nl_down_refused_on_a_tiled_arena(dev, pkg):
    """The tiled arena format regroups IQ3_S bytes; a pack with an IQ4_NL part in it is refused
    before anything is enqueued."""
    H, F = 2048, 512
    lib = dev.lib
    pb = pkg.synth.expert_pack_bytes(H, F)          # a size the tiling accepts
    assert lib.q4_hip_experts_alloc_a(3, 2, pb)
    try:
        assert lib.q4_cuda_experts_tiled_a(3) == 1
        base, stride = lib.q4_hip_experts_base_a(3), lib.q4_hip_experts_stride_a(3)
        slots, wts = np.array([0], np.int32), np.array([1.0], np.float32)
        d_x, d_y, d_h = dev.malloc(H * 4), dev.malloc(H * 4), dev.malloc(64 * F * 4)
        n0 = lib.q4_cuda_launch_count()
        assert not lib.q4_hip_moe_exec(base, stride, slots.ctypes.data, wts.ctypes.data, 1, IQ3_S, 0, IQ3_S, 1,
                                       IQ4_NL, 2, d_x, d_h, None, None, d_y, F, H, H)
        assert lib.q4_cuda_launch_count() == n0
    finally:
        lib.q4_hip_experts_free_a(3)


def test_mixed_pack_of_a_tile_multiple_size_is_not_tiled(dev, pkg, oracle):
    """An arena is tiled only when its slot size is that of an all-IQ3_S pack.  Here the pack has
    an IQ4_NL down projection and its size is a multiple of the 880-byte tile all the same
    (hidden 2816, intermediate 1280): it must stay in the engine's byte order on upload and run."""
    H, F, n_slots, k = 2816, 1280, 3, 2
    rng = np.random.default_rng(9)
    packs = pkg.synth.expert_packs_typed(rng, n_slots, H, F, IQ3_S, IQ4_NL)
    pb = packs.shape[1]
    assert pb % 880 == 0 and pb % 84480 != 0
    lib = dev.lib
    assert lib.q4_hip_experts_alloc_a(3, n_slots, pb)           # the default format rule decides
    try:
        assert lib.q4_cuda_experts_tiled_a(3) == 0
        for e in range(n_slots):
            row = np.ascontiguousarray(packs[e])
            assert lib.q4_hip_experts_put_a(3, e, row.ctypes.data, pb)
        back = np.empty(pb, np.uint8)
        assert lib.q4_cuda_experts_get_a(3, 1, back.ctypes.data, pb)
        assert np.array_equal(back, packs[1])
        base, stride = lib.q4_hip_experts_base_a(3), lib.q4_hip_experts_stride_a(3)
        rb = pkg.synth.row_bytes(IQ3_S, H)
        og, ou, od = 0, F * rb, 2 * F * rb
        x = rng.standard_normal(H).astype(np.float32)
        slots = np.array([2, 0], np.int32)
        wts = rng.random(k).astype(np.float32)
        d_x, d_y, d_h = dev.upload(x), dev.malloc(H * 4), dev.malloc(64 * F * 4)
        assert lib.q4_hip_fill(d_y, 0.0, H)
        assert lib.q4_hip_moe_exec(base, stride, slots.ctypes.data, wts.ctypes.data, k, IQ3_S, og, IQ3_S, ou,
                                   IQ4_NL, od, d_x, d_h, None, None, d_y, F, H, H)
        y = dev.download(d_y, (H,), np.float32)
        want = oracle.expert_job_t([packs[s] for s in slots], wts, x, H, F, IQ4_NL, IQ3_S)
        assert np.linalg.norm(y - want) / np.linalg.norm(want) <= 1e-3
        assert lib.q4_cuda_device_error() == 0
    finally:
        lib.q4_hip_experts_free_a(3)


@pytest.mark.parametrize("H,F,gu,dn,n_tok", [(2048, 512, IQ3_S, IQ4_NL, 5), (512, 256, IQ4_XS, IQ3_S, 33),
                                             (512, 256, IQ4_NL, IQ4_XS, 3), (2048, 512, IQ4_XS, IQ4_XS, 20)])
def test_many_token_layer_with_other_formats(dev, pkg, oracle, H, F, gu, dn, n_tok):
    """A layer whose experts mix formats through the many-token call (q4_cuda_moe_layer_nt: grouped
    products per format) and, for 2..8 tokens, the verify-window call: routing ids exact, outputs
    within 1e-3 of the oracle token by token, and the window equal to the one-token call."""
    rng = np.random.default_rng(11 * H + gu + 3 * dn)
    E, K = 16, 4
    packs = pkg.synth.expert_packs_typed(rng, E + 1, H, F, gu, dn)      # slot E: the shared expert
    pb = packs.shape[1]
    router = (rng.standard_normal((E, H)) * 0.05).astype(np.float32)
    norm_w = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    xs = rng.standard_normal((n_tok, H)).astype(np.float32)
    lib = dev.lib
    lib.q4_cuda_set_tiled_default(0)
    try:
        assert lib.q4_hip_experts_alloc_a(3, E + 1, pb)
    finally:
        lib.q4_cuda_set_tiled_default(1)
    try:
        for e in range(E + 1):
            row = np.ascontiguousarray(packs[e])
            assert lib.q4_hip_experts_put_a(3, e, row.ctypes.data, pb)
        base, stride = lib.q4_hip_experts_base_a(3), lib.q4_hip_experts_stride_a(3)
        rb = pkg.synth.row_bytes(gu, H)
        og, ou, od = 0, F * rb, 2 * F * rb
        ws = lib.q4_cuda_moe_layer_n_ws_bytes(n_tok, K, E, H, F)
        d_ws, d_x = dev.malloc(ws), dev.upload(xs)
        d_y, d_ids, d_wts = dev.malloc(n_tok * H * 4), dev.malloc(n_tok * K * 4), dev.malloc(n_tok * K * 4)
        assert lib.q4_cuda_moe_layer_nt(base, stride, gu, og, ou, dn, od, E, d_x, dev.upload(norm_w), 1e-6,
                                        dev.upload(router), E, K, H, F, n_tok, d_y, d_ids, d_wts, d_ws, ws)
        y = dev.download(d_y, (n_tok, H), np.float32)
        ids = dev.download(d_ids, (n_tok, K), np.int32)
        wts = dev.download(d_wts, (n_tok, K), np.float32)
        for t in range(n_tok):
            xn = oracle.rms_norm(xs[t], norm_w, 1e-6)
            p = oracle.softmax(oracle.gemv_f32(router, xn))
            ids0, w0 = oracle.topk(p, K)
            assert ids[t].tolist() == ids0.tolist(), t
            assert np.abs(wts[t] - w0).max() <= 1e-6
            want = oracle.expert_job_t([packs[i] for i in ids0] + [packs[E]], list(w0) + [1.0], xn, H, F, dn, gu)
            assert np.linalg.norm(y[t] - want) / np.linalg.norm(want) <= 1e-3, t
        assert not lib.q4_cuda_moe_layer_nt(base, stride, gu, og, ou, 12, od, E, d_x, None, 1e-6,
                                            dev.upload(router), E, K, H, F, n_tok, d_y, None, None, d_ws, ws)
        if n_tok <= 8:
            # the verify window (src/q4.h:887-897) on the same picks: 64 list entries per token
            assert lib.q4_hip_moe_win_ok(gu, gu, dn, H, F, n_tok)
            es = np.full((n_tok, 64), -1, np.int32)
            ew = np.zeros((n_tok, 64), np.float32)
            xn_all = np.stack([oracle.rms_norm(x, norm_w, 1e-6) for x in xs])
            for t in range(n_tok):
                es[t, :K], ew[t, :K] = ids[t], wts[t]
            nh = np.full(n_tok, K, np.int32)
            d_yw = dev.malloc(n_tok * H * 4)
            assert lib.q4_hip_fill(d_yw, 0.0, n_tok * H)
            assert lib.q4_hip_moe_exec_win(base, stride, dev.upload(es), dev.upload(ew), dev.upload(nh), n_tok,
                                           gu, og, gu, ou, dn, od, dev.upload(xn_all), dev.malloc(n_tok * 64 * F * 4),
                                           d_yw, F, H, H)
            yw = dev.download(d_yw, (n_tok, H), np.float32)
            for t in range(n_tok):
                want = oracle.expert_job_t([packs[i] for i in ids[t]], wts[t], xn_all[t], H, F, dn, gu)
                assert np.linalg.norm(yw[t] - want) / np.linalg.norm(want) <= 1e-3, t
        assert lib.q4_cuda_device_error() == 0
    finally:
        lib.q4_hip_experts_free_a(3)
