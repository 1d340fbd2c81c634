"""Parity at the sizes of the benchmark configurations, through the C ABI, against the CPU oracle.

config 3: 2048 tokens x 512 experts + shared, expert popularity skewed by a Zipf(1.1) bias on
          the router logits (the benchmark's construction): the hottest expert has ~2000 rows,
          most have none; default kernel choice and CUDA-core kernels only.
config 2: 4 tokens x 512 experts top-10 through 3 chained layers.
Routing ids exact for every token (a pick whose probability is within 1e-6 relative of the
first expert left out is reported, not asserted: src/q4_moe.c:3287-3398 measures the same
thing); outputs rel-L2 <= 1e-3 against the oracle on sampled tokens; a token alone against the
same token in the batch: <= 2e-5 on the CUDA-core kernels (the router product of 512 tokens or
more sums in another order; smaller batches are bit for bit, tests/test_grouped_gpu.py), <= 2e-3
in the default mode (measured and printed)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

H, F, E, K = 2048, 512, 512, 10


def _rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b), 1e-30))


def _oracle_routing(oracle, L, xs):
    """ids [T, K], and per token whether its last pick is a near-tie with the first expert left out."""
    ids = np.zeros((len(xs), K), np.int32)
    near = np.zeros(len(xs), bool)
    for t, x in enumerate(xs):
        xn = oracle.rms_norm(x, L["norm_w"], 1e-6)
        p = oracle.softmax(oracle.gemv_f32(L["router"], xn))
        ids[t], _ = oracle.topk(p, K)
        s = np.sort(p)[::-1]
        near[t] = (s[K - 1] - s[K]) <= 1e-6 * s[K - 1]
    return ids, near


def _layer_n(dev, layer, d_x, n_tok, d_y, d_ids, d_ws, ws):
    assert dev.lib.q4_cuda_moe_layer_n(layer.base, layer.stride, layer.og, layer.ou, layer.od, layer.shared_slot,
                                       d_x, layer.d_norm, 1e-6, layer.d_router, E, K, H, F, n_tok, d_y, d_ids,
                                       None, d_ws, ws)


def test_config3_prefill_2048_tokens_zipf(dev, pkg, oracle):
    T = 2048
    L = pkg.synth.layer(3003, E, H, F)
    xs = pkg.synth.hidden(3004, T, H)
    # the benchmark's skew: the same value in coordinate 0 of every token, norm weight 1 there,
    # router column 0 = log Zipf(1.1) mass / (normalised value)
    A = 4.0
    xs[:, 0] = A
    L["norm_w"][0] = 1.0
    xn0 = A / np.sqrt((A * A + H - 1.0) / H)
    L["router"][:, 0] = (pkg.synth.zipf_bias(E, 1.1) / xn0).astype(np.float32)
    ids0, near = _oracle_routing(oracle, L, xs)
    hist = np.bincount(ids0.ravel(), minlength=E)
    assert hist.max() > 1500 and (hist == 0).sum() > 100, "the skew this test is about"
    layer = pkg.MoeLayer(dev, L["experts"], L["shared"], L["router"], L["norm_w"], H, F, K, arena=1)
    lib = dev.lib
    try:
        ws = lib.q4_cuda_moe_layer_n_ws_bytes(T, K, E, H, F)
        d_ws, d_x = dev.malloc(ws), dev.upload(xs)
        d_y, d_ids = dev.malloc(T * H * 4), dev.malloc(T * K * 4)
        # sampled tokens: rows of the hottest expert, of experts with few rows (the streaming kernel's;
        # the switch to the tensor-core kernel is at 6 rows in a call of this size, at 12 in small
        # ones), of a one-row expert, and random ones
        rng = np.random.default_rng(5)

        def tokens_of(e, n):
            t = np.nonzero((ids0 == e).any(axis=1))[0]
            return t[:n].tolist()

        def expert_with(lo, hi):
            c = np.nonzero((hist >= lo) & (hist <= hi))[0]
            return int(c[0]) if len(c) else None
        picks = tokens_of(int(hist.argmax()), 8)
        for lo, hi in ((5, 5), (6, 6), (11, 11), (12, 12), (1, 1), (2, 4), (13, 64), (65, 400)):
            e = expert_with(lo, hi)
            if e is not None:
                picks += tokens_of(e, 3)
        picks = sorted(set(picks) | set(rng.choice(T, 64, replace=False).tolist()))
        assert len(picks) >= 64
        want = {t: oracle.moe_layer(xs[t], L["norm_w"], 1e-6, L["router"], K, L["experts"], L["shared"], H, F)[0]
                for t in picks}
        results = {}
        for mode in (-1, 0):
            assert lib.q4_cuda_mmq_tc_mode(mode)
            try:
                _layer_n(dev, layer, d_x, T, d_y, d_ids, d_ws, ws)
                y = dev.download(d_y, (T, H), np.float32)
                ids = dev.download(d_ids, (T, K), np.int32)
            finally:
                assert lib.q4_cuda_mmq_tc_mode(-1)
            differ = np.nonzero((ids != ids0).any(axis=1))[0]
            assert all(near[t] for t in differ), (mode, differ[:8], "picks differ on tokens without a near-tie")
            print("config 3, mode %d: %d of %d tokens with a near-tie at the cut, %d of them routed differently"
                  % (mode, int(near.sum()), T, len(differ)))
            worst = max(_rel(y[t], want[t]) for t in picks if t not in set(differ.tolist()))
            assert worst <= 1e-3, (mode, worst)
            results[mode] = y
        # The two kernel choices agree to rounding everywhere.  The bound is not the 1e-6 of a
        # single product: gate/up results that differ in the last bits flip an int8 rounding of
        # the hidden row now and then, and one flip moves a down row by ~1e-4.
        d = np.array([_rel(results[-1][t], results[0][t]) for t in range(T)])
        print("config 3: default kernel choice vs CUDA-core kernels, rel-L2 median %.3g, 99th percentile %.3g, "
              "max %.3g (token %d)" % (np.median(d), np.percentile(d, 99), d.max(), int(d.argmax())))
        tw = int(d.argmax())
        yw = oracle.moe_layer(xs[tw], L["norm_w"], 1e-6, L["router"], K, L["experts"], L["shared"], H, F)[0]
        print("that token against the oracle: default %.3g, CUDA-core kernels %.3g"
              % (_rel(results[-1][tw], yw), _rel(results[0][tw], yw)))
        # what the default path promises at this size: all but a few tokens in a thousand within the
        # expert tolerance, none beyond twice it; the CUDA-core kernels (mode 0) keep every token
        # at the 1e-6 level
        assert np.percentile(d, 99) <= 1e-3 and d.max() < 2e-3
        # a token alone and in the batch
        d_y1 = dev.malloc(H * 4)
        for t in picks[:6]:
            for mode in (0, -1):
                assert lib.q4_cuda_mmq_tc_mode(mode)
                try:
                    _layer_n(dev, layer, d_x + t * H * 4, 1, d_y1, None, d_ws, ws)
                finally:
                    assert lib.q4_cuda_mmq_tc_mode(-1)
                y1 = dev.download(d_y1, (H,), np.float32)
                if mode == 0:
                    # the expert arithmetic is the same sum in the same order; the router product of a
                    # batch of 512 tokens or more is a tiled matrix product that adds a logit's terms
                    # in another order than the one-token product, so the weights differ in the last
                    # bits (batches below 512 are bit for bit: tests/test_grouped_gpu.py)
                    assert _rel(y1, results[0][t]) <= 2e-5, t
                else:       # same bound, same reason: the token's experts may change kernel with the batch
                    assert _rel(y1, results[-1][t]) <= 2e-3, t
        assert lib.q4_cuda_device_error() == 0
    finally:
        lib.q4_cuda_mmq_tc_mode(-1)
        layer.close()


def test_config2_verify_window_512_experts_three_chained_layers(dev, pkg, oracle):
    T, NL = 4, 3
    layers = [pkg.synth.layer(2002 + l, E, H, F) for l in range(NL)]
    xs = pkg.synth.hidden(2001, T, H)
    lib = dev.lib
    ws = lib.q4_cuda_moe_layer_n_ws_bytes(T, K, E, H, F)
    d_ws = dev.malloc(ws)
    d_a, d_b, d_ids = dev.upload(xs), dev.malloc(T * H * 4), dev.malloc(T * K * 4)
    x_in = xs
    for l, L in enumerate(layers):      # one layer resident at a time (693 MB each)
        layer = pkg.MoeLayer(dev, L["experts"], L["shared"], L["router"], L["norm_w"], H, F, K, arena=1)
        try:
            _layer_n(dev, layer, d_a, T, d_b, d_ids, d_ws, ws)
            y = dev.download(d_b, (T, H), np.float32)
            ids = dev.download(d_ids, (T, K), np.int32)
            ids0, near = _oracle_routing(oracle, L, x_in)
            for t in range(T):
                if not near[t]:
                    assert ids[t].tolist() == ids0[t].tolist(), (l, t)
                    # each layer against the oracle on the device's own input rows (a chained oracle
                    # would compare rounding flips of the layers' quantisers, not the kernels)
                    y0 = oracle.moe_layer(x_in[t], L["norm_w"], 1e-6, L["router"], K, L["experts"], L["shared"],
                                          H, F)[0]
                    assert _rel(y[t], y0) <= 1e-3, (l, t)
            x_in = y
            d_a, d_b = d_b, d_a          # the layer's output rows are the next layer's input rows
        finally:
            layer.close()
    assert lib.q4_cuda_device_error() == 0
