"""The persistent decode kernel over a stack of layers (q4_cuda_decode_stack_*), through the
C ABI: bit for bit against the one-layer call chained on the device, and every layer against
the CPU oracle on the same input row: routing ids exact, weights within 1e-6, outputs within
rel-L2 1e-3."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

REL_TOL = 1e-3
H, F = 2048, 512


def _rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b), 1e-30))


class Stack:
    """n_layers MoE layers in one arena: layer l owns slots [l * (E + 1), (l + 1) * (E + 1))."""

    def __init__(self, dev, pkg, layers, topk, arena=1):
        self.dev, self.lib = dev, dev.lib
        lib = self.lib
        self.layers, self.topk, self.arena = layers, topk, arena
        self.E = E = layers[0]["experts"].shape[0]
        self.pack = pkg.synth.expert_pack_bytes(H, F)
        L = len(layers)
        assert lib.q4_hip_experts_alloc_a(arena, L * (E + 1), self.pack)
        for l, ly in enumerate(layers):
            for e in range(E + 1):
                row = np.ascontiguousarray(ly["experts"][e] if e < E else ly["shared"])
                assert lib.q4_hip_experts_put_a(arena, l * (E + 1) + e, row.ctypes.data, self.pack)
        self.base = lib.q4_hip_experts_base_a(arena)
        self.stride = lib.q4_hip_experts_stride_a(arena)
        rb = pkg.synth.iq3s_row_bytes(H)
        self.og, self.ou, self.od = 0, F * rb, 2 * F * rb
        self.d_router = [dev.upload(ly["router"]) for ly in layers]
        self.d_norm = [dev.upload(ly["norm_w"]) if ly["norm_w"] is not None else None for ly in layers]
        self.d_x, self.d_y = dev.malloc(H * 4), dev.malloc(H * 4)
        self.d_ids, self.d_wts = dev.malloc(L * topk * 4), dev.malloc(L * topk * 4)

    def layer_base(self, l):
        return self.base + l * (self.E + 1) * self.stride

    def plan(self, first=0, count=None):
        count = len(self.layers) - first if count is None else count

        class Desc(ctypes.Structure):
            _fields_ = [("base", ctypes.c_void_p), ("norm", ctypes.c_void_p), ("router", ctypes.c_void_p)]
        arr = (Desc * count)()
        for i in range(count):
            arr[i].base = self.layer_base(first + i)
            arr[i].norm = self.d_norm[first + i]
            arr[i].router = self.d_router[first + i]
        return self.lib.q4_cuda_decode_stack_plan(arr, count, self.stride, self.og, self.ou, self.od, self.E,
                                                  1e-6, self.E, self.topk, H, F)

    def run(self, plan, x, n_layers):
        self.dev.write(self.d_x, x)
        assert self.lib.q4_cuda_decode_stack_dev(plan, self.d_x, self.d_y, self.d_ids, self.d_wts)
        return (self.dev.download(self.d_y, (H,), np.float32),
                self.dev.download(self.d_ids, (n_layers, self.topk), np.int32),
                self.dev.download(self.d_wts, (n_layers, self.topk), np.float32))

    def one_layer(self, l, x):
        self.dev.write(self.d_x, x)
        assert self.lib.q4_cuda_moe_decode(self.layer_base(l), self.stride, self.og, self.ou, self.od, self.E,
                                           self.d_x, self.d_norm[l], 1e-6, self.d_router[l], self.E, self.topk,
                                           H, F, self.d_y, self.d_ids, self.d_wts)
        return self.dev.download(self.d_y, (H,), np.float32)

    def close(self):
        self.lib.q4_hip_experts_free_a(self.arena)


@pytest.mark.parametrize("n_expert,topk,n_layers", [(64, 8, 4), (512, 10, 2), (24, 4, 3), (32, 11, 1), (16, 1, 2)])
def test_stack_matches_oracle_and_one_layer_calls(dev, pkg, oracle, n_expert, topk, n_layers):
    layers = [pkg.synth.layer(300 + 7 * l + n_expert, n_expert, H, F) for l in range(n_layers)]
    st = Stack(dev, pkg, layers, topk)
    lib = dev.lib
    try:
        plan = st.plan()
        assert plan and lib.q4_cuda_decode_stack_layers(plan) == n_layers
        for t, x in enumerate(pkg.synth.hidden(17 + n_expert, 2, H)):
            y, ids, wts = st.run(plan, x, n_layers)
            # Layer by layer: the one-layer call on the device's own intermediate row must give
            # the stack's result bit for bit, and each layer is compared with the oracle on that
            # same input row (a chained oracle would not do: one flipped int8 rounding in a
            # layer's input moves its output by far more than the kernels differ).
            xi = x
            for l in range(n_layers):
                ly = layers[l]
                y0, ids0, w0, _ = oracle.moe_layer(xi, ly["norm_w"], 1e-6, ly["router"], topk, ly["experts"],
                                                   ly["shared"], H, F)
                xi = st.one_layer(l, xi)
                assert ids[l].tolist() == ids0.tolist(), (t, l)
                assert np.abs(wts[l] - w0).max() <= 1e-6
                assert _rel(xi, y0) <= REL_TOL, (t, l)
            assert np.array_equal(y.view(np.uint32), xi.view(np.uint32))
        lib.q4_cuda_decode_stack_free(plan)
        assert lib.q4_cuda_device_error() == 0
    finally:
        st.close()


def test_stack_in_a_graph_replays_with_fresh_input(dev, pkg):
    """A captured stack launch replays correctly: the kernel's hand-over words are stamped from
    a device-side launch counter, not from launch arguments a graph would freeze."""
    n_expert, topk, n_layers = 32, 4, 3
    layers = [pkg.synth.layer(400 + l, n_expert, H, F) for l in range(n_layers)]
    st = Stack(dev, pkg, layers, topk)
    lib = dev.lib
    try:
        plan = st.plan()
        xs = pkg.synth.hidden(5, 3, H)
        want = [st.run(plan, x, n_layers)[0] for x in xs]
        assert lib.q4_hip_graph_begin() == 1
        assert lib.q4_cuda_decode_stack_dev(plan, st.d_x, st.d_y, None, None)
        g = lib.q4_hip_graph_end()
        assert g
        for x, w in zip(xs, want):
            dev.write(st.d_x, x)
            assert lib.q4_hip_graph_launch(g) and lib.q4_hip_graph_launch(g)
            assert np.array_equal(dev.download(st.d_y, (H,), np.float32).view(np.uint32), w.view(np.uint32))
        lib.q4_hip_graph_free(g)
        lib.q4_cuda_decode_stack_free(plan)
        assert lib.q4_cuda_device_error() == 0
    finally:
        st.close()


def test_stack_host_buffers(dev, pkg):
    n_expert, topk, n_layers = 32, 4, 2
    layers = [pkg.synth.layer(500 + l, n_expert, H, F) for l in range(n_layers)]
    st = Stack(dev, pkg, layers, topk)
    lib = dev.lib
    try:
        plan = st.plan()
        h_x, h_y = lib.q4_hip_host_alloc_coh(H * 4), lib.q4_hip_host_alloc_coh(H * 4)
        y_page = np.zeros(H, np.float32)
        for x in pkg.synth.hidden(6, 2, H):
            want = st.run(plan, x, n_layers)[0]
            ctypes.memmove(h_x, x.ctypes.data, H * 4)
            ctypes.memset(h_y, 0, H * 4)
            assert lib.q4_cuda_decode_stack_host(plan, h_x, h_y)
            got = np.ctypeslib.as_array(ctypes.cast(h_y, ctypes.POINTER(ctypes.c_float)), (H,)).copy()
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
            assert lib.q4_cuda_decode_stack_host(plan, x.ctypes.data, y_page.ctypes.data)   # pageable: copy + sync
            assert np.array_equal(y_page.view(np.uint32), want.view(np.uint32))
        # a result buffer that is freed is forgotten by the plan: the next buffer, wherever the
        # allocator puts it, is looked up again
        lib.q4_hip_host_free_coh(h_y)
        h_y2 = lib.q4_hip_host_alloc_coh(H * 4)
        assert lib.q4_cuda_decode_stack_host(plan, h_x, h_y2)
        got = np.ctypeslib.as_array(ctypes.cast(h_y2, ctypes.POINTER(ctypes.c_float)), (H,)).copy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        lib.q4_hip_host_free_coh(h_x)
        lib.q4_hip_host_free_coh(h_y2)
        lib.q4_cuda_decode_stack_free(plan)
        assert lib.q4_cuda_device_error() == 0
    finally:
        st.close()


def test_picks_follow_probability_order_when_logits_collapse(dev, pkg, oracle):
    """The kernel picks on logit order first (to start the weight copies early) and checks
    the result against the probability order the reference defines
    (src/q4_quant.c:715-755): two different logits that round to the same probability must
    go to the lower index.  Router rows are zero except column 0, x is zero except element 0,
    so logit_e = router[e][0] * xn[0] exactly."""
    n_expert, topk = 64, 4
    ly = pkg.synth.layer(77, n_expert, H, F)
    ly["norm_w"] = np.ones(H, np.float32)
    x = np.zeros(H, np.float32)
    x[0] = 1.0
    xn0 = oracle.rms_norm(x, None, 1e-6)[0]
    col = np.full(n_expert, -0.05, np.float32)
    col[[40, 7, 21]] = [0.08, 0.06, 0.05]          # three clear picks
    a = np.float32(2e-3)
    col[50] = a                                     # lower logit, lower index ...
    col[51] = np.nextafter(a, np.float32(1))        # ... and its neighbour one ulp above
    r = np.zeros((n_expert, H), np.float32)
    r[:, 0] = col
    ly["router"] = r
    logits = col * xn0
    assert logits[51] > logits[50]
    m = logits.max()
    # the pair already collapses in (logit - max), so every expf gives the two one probability
    assert np.float32(logits[50] - m) == np.float32(logits[51] - m)
    p = oracle.softmax(logits)
    assert p[50] == p[51]
    y0, ids0, w0, _ = oracle.moe_layer(x, ly["norm_w"], 1e-6, r, topk, ly["experts"], ly["shared"], H, F)
    assert ids0.tolist() == [40, 7, 21, 50]
    st = Stack(dev, pkg, [ly], topk)
    try:
        plan = st.plan()
        y, ids, wts = st.run(plan, x, 1)
        assert ids[0].tolist() == ids0.tolist()
        assert np.abs(wts[0] - w0).max() <= 1e-6
        assert _rel(y, y0) <= REL_TOL
        dev.lib.q4_cuda_decode_stack_free(plan)
        assert dev.lib.q4_cuda_device_error() == 0
    finally:
        st.close()


def test_equal_logits_inside_the_picks_are_reported_by_index(dev, pkg, oracle):
    """Equal logits: lower index first, both among the picks and at the boundary; all logits
    equal: the first topk experts."""
    n_expert, topk = 48, 6
    ly = pkg.synth.layer(78, n_expert, H, F)
    ly["norm_w"] = np.ones(H, np.float32)
    x = np.zeros(H, np.float32)
    x[0] = 1.0
    for col in (np.where(np.arange(n_expert) % 5 == 0, 0.04, 0.0).astype(np.float32),
                np.zeros(n_expert, np.float32)):
        r = np.zeros((n_expert, H), np.float32)
        r[:, 0] = col
        ly["router"] = r
        y0, ids0, w0, _ = oracle.moe_layer(x, ly["norm_w"], 1e-6, r, topk, ly["experts"], ly["shared"], H, F)
        st = Stack(dev, pkg, [ly], topk)
        try:
            plan = st.plan()
            y, ids, wts = st.run(plan, x, 1)
            assert ids[0].tolist() == ids0.tolist()
            assert np.abs(wts[0] - w0).max() <= 1e-6
            assert _rel(y, y0) <= REL_TOL
            dev.lib.q4_cuda_decode_stack_free(plan)
        finally:
            st.close()
    assert dev.lib.q4_cuda_device_error() == 0


def test_a_wait_that_runs_out_is_reported_and_the_next_call_works(dev, pkg, oracle):
    """Every wait for another CTA's values is bounded.  With the bound set to one poll some
    waits run out: the kernel still ends, the error word carries bit 2 (value 4), the
    host-buffer call answers false, and the next call with the normal bound is correct."""
    n_expert, topk, n_layers = 32, 4, 3
    layers = [pkg.synth.layer(600 + l, n_expert, H, F) for l in range(n_layers)]
    st = Stack(dev, pkg, layers, topk)
    lib = dev.lib
    try:
        plan = st.plan()
        x = pkg.synth.hidden(8, 1, H)[0]
        want = x
        for l in range(n_layers):
            want = st.one_layer(l, want)
        lib.q4_cuda_decode_wait_limit(1)
        dev.write(st.d_x, x)
        assert lib.q4_cuda_decode_stack_dev(plan, st.d_x, st.d_y, None, None)
        dev.sync()
        err = lib.q4_cuda_device_error()
        assert err & 4, err
        h_x, h_y = lib.q4_hip_host_alloc_coh(H * 4), lib.q4_hip_host_alloc_coh(H * 4)
        ctypes.memmove(h_x, x.ctypes.data, H * 4)
        ok = lib.q4_cuda_decode_stack_host(plan, h_x, h_y)
        err = lib.q4_cuda_device_error()
        assert (not ok) == bool(err & 4)
        lib.q4_cuda_decode_wait_limit(0)
        y, _, _ = st.run(plan, x, n_layers)
        assert lib.q4_cuda_device_error() == 0
        assert np.array_equal(y.view(np.uint32), want.view(np.uint32))
        assert lib.q4_cuda_decode_stack_host(plan, h_x, h_y)
        lib.q4_hip_host_free_coh(h_x)
        lib.q4_hip_host_free_coh(h_y)
        lib.q4_cuda_decode_stack_free(plan)
    finally:
        lib.q4_cuda_decode_wait_limit(0)
        st.close()


def test_session_steps_match_launches_bit_for_bit(dev, pkg):
    """A session (the kernel stays resident, a step costs no launch) gives, step by step, what the
    same layers give as launches: one layer per step walks the plan cyclically, all layers per step
    is the stack call.  Also: the kernel leaving on its idle limit and on its step limit is
    transparent to the caller, and the library works as before once the session has ended."""
    import time
    n_expert, topk, n_layers = 64, 6, 3
    layers = [pkg.synth.layer(700 + l, n_expert, H, F) for l in range(n_layers)]
    st = Stack(dev, pkg, layers, topk)
    lib = dev.lib
    try:
        plan = st.plan()
        xs = pkg.synth.hidden(71, 8, H)
        want1 = [st.one_layer(s % n_layers, x) for s, x in enumerate(xs)]      # step s = layer s mod 3
        wantL = [st.run(plan, x, n_layers)[0] for x in xs[:3]]
        y = np.zeros(H, np.float32)

        def step(ses, x):
            x = np.ascontiguousarray(x, np.float32)
            assert lib.q4_cuda_decode_session_step(ses, x.ctypes.data, y.ctypes.data)
            return y.copy()
        ses = lib.q4_cuda_decode_session_begin(plan, 1, 5, 150)      # at most 5 steps per launch, 150 ms idle
        assert ses
        assert not lib.q4_cuda_decode_session_begin(plan, 1, 0, 0), "one session at a time"
        # while the session's kernel is resident the launching decode calls answer false
        assert not lib.q4_cuda_decode_stack_dev(plan, st.d_x, st.d_y, None, None)
        for s in range(8):                  # crosses the 5-step limit: the kernel is started again where it was
            got = step(ses, xs[s])
            assert np.array_equal(got.view(np.uint32), want1[s].view(np.uint32)), s
        time.sleep(0.4)                     # beyond the idle limit: the kernel has left
        got = step(ses, xs[2])              # step 8: layer 8 mod 3 = 2
        assert np.array_equal(got.view(np.uint32), want1[2].view(np.uint32))
        assert lib.q4_cuda_decode_session_end(ses)
        assert lib.q4_cuda_device_error() == 0
        ses = lib.q4_cuda_decode_session_begin(plan, 0, 0, 0)        # every layer of the plan per step
        assert ses
        for x, w in zip(xs[:3], wantL):
            assert np.array_equal(step(ses, x).view(np.uint32), w.view(np.uint32))
        lib.q4_cuda_decode_stack_free(plan)                          # ends the session that runs on the plan
        plan = st.plan()
        assert np.array_equal(st.run(plan, xs[0], n_layers)[0].view(np.uint32), wantL[0].view(np.uint32))
        lib.q4_cuda_decode_stack_free(plan)
        assert lib.q4_cuda_device_error() == 0
    finally:
        st.close()


def test_shared_expert_gate_and_stream_epilogue(dev, pkg, oracle):
    """The two optional extras of a plan.  set_sgate: the shared expert enters with weight
    sigmoid(sgate . xn) (src/q4_moe.c:1404-1435) -- against the oracle's routed sum plus the gated
    shared expert.  set_final: the last layer also updates the hc residual streams -- bit for bit
    what q4_hip_moe_final does with the layer's y (src/q4_rocm.cu:15990-16003)."""
    n_expert, topk, hc = 64, 6, 4
    L = pkg.synth.layer(900, n_expert, H, F)
    st = Stack(dev, pkg, [L], topk)
    lib = dev.lib
    rng = np.random.default_rng(91)
    try:
        plan = st.plan()
        x = pkg.synth.hidden(92, 1, H)[0]
        y_plain = st.run(plan, x, 1)[0]
        sg = (rng.standard_normal(H) * 0.05).astype(np.float32)
        assert lib.q4_cuda_decode_stack_set_sgate(plan, 0, dev.upload(sg))
        assert not lib.q4_cuda_decode_stack_set_sgate(plan, 1, None)
        y_g = st.run(plan, x, 1)[0]
        y_routed, ids, wts, xn = oracle.moe_layer(x, L["norm_w"], 1e-6, L["router"], topk, L["experts"], None, H, F)
        gate = 1.0 / (1.0 + np.exp(-float(np.dot(sg.astype(np.float64), xn.astype(np.float64)))))
        assert 0.02 < gate < 0.98
        want = y_routed + oracle.expert_job([L["shared"]], [np.float32(gate)], xn, H, F)
        assert _rel(y_g, want) <= REL_TOL
        assert _rel(y_g, y_plain) > 1e-2, "the gate must have changed the result"
        assert lib.q4_cuda_decode_stack_set_sgate(plan, 0, None)
        assert np.array_equal(st.run(plan, x, 1)[0].view(np.uint32), y_plain.view(np.uint32))
        # the stream epilogue
        res0 = rng.standard_normal((hc, H)).astype(np.float32)
        inj = rng.standard_normal(hc).astype(np.float32)
        zeros = dev.upload(np.zeros(H, np.float32))
        d_inj = dev.upload(inj)
        d_res_a, d_res_b = dev.upload(res0), dev.upload(res0)
        assert lib.q4_hip_moe_final(d_res_a, st.d_y, zeros, zeros, None, d_inj, H, hc)   # st.d_y holds y_plain
        assert lib.q4_cuda_decode_stack_set_final(plan, d_res_b, d_inj, hc)
        assert not lib.q4_cuda_decode_stack_set_final(plan, d_res_b, d_inj, 65)
        y2 = st.run(plan, x, 1)[0]
        assert np.array_equal(y2.view(np.uint32), y_plain.view(np.uint32))
        ra, rb = dev.download(d_res_a, (hc, H), np.float32), dev.download(d_res_b, (hc, H), np.float32)
        assert np.array_equal(ra.view(np.uint32), rb.view(np.uint32))
        f = 2.0 / (1.0 + np.exp(-inj.astype(np.float64) / hc))
        assert np.abs(rb - (res0 + y_plain[None, :] * f[:, None])).max() <= 1e-5 * np.abs(rb).max()
        assert lib.q4_cuda_decode_stack_set_final(plan, None, None, 0)
        st.run(plan, x, 1)
        assert np.array_equal(dev.download(d_res_b, (hc, H), np.float32).view(np.uint32), rb.view(np.uint32))
        lib.q4_cuda_decode_stack_free(plan)
        assert lib.q4_cuda_device_error() == 0
    finally:
        st.close()
