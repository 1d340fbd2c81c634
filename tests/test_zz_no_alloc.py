"""The allocation-free expert entry point (collected last on purpose).

Some hosts cannot allocate device memory by the time experts run: the engine's
planner has given all free memory to expert slots, or a stream capture is open, or
the loop cannot afford an allocation's device-wide sync.  For them the library has
one entry point whose scratch is a fixed array in the library image.  Here it is
called through the C ABI twice in a row, with different inputs, on a tiled arena and on
one in the engine's byte order, on the library's stream and on one the caller made, and
must give what the ordinary entry point (q4_hip_moe_exec_dev) gives for the same inputs:
the hidden rows bit for bit (the same kernels on the same bytes), y up to the order of
the atomic adds, and both within the expert tolerance of the CPU oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

IQ3_S = 21
REL_TOL = 1e-3   # the tolerance the expert-output tests use


def _rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b), 1e-30))


def _caller_stream():
    """A stream of the caller's own (CUDA runtime through cuda-python); (handle, sync, destroy)."""
    from cuda.bindings import runtime as rt
    err, st = rt.cudaStreamCreateWithFlags(rt.cudaStreamNonBlocking)
    assert int(err) == 0, err
    return int(st), (lambda: rt.cudaStreamSynchronize(st)), (lambda: rt.cudaStreamDestroy(st))


@pytest.mark.parametrize("tiled,own_stream", [(True, False), (False, False), (True, True)])
def test_no_alloc_entry_matches_exec_dev_twice(dev, pkg, oracle, tiled, own_stream):
    H, F, n_slots = 2048, 512, 12
    rng = np.random.default_rng(77)
    packs = pkg.synth.expert_packs(rng, n_slots, H, F)
    lib = dev.lib
    lib.q4_cuda_set_tiled_default(1 if tiled else 0)
    try:
        layer = pkg.MoeLayer(dev, packs, None, np.zeros((n_slots, H), np.float32), None, H, F, 1, arena=3)
    finally:
        lib.q4_cuda_set_tiled_default(1)
    assert bool(lib.q4_cuda_experts_tiled_a(3)) == tiled
    stream, sync, destroy = lib.q4_hip_stream(), dev.sync, (lambda: None)
    if own_stream:
        stream, sync, destroy = _caller_stream()
    try:
        d_h2 = dev.malloc(16 * F * 4)
        d_y2 = dev.malloc(H * 4)
        for call in range(2):
            n = 5 + 3 * call
            slots = rng.choice(n_slots, n, replace=False).astype(np.int32)
            wts = rng.random(n).astype(np.float32)
            x = rng.standard_normal(H).astype(np.float32)
            d_es, d_ew, d_n = dev.upload(slots), dev.upload(wts), dev.upload(np.array([n], np.int32))
            dev.write(layer.d_x, x)
            # the existing entry point
            assert lib.q4_hip_fill(layer.d_y, 0.0, H)
            assert lib.q4_hip_moe_exec_dev(layer.base, layer.stride, d_es, d_ew, d_n, IQ3_S, layer.og,
                                           IQ3_S, layer.ou, IQ3_S, layer.od, layer.d_x, layer.d_h,
                                           None, None, layer.d_y, F, H, H)
            y_ref = dev.download(layer.d_y, (H,), np.float32)
            h_ref = dev.download(layer.d_h, (n, F), np.float32)
            # the allocation-free one (the zero fill of its y goes through the library's stream:
            # wait for it before another stream adds to y)
            assert lib.q4_hip_fill(d_y2, 0.0, H)
            dev.sync()
            assert lib.q4_cuda_moe_exec_noalloc(layer.base, layer.stride, d_es, d_ew, n, layer.og,
                                                layer.ou, layer.od, layer.d_x, d_h2, d_y2, F, H, H,
                                                stream)
            sync()
            y = dev.download(d_y2, (H,), np.float32)
            h = dev.download(d_h2, (n, F), np.float32)
            assert np.isfinite(y).all() and np.abs(y_ref).max() > 0
            assert np.array_equal(h.view(np.uint32), h_ref.view(np.uint32))
            assert _rel(y, y_ref) <= 1e-5          # the same terms, added by atomics in any order
            y0 = oracle.expert_job([packs[i] for i in slots], wts, x, H, F)
            assert _rel(y, y0) <= REL_TOL and _rel(y_ref, y0) <= REL_TOL
        # sizes beyond the fixed scratch are refused, nothing is queued
        big = dev.upload(np.zeros(17, np.int32))
        assert not lib.q4_cuda_moe_exec_noalloc(layer.base, layer.stride, big, d_ew, 17, layer.og,
                                                layer.ou, layer.od, layer.d_x, d_h2, d_y2, F, H, H,
                                                stream)
        assert not lib.q4_cuda_moe_exec_noalloc(layer.base, layer.stride, d_es, d_ew, 2, layer.og,
                                                layer.ou, layer.od, layer.d_x, d_h2, d_y2, 4096, H, H,
                                                stream)
        assert not lib.q4_cuda_moe_exec_noalloc(layer.base, layer.stride, d_es, d_ew, 2, layer.og,
                                                layer.ou, layer.od, layer.d_x, d_h2, d_y2, F, 8192, H,
                                                stream)
        sync()
        assert lib.q4_cuda_device_error() == 0
    finally:
        destroy()
        layer.close()
