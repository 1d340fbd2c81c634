"""The allocation-free expert entry point (collected last on purpose).

Some hosts cannot allocate device memory by the time experts run: the engine's
planner has given all free memory to expert slots, or a stream capture is open, or
the loop cannot afford an allocation's device-wide sync.  For them the library has
one entry point whose scratch is a fixed array in the library image.  Here it is
called through the C ABI twice in a row, with different inputs, and must give what
the ordinary entry point (q4_hip_moe_exec_dev) gives for the same inputs."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

IQ3_S = 21
REL_TOL = 1e-3   # the tolerance the expert-output tests use


def _rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b), 1e-30))


def test_no_alloc_entry_matches_exec_dev_twice(dev, pkg):
    H, F, n_slots = 2048, 512, 12
    rng = np.random.default_rng(77)
    packs = pkg.synth.expert_packs(rng, n_slots, H, F)
    layer = pkg.MoeLayer(dev, packs, None, np.zeros((n_slots, H), np.float32), None, H, F, 1, arena=3)
    lib = dev.lib
    try:
        d_h2 = dev.malloc(16 * F * 4)
        d_y2 = dev.malloc(H * 4)
        stream = lib.q4_hip_stream()
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
            # the allocation-free one, on the same stream
            assert lib.q4_hip_fill(d_y2, 0.0, H)
            assert lib.q4_cuda_moe_exec_noalloc(layer.base, layer.stride, d_es, d_ew, n, layer.og,
                                                layer.ou, layer.od, layer.d_x, d_h2, d_y2, F, H, H,
                                                stream)
            y = dev.download(d_y2, (H,), np.float32)
            h = dev.download(d_h2, (n, F), np.float32)
            assert np.isfinite(y).all() and np.abs(y_ref).max() > 0
            assert _rel(h, h_ref) <= REL_TOL
            assert _rel(y, y_ref) <= REL_TOL
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
        assert lib.q4_cuda_device_error() == 0
    finally:
        layer.close()
