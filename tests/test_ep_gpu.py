"""Expert-parallel layer on 2 GPUs (one process per GPU, NCCL) against the single-GPU
layer and the CPU oracle.  Skipped on a box with one GPU."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _n_gpus():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=30).stdout
    except Exception:
        return 0
    return sum(1 for line in out.splitlines() if line.startswith("GPU "))


@pytest.mark.skipif(_n_gpus() < 2, reason="needs two GPUs")
def test_ep_layer_two_gpus(tmp_path, dev, pkg, oracle):
    world, port = 2, 29000 + os.getpid() % 2000
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "ep_gpu_worker.py"), str(r), str(world),
                               str(port), str(tmp_path)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                              text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            pytest.fail("expert-parallel ranks timed out")
        outs.append(o)
    for r, p in enumerate(procs):
        assert p.returncode == 0, outs[r][-3000:]
    y = np.concatenate([np.load(os.path.join(str(tmp_path), "y%d.npy" % r)) for r in range(world)])
    H, F, E, K, T = 2048, 512, 16, 4, 10
    L = pkg.synth.layer(7, E, H, F)
    xs = pkg.synth.hidden(8, T, H)
    # single GPU, same library
    layer = pkg.MoeLayer(dev, L["experts"], L["shared"], L["router"], L["norm_w"], H, F, K)
    lib = dev.lib
    ws = lib.q4_cuda_moe_layer_n_ws_bytes(T, K, E, H, F)
    d_ws, d_x, d_y = dev.malloc(ws), dev.upload(xs), dev.malloc(T * H * 4)
    assert lib.q4_cuda_moe_layer_n(layer.base, layer.stride, layer.og, layer.ou, layer.od, E, d_x,
                                   layer.d_norm, 1e-6, layer.d_router, E, K, H, F, T, d_y, None, None,
                                   d_ws, ws)
    y1 = dev.download(d_y, (T, H), np.float32)
    layer.close()
    for t in range(T):
        y0 = oracle.moe_layer(xs[t], L["norm_w"], 1e-6, L["router"], K, L["experts"], L["shared"], H, F)[0]
        n0 = np.linalg.norm(y0)
        assert np.linalg.norm(y[t] - y1[t]) / n0 < 1e-5        # only the summation order differs
        assert np.linalg.norm(y[t] - y0) / n0 < 1e-3
    # the one-collective form: every rank ends with all rows, the same on every rank
    ya = [np.load(os.path.join(str(tmp_path), "ya%d.npy" % r)) for r in range(world)]
    assert np.array_equal(ya[0], ya[1])
    modes = [open(os.path.join(str(tmp_path), "mode%d.txt" % r)).read() for r in range(world)]
    assert modes[0] == modes[1]
    print("all-reduce of the one-collective form: %s" %
          ("the library's kernel over peer memory" if modes[0] == "1" else "ncclAllReduce (peer buffers not mapped)"))
    for t in range(T):
        n0 = np.linalg.norm(y1[t])
        assert np.linalg.norm(ya[0][t] - y1[t]) / n0 < 1e-5
