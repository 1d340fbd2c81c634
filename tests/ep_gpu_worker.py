"""One rank of the expert-parallel layer on its own GPU (libq4cuda_ep.so over NCCL).

argv: rank world port out_dir.  Writes y of its tokens to out_dir/y<rank>.npy; the parent
test compares the concatenation with the single-GPU layer and the CPU oracle.  torch is
not imported: the process binds the system NCCL through the library."""
import ctypes
import os
import socket
import sys
import time

import numpy as np

rank, world, port, out_dir = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
os.environ["CUDA_VISIBLE_DEVICES"] = str(rank)
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

H, F, E, K, T_LOCAL = 2048, 512, 16, 4, 5


def swap_id(make):
    if rank == 0:
        ident = make()
        srv = socket.socket()
        srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        srv.bind(("127.0.0.1", port))
        srv.listen(world)
        for _ in range(world - 1):
            c, _ = srv.accept()
            c.sendall(ident)
            c.close()
        srv.close()
        return ident
    end = time.time() + 60
    while True:
        try:
            c = socket.create_connection(("127.0.0.1", port), timeout=5)
            break
        except OSError:
            if time.time() > end:
                raise
            time.sleep(0.2)
    buf = b""
    while len(buf) < 128:
        part = c.recv(128 - len(buf))
        assert part
        buf += part
    return buf


def main():
    pkg = entry.load_package()
    dev = pkg.Device()
    lib = dev.lib
    ep = pkg.capi.load_ep()

    def make():
        b = ctypes.create_string_buffer(128)
        assert ep.q4_cuda_ep_unique_id(b)
        return b.raw
    assert ep.q4_cuda_ep_init(swap_id(make), rank, world)
    assert ep.q4_cuda_ep_rank() == rank and ep.q4_cuda_ep_world() == world
    L = pkg.synth.layer(7, E, H, F)
    xs = pkg.synth.hidden(8, world * T_LOCAL, H)
    first, count = pkg.host.ep_expert_range(rank, world, E)
    pack = pkg.synth.expert_pack_bytes(H, F)
    assert lib.q4_hip_experts_alloc_a(0, count + 1, pack)
    for j in range(count):
        row = np.ascontiguousarray(L["experts"][first + j])
        assert lib.q4_hip_experts_put_a(0, j, row.ctypes.data, pack)
    sh = np.ascontiguousarray(L["shared"])
    assert lib.q4_hip_experts_put_a(0, count, sh.ctypes.data, pack)
    base, stride = lib.q4_hip_experts_base_a(0), lib.q4_hip_experts_stride_a(0)
    rb = pkg.synth.iq3s_row_bytes(H)
    d_x = dev.upload(xs[rank * T_LOCAL:(rank + 1) * T_LOCAL])
    d_y = dev.malloc(T_LOCAL * H * 4)
    d_router, d_norm = dev.upload(L["router"]), dev.upload(L["norm_w"])
    ws = ep.q4_cuda_ep_layer_ws_bytes(world, T_LOCAL, K, E, H, F)
    d_ws = dev.malloc(ws)
    # refusals: scratch too small, expert count not divisible
    assert not ep.q4_cuda_ep_layer(base, stride, 0, F * rb, 2 * F * rb, 1, d_x, d_norm, 1e-6, d_router,
                                   E, K, H, F, T_LOCAL, d_y, d_ws, ws - 1)
    assert not ep.q4_cuda_ep_layer(base, stride, 0, F * rb, 2 * F * rb, 1, d_x, d_norm, 1e-6, d_router,
                                   E + 1, K, H, F, T_LOCAL, d_y, d_ws, ws)
    ys = []
    for _ in range(2):      # twice: the scratch carries nothing from call to call
        assert ep.q4_cuda_ep_layer(base, stride, 0, F * rb, 2 * F * rb, 1, d_x, d_norm, 1e-6, d_router,
                                   E, K, H, F, T_LOCAL, d_y, d_ws, ws)
        dev.sync()
        ys.append(dev.download(d_y, (T_LOCAL, H), np.float32))
    assert np.array_equal(ys[0], ys[1])
    # the one-collective form: all token rows on every rank, one all-reduce; the rows of this
    # rank's tokens must agree with the two-exchange form (another order of the sum over ranks)
    d_xa = dev.upload(xs)
    d_ya = dev.malloc(world * T_LOCAL * H * 4)
    assert ep.q4_cuda_ep_layer_ar(base, stride, 0, F * rb, 2 * F * rb, 1, d_xa, d_norm, 1e-6, d_router,
                                  E, K, H, F, T_LOCAL, d_ya, d_ws, ws)
    dev.sync()
    ya = dev.download(d_ya, (world * T_LOCAL, H), np.float32)
    mine = ya[rank * T_LOCAL:(rank + 1) * T_LOCAL]
    assert np.linalg.norm(mine - ys[0]) <= 1e-5 * np.linalg.norm(ys[0])
    np.save(os.path.join(out_dir, "ya%d.npy" % rank), ya)
    # the all-reduce itself: the library's kernel over mapped peer memory where every rank could map
    # the others' buffers (mode 1), else ncclAllReduce.  Repeated calls give the same bits (sum in rank
    # order; the two buffer copies alternate), and the two modes agree up to the order of the sum.
    mode = ep.q4_cuda_ep_allreduce_mode(1)        # ask for the kernel (also the default where the buffers could be mapped)
    open(os.path.join(out_dir, "mode%d.txt" % rank), "w").write(str(mode))
    for _ in range(5):
        assert ep.q4_cuda_ep_layer_ar(base, stride, 0, F * rb, 2 * F * rb, 1, d_xa, d_norm, 1e-6, d_router,
                                      E, K, H, F, T_LOCAL, d_ya, d_ws, ws)
        dev.sync()
        again = dev.download(d_ya, (world * T_LOCAL, H), np.float32)
        if mode == 1:
            assert np.array_equal(again.view(np.uint32), ya.view(np.uint32))
    assert ep.q4_cuda_ep_error() == 0
    assert ep.q4_cuda_ep_allreduce_mode(0) == 0
    assert ep.q4_cuda_ep_layer_ar(base, stride, 0, F * rb, 2 * F * rb, 1, d_xa, d_norm, 1e-6, d_router,
                                  E, K, H, F, T_LOCAL, d_ya, d_ws, ws)
    dev.sync()
    nccl = dev.download(d_ya, (world * T_LOCAL, H), np.float32)
    assert np.linalg.norm(nccl - ya) <= 1e-6 * np.linalg.norm(ya)
    if mode == 1:
        # a rank routes only its own tokens, the picks are gathered through peer memory: the same bits
        ep.q4_cuda_ep_split_routing(1)
        for _ in range(3):
            assert ep.q4_cuda_ep_layer_ar(base, stride, 0, F * rb, 2 * F * rb, 1, d_xa, d_norm, 1e-6, d_router,
                                          E, K, H, F, T_LOCAL, d_ya, d_ws, ws)
            dev.sync()
            got = dev.download(d_ya, (world * T_LOCAL, H), np.float32)
            assert np.array_equal(got.view(np.uint32), ya.view(np.uint32))
        assert ep.q4_cuda_ep_error() == 0
        ep.q4_cuda_ep_split_routing(0)
    ep.q4_cuda_ep_allreduce_mode(2)
    f2 = (ctypes.c_float * 2)()
    assert ep.q4_cuda_ep_exchange_floor_us(T_LOCAL, H, K, E, F, d_ws, ws, 5, f2) and f2[0] > 0 and f2[1] > 0
    assert lib.q4_cuda_device_error() == 0
    f = ctypes.c_float(float(rank + 1))
    assert ep.q4_cuda_ep_allreduce_max(ctypes.byref(f)) and f.value == float(world)
    np.save(os.path.join(out_dir, "y%d.npy" % rank), ys[0])
    ep.q4_cuda_ep_shutdown()
    print("rank %d ok" % rank)


if __name__ == "__main__":
    main()
