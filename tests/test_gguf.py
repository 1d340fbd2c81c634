"""Expert packs out of a GGUF file (suzuku-engine-q4_b200/host/q4_gguf_experts.c): the test
writes a small model file itself -- metadata of every value kind, a custom alignment, the three
stacked expert tensors of two layers, shared-expert tensors, unrelated tensors in between -- and
checks the slicing against the bytes it wrote (src/q4_expert.c:962-993 defines the pack as
gate | up | down slices of the stacked tensors).  The GPU part loads a layer into an arena
through the C host and runs experts from it."""
import ctypes as C
import os
import struct
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "suzuku-engine-q4_b200")
BUILD = os.path.join(ROOT, "tests", "host_c", "_build")
IQ3_S, IQ4_NL, F32 = 21, 20, 0


def _gstr(s):
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, tensors, alignment=64):
    """tensors: list of (name, ggml type, ne tuple (fastest first), bytes)."""
    kv = [
        (b"general.architecture", 8, _gstr("qwen-test")),
        (b"general.alignment", 4, struct.pack("<I", alignment)),
        (b"test.u8", 0, struct.pack("<B", 7)), (b"test.i16", 3, struct.pack("<h", -3)),
        (b"test.f32", 6, struct.pack("<f", 1.5)), (b"test.bool", 7, struct.pack("<B", 1)),
        (b"test.u64", 10, struct.pack("<Q", 1 << 40)), (b"test.f64", 12, struct.pack("<d", 2.5)),
        (b"test.arr_i32", 9, struct.pack("<IQ", 5, 3) + struct.pack("<3i", 1, 2, 3)),
        (b"tokenizer.tokens", 9, struct.pack("<IQ", 8, 3) + _gstr("a") + _gstr("bc") + _gstr("")),
    ]
    head = struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(kv))
    for k, t, v in kv:
        head += struct.pack("<Q", len(k)) + k + struct.pack("<I", t) + v
    off, infos, blobs = 0, b"", []
    for name, typ, ne, data in tensors:
        infos += _gstr(name) + struct.pack("<I", len(ne)) + b"".join(struct.pack("<Q", n) for n in ne)
        infos += struct.pack("<IQ", typ, off)
        blobs.append((off, data))
        off = (off + len(data) + alignment - 1) // alignment * alignment
    head += infos
    data_off = (len(head) + alignment - 1) // alignment * alignment
    with open(path, "wb") as f:
        f.write(head + b"\0" * (data_off - len(head)))
        for o, d in blobs:
            f.seek(data_off + o)
            f.write(d)
    return data_off


class Tensor(C.Structure):
    _fields_ = [("name", C.c_char * 128), ("n_dims", C.c_uint32), ("ne", C.c_uint64 * 4), ("type", C.c_uint32),
                ("offset", C.c_uint64), ("nbytes", C.c_uint64)]


class Gguf(C.Structure):
    _fields_ = [("fd", C.c_int), ("version", C.c_uint32), ("n_tensors", C.c_uint64), ("data_off", C.c_uint64),
                ("alignment", C.c_uint32), ("tensors", C.POINTER(Tensor))]


def _lib(with_device):
    os.makedirs(BUILD, exist_ok=True)
    out = os.path.join(BUILD, "libq4host_dev.so" if with_device else "libq4gguf.so")
    src = [os.path.join(PKG, "host", "q4_gguf_experts.c")]
    cmd = ["gcc", "-O2", "-std=c11", "-Wall", "-Werror", "-fPIC", "-shared", "-o", out]
    if with_device:
        src.append(os.path.join(PKG, "host", "q4_moe_b200.c"))
        cmd += src + ["-L", PKG, "-lq4cuda", "-Wl,-rpath," + PKG]
    else:
        cmd += src
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    lib = C.CDLL(out)
    lib.q4b_gguf_open.restype = C.c_bool
    lib.q4b_gguf_expert_parts.restype = C.c_bool
    lib.q4b_gguf_read_pack.restype = C.c_int64
    lib.q4b_gguf_read_shared_pack.restype = C.c_int64
    lib.q4b_gguf_row_bytes.restype = C.c_uint64
    lib.q4b_gguf_find.restype = C.POINTER(Tensor)
    return lib


def _model(rng, H, F, E, layers, down_type=IQ3_S):
    """Stacked tensors of `layers` layers + shared-expert tensors for layer 0; returns (tensor list, expected)."""
    rbg = H // 256 * 110
    rbd = F // 256 * 110 if down_type == IQ3_S else F // 32 * 18
    tensors, want = [("token_embd.weight", F32, (8, 4), rng.bytes(8 * 4 * 4))], {}
    for l in range(layers):
        g, u = (rng.integers(0, 256, (E, F * rbg), dtype=np.uint8) for _ in range(2))
        d = rng.integers(0, 256, (E, H * rbd), dtype=np.uint8)
        tensors += [("blk.%d.ffn_gate_exps.weight" % l, IQ3_S, (H, F, E), g.tobytes()),
                    ("blk.%d.attn_norm.weight" % l, F32, (H,), rng.bytes(H * 4)),
                    ("blk.%d.ffn_up_exps.weight" % l, IQ3_S, (H, F, E), u.tobytes()),
                    ("blk.%d.ffn_down_exps.weight" % l, down_type, (F, H, E), d.tobytes())]
        want[l] = np.concatenate([g, u, d], axis=1)
    sh = [rng.integers(0, 256, n, dtype=np.uint8) for n in (F * rbg, F * rbg, H * rbd)]
    tensors += [("blk.0.ffn_gate_shexp.weight", IQ3_S, (H, F), sh[0].tobytes()),
                ("blk.0.ffn_up_shexp.weight", IQ3_S, (H, F), sh[1].tobytes()),
                ("blk.0.ffn_down_shexp.weight", down_type, (F, H), sh[2].tobytes())]
    want["shared"] = np.concatenate(sh)
    return tensors, want


@pytest.mark.parametrize("down_type", [IQ3_S, IQ4_NL])
def test_gguf_slicing(tmp_path, down_type):
    lib = _lib(False)
    rng = np.random.default_rng(4)
    H, F, E = 512, 256, 5
    tensors, want = _model(rng, H, F, E, 2, down_type)
    path = str(tmp_path / "m.gguf")
    data_off = write_gguf(path, tensors, alignment=64)
    g = Gguf()
    assert lib.q4b_gguf_open(C.byref(g), path.encode())
    assert g.version == 3 and g.n_tensors == len(tensors) and g.alignment == 64 and g.data_off == data_off
    assert lib.q4b_gguf_row_bytes(IQ3_S, 2048) == 880 and lib.q4b_gguf_row_bytes(IQ3_S, 100) == 0
    t = lib.q4b_gguf_find(C.byref(g), b"blk.1.ffn_down_exps.weight")
    assert t and t.contents.type == down_type and list(t.contents.ne[:3]) == [F, H, E]
    tg, tu, td = (C.POINTER(Tensor)() for _ in range(3))
    og, ou, od, tot = (C.c_uint64() for _ in range(4))
    ne = C.c_uint32()
    assert lib.q4b_gguf_expert_parts(C.byref(g), 1, C.byref(tg), C.byref(tu), C.byref(td), C.byref(og), C.byref(ou),
                                     C.byref(od), C.byref(tot), C.byref(ne))
    sg = F * (H // 256 * 110)
    assert (og.value, ou.value, od.value, tot.value, ne.value) == (0, sg, 2 * sg, want[1].shape[1], E)
    buf = np.zeros(tot.value, np.uint8)
    for l in (0, 1):
        for e in range(E):
            assert lib.q4b_gguf_read_pack(C.byref(g), l, e, C.c_void_p(buf.ctypes.data)) == tot.value
            assert np.array_equal(buf, want[l][e])
    assert lib.q4b_gguf_read_pack(C.byref(g), 0, E, C.c_void_p(buf.ctypes.data)) == -1          # no such expert
    assert not lib.q4b_gguf_expert_parts(C.byref(g), 2, None, None, None, None, None, None, None, None)   # no such layer
    assert lib.q4b_gguf_read_shared_pack(C.byref(g), 0, C.c_void_p(buf.ctypes.data), C.c_uint64(tot.value)) == tot.value
    assert np.array_equal(buf, want["shared"])
    assert lib.q4b_gguf_read_shared_pack(C.byref(g), 1, C.c_void_p(buf.ctypes.data), C.c_uint64(tot.value)) == -1
    lib.q4b_gguf_close(C.byref(g))
    # a file that is not GGUF, and a truncated one, are refused
    bad = str(tmp_path / "bad.gguf")
    open(bad, "wb").write(b"GGML" + b"\0" * 64)
    assert not lib.q4b_gguf_open(C.byref(g), bad.encode())
    open(bad, "wb").write(open(path, "rb").read()[:200])
    assert not lib.q4b_gguf_open(C.byref(g), bad.encode())


class Layer(C.Structure):
    _fields_ = [("arena", C.c_int), ("first_slot", C.c_uint32), ("shared_slot", C.c_int32), ("n_embd", C.c_uint32),
                ("n_ff", C.c_uint32), ("n_expert", C.c_uint32), ("topk", C.c_uint32), ("og", C.c_uint64),
                ("ou", C.c_uint64), ("od", C.c_uint64), ("d_router", C.c_void_p), ("d_norm_w", C.c_void_p),
                ("eps", C.c_float)]


@pytest.mark.gpu
def test_gguf_layer_into_an_arena_and_run(tmp_path, dev, pkg, oracle):
    lib = _lib(True)
    lib.q4b_moe_layer_load_gguf.restype = C.c_bool
    rng = np.random.default_rng(6)
    H, F, E = 2048, 512, 4
    # packs with sane scales, stacked the way a model file stores them
    packs = pkg.synth.expert_packs(rng, E + 1, H, F)
    sg = F * (H // 256 * 110)
    tensors = [("blk.0.ffn_gate_exps.weight", IQ3_S, (H, F, E), packs[:E, :sg].tobytes()),
               ("blk.0.ffn_up_exps.weight", IQ3_S, (H, F, E), packs[:E, sg:2 * sg].tobytes()),
               ("blk.0.ffn_down_exps.weight", IQ3_S, (F, H, E), packs[:E, 2 * sg:].tobytes()),
               ("blk.0.ffn_gate_shexp.weight", IQ3_S, (H, F), packs[E, :sg].tobytes()),
               ("blk.0.ffn_up_shexp.weight", IQ3_S, (H, F), packs[E, sg:2 * sg].tobytes()),
               ("blk.0.ffn_down_shexp.weight", IQ3_S, (F, H), packs[E, 2 * sg:].tobytes())]
    path = str(tmp_path / "l.gguf")
    write_gguf(path, tensors, alignment=32)
    g, L = Gguf(), Layer()
    assert lib.q4b_gguf_open(C.byref(g), path.encode())
    dlib = dev.lib
    try:
        assert lib.q4b_moe_layer_load_gguf(C.byref(L), 3, C.byref(g), 0)
        assert (L.n_embd, L.n_ff, L.n_expert, L.shared_slot, L.ou, L.od) == (H, F, E, E, sg, 2 * sg)
        assert dlib.q4_cuda_experts_tiled_a(3) == 1
        back = np.zeros(packs.shape[1], np.uint8)
        for e in range(E + 1):
            assert dlib.q4_cuda_experts_get_a(3, e, back.ctypes.data, back.nbytes)
            assert np.array_equal(back, packs[e])
        base, stride = dlib.q4_hip_experts_base_a(3), dlib.q4_hip_experts_stride_a(3)
        x = rng.standard_normal(H).astype(np.float32)
        slots, wts = np.array([3, E, 1], np.int32), np.array([0.5, 1.0, 0.25], np.float32)
        d_x, d_y, d_h = dev.upload(x), dev.malloc(H * 4), dev.malloc(64 * F * 4)
        assert dlib.q4_hip_fill(d_y, 0.0, H)
        assert dlib.q4_hip_moe_exec(base, stride, slots.ctypes.data, wts.ctypes.data, 3, IQ3_S, L.og, IQ3_S, L.ou,
                                    IQ3_S, L.od, d_x, d_h, None, None, d_y, F, H, H)
        y = dev.download(d_y, (H,), np.float32)
        want = oracle.expert_job([packs[s] for s in slots], wts, x, H, F)
        assert np.linalg.norm(y - want) / np.linalg.norm(want) <= 1e-3
    finally:
        dlib.q4_hip_experts_free_a(3)
        lib.q4b_gguf_close(C.byref(g))
