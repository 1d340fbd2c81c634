"""The arena's tiled storage format: a lossless permutation of the engine's
bytes, and every kernel gives the same answers on it."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def _rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b), 1e-30))


@pytest.fixture()
def arena(dev, pkg):
    made = []

    def make(packs, tiled=True, arena_id=2):
        lib = dev.lib
        lib.q4_cuda_set_tiled_default(2 if tiled else 0)   # 2: these slots hold IQ3_S bytes only, whatever their size
        assert lib.q4_hip_experts_alloc_a(arena_id, packs.shape[0], packs.shape[1])
        lib.q4_cuda_set_tiled_default(1)
        made.append(arena_id)
        for i in range(packs.shape[0]):
            row = np.ascontiguousarray(packs[i])
            assert lib.q4_hip_experts_put_a(arena_id, i, row.ctypes.data, row.nbytes)
        return arena_id

    yield make
    for a in made:
        dev.lib.q4_hip_experts_free_a(a)


def test_put_get_round_trip_is_identity(dev, arena):
    rng = np.random.default_rng(0)
    packs = rng.integers(0, 256, size=(3, 880 * 37), dtype=np.uint8)
    a = arena(packs, tiled=True)
    assert dev.lib.q4_cuda_experts_tiled_a(a) == 1
    raw = dev.download(dev.lib.q4_hip_experts_dev_a(a, 1), (packs.shape[1],), np.uint8)
    assert not np.array_equal(raw, packs[1])                      # stored permuted ...
    assert np.array_equal(np.sort(raw.reshape(-1, 880)[:, :112], axis=1),
                          np.sort(np.concatenate([packs[1].reshape(-1, 8, 110)[:, :, 0:2].reshape(-1, 16),
                                                  packs[1].reshape(-1, 8, 110)[:, :, 106:110].reshape(-1, 32),
                                                  packs[1].reshape(-1, 8, 110)[:, :, 66:74].reshape(-1, 64)],
                                                 axis=1), axis=1))  # ... same bytes per tile
    for i in range(3):
        back = np.zeros(packs.shape[1], np.uint8)
        assert dev.lib.q4_cuda_experts_get_a(a, i, back.ctypes.data, back.nbytes)
        assert np.array_equal(back, packs[i])


def test_untiled_arena_keeps_bytes(dev, arena):
    rng = np.random.default_rng(1)
    packs = rng.integers(0, 256, size=(2, 880 * 4), dtype=np.uint8)
    a = arena(packs, tiled=False)
    assert dev.lib.q4_cuda_experts_tiled_a(a) == 0
    raw = dev.download(dev.lib.q4_hip_experts_dev_a(a, 1), (packs.shape[1],), np.uint8)
    assert np.array_equal(raw, packs[1])


def test_odd_slot_size_is_not_tiled(dev):
    lib = dev.lib
    assert lib.q4_hip_experts_alloc_a(3, 2, 880 * 3 + 110)
    try:
        assert lib.q4_cuda_experts_tiled_a(3) == 0
    finally:
        lib.q4_hip_experts_free_a(3)


def test_dequant_and_idot_on_tiled_arena(dev, pkg, oracle, arena):
    rng = np.random.default_rng(2)
    rows, cols = 16, 2048
    w = pkg.synth.iq3s_blocks(rng, rows * cols // 256).reshape(1, -1)
    a = arena(w, tiled=True)
    d_w = dev.lib.q4_hip_experts_dev_a(a, 0)
    d_o = dev.malloc(rows * cols * 4)
    assert dev.lib.q4_cuda_iq3s_dequant(d_w, rows, cols, d_o)
    got = dev.download(d_o, (rows, cols), np.float32)
    rb = cols // 256 * 110
    x = rng.standard_normal(cols).astype(np.float32)
    xq = oracle.quant8(x)
    d_I = dev.malloc(rows * cols // 32 * 4)
    assert dev.lib.q4_cuda_iq3s_idot(d_w, rows, cols, dev.upload(np.ascontiguousarray(xq["q"])), d_I)
    I = dev.download(d_I, (rows, cols // 32), np.int32)
    for r in range(rows):
        row = w[0][r * rb:(r + 1) * rb]
        assert np.array_equal(_bits(got[r]), _bits(oracle.dequant_row(row, cols)))
        assert np.array_equal(I[r], oracle.group_idot(row, xq, cols))


def test_down_shaped_matrix_on_tiled_arena(dev, pkg, oracle, arena):
    """Two super-blocks per row: a tile holds four rows."""
    rng = np.random.default_rng(3)
    rows, cols = 64, 512
    w = pkg.synth.iq3s_blocks(rng, rows * cols // 256).reshape(1, -1)
    a = arena(w, tiled=True)
    d_w = dev.lib.q4_hip_experts_dev_a(a, 0)
    x = rng.standard_normal(cols).astype(np.float32)
    xq = oracle.quant8(x)
    d_I = dev.malloc(rows * cols // 32 * 4)
    assert dev.lib.q4_cuda_iq3s_idot(d_w, rows, cols, dev.upload(np.ascontiguousarray(xq["q"])), d_I)
    I = dev.download(d_I, (rows, cols // 32), np.int32)
    rb = cols // 256 * 110
    for r in range(rows):
        assert np.array_equal(I[r], oracle.group_idot(w[0][r * rb:(r + 1) * rb], xq, cols))


@pytest.mark.parametrize("tiled", [True, False])
def test_layer_same_answer_in_both_formats(dev, pkg, oracle, tiled):
    """Tiled arena -> the single persistent kernel; engine byte order -> the launch chain."""
    H, F, E, K = 2048, 512, 64, 6
    L = pkg.synth.layer(31, E, H, F)
    x = pkg.synth.hidden(32, 1, H)[0]
    dev.lib.q4_cuda_set_tiled_default(1 if tiled else 0)
    try:
        layer = pkg.MoeLayer(dev, L["experts"], L["shared"], L["router"], L["norm_w"], H, F, K, arena=1)
    finally:
        dev.lib.q4_cuda_set_tiled_default(1)
    try:
        assert dev.lib.q4_cuda_experts_tiled_a(1) == (1 if tiled else 0)
        n0 = dev.lib.q4_cuda_launch_count()
        y, ids, wts = layer.decode(x)
        launches = dev.lib.q4_cuda_launch_count() - n0
        assert launches == (1 if tiled else 6)
        y0, ids0, w0, _ = oracle.moe_layer(x, L["norm_w"], 1e-6, L["router"], K, L["experts"],
                                           L["shared"], H, F)
        assert ids.tolist() == ids0.tolist()
        assert np.abs(wts - w0).max() <= 1e-6
        assert _rel(y, y0) <= 1e-3
        # the persistent kernel is reproducible bit for bit
        y2, _, _ = layer.decode(x)
        assert np.array_equal(_bits(y), _bits(y2))
        assert dev.lib.q4_cuda_device_error() == 0
    finally:
        layer.close()
