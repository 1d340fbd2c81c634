"""The dense product of up to 8 activation rows in 8-bit form (q4_mmvq_n) on Q6_K, Q4_K, Q5_K,
IQ4_XS and IQ4_NL weights, through the C ABI.

Mirrors the reference's own two tests of this product (src/q4_test.c:2658-2779): accuracy against
the dequantised weights in double (rel-L2 < 2e-2) for every type and 2..8 rows, and rows of calls of
1..7 activation rows bit-identical to the same rows of a call of 8 (K = 2560, R = 512) in the
verify-scope mode.  On top of that every value is compared bit for bit with the CPU oracle's
restatement of the product's arithmetic (src/q4_mmvq.cu:36-57, 195-243)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TYPES = {14: "Q6_K", 12: "Q4_K", 13: "Q5_K", 23: "IQ4_XS", 20: "IQ4_NL"}


def _bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def _weights(pkg, rng, ty, rows, K):
    return np.stack([pkg.synth.blocks_of(rng, ty, pkg.synth.row_bytes(ty, K)) for _ in range(rows)])


def _acts(rng, n, K):
    return (rng.integers(-1000, 1001, (n, K)) * 1e-3).astype(np.float32)     # src/q4_test.c:2685


@pytest.fixture()
def mv(dev):
    lib = dev.lib
    lib.q4_mmvq_warm()
    yield lib
    lib.q4_mmvq_release()
    lib.q4_mmvq_verify(0)
    lib.q4_mmvq_set(1)


@pytest.mark.parametrize("ty", sorted(TYPES))
def test_rows_match_oracle_bit_for_bit_and_dequantised_weights(dev, pkg, oracle, mv, ty):
    K, R = 2560, 256
    rng = np.random.default_rng(100 + ty)
    w = _weights(pkg, rng, ty, R, K)
    d_w = dev.upload(w)
    deq = np.stack([oracle.mv_dequant_row(ty, r, K) for r in w]).astype(np.float64)
    for n in range(2, 9):
        xs = _acts(rng, n, K)
        xs[0, 64:96] = 0.0                         # a group of zeros: d = 0, q = 0
        d_x, d_y = dev.upload(xs), dev.malloc(n * R * 4)
        assert mv.q4_mmvq_n(ty, d_w, R, K, d_x, d_y, 0.25, n), (TYPES[ty], n)
        y = dev.download(d_y, (n, R), np.float32)
        want = 0.25 * xs.astype(np.float64) @ deq.T
        assert np.linalg.norm(y - want) / np.linalg.norm(want) < 2e-2, (TYPES[ty], n)
        rows = range(0, R, 1 if n in (2, 8) else 17)
        ref = oracle.mv_rows(ty, w[list(rows)], len(rows), K, xs, 0.25)
        assert np.array_equal(_bits(y[:, list(rows)]), _bits(ref)), (TYPES[ty], n)
        dev.free(d_x)
        dev.free(d_y)
    assert dev.lib.q4_cuda_device_error() == 0


@pytest.mark.parametrize("ty", sorted(TYPES))
def test_a_row_does_not_depend_on_the_number_of_rows(dev, pkg, mv, ty):
    """src/q4_test.c:2736-2779: mode 2, inside a verify scope, 1..7 rows against 8."""
    K, R = 2560, 512
    rng = np.random.default_rng(200 + ty)
    w = _weights(pkg, rng, ty, R, K)
    xs = _acts(rng, 8, K)
    d_w, d_x, d_y = dev.upload(w), dev.upload(xs), dev.malloc(8 * R * 4)
    mv.q4_mmvq_set(2)
    assert mv.q4_mmvq_on() == 2
    assert not mv.q4_mmvq_n(ty, d_w, R, K, d_x, d_y, 1.0, 8), "mode 2 works inside a verify scope only"
    mv.q4_mmvq_verify(1)
    assert mv.q4_mmvq_n(ty, d_w, R, K, d_x, d_y, 1.0, 8)
    y8 = dev.download(d_y, (8, R), np.float32)
    assert np.abs(y8).max() > 0
    for n in range(1, 8):
        assert mv.q4_mmvq_n(ty, d_w, R, K, d_x, d_y, 1.0, n)
        y = dev.download(d_y, (n, R), np.float32)
        assert np.array_equal(_bits(y), _bits(y8[:n])), (TYPES[ty], n)
    mv.q4_mmvq_verify(0)
    assert not mv.q4_mmvq_n(ty, d_w, R, K, d_x, d_y, 1.0, 4)


def test_policy_hold_and_widest_row(dev, pkg, oracle, mv):
    lib = dev.lib
    ty, K, R = 14, 16384, 40            # the widest row the scratch takes
    rng = np.random.default_rng(7)
    w = _weights(pkg, rng, ty, R, K)
    xs = _acts(rng, 3, K)
    d_w, d_x, d_y = dev.upload(w), dev.upload(xs), dev.malloc(3 * R * 4)
    assert mv.q4_mmvq_n(ty, d_w, R, K, d_x, d_y, 1.0, 3)
    y = dev.download(d_y, (3, R), np.float32)
    assert np.array_equal(_bits(y[:, :5]), _bits(oracle.mv_rows(ty, w[:5], 5, K, xs)))
    # refusals: nothing queued
    n0 = lib.q4_cuda_launch_count()
    assert not mv.q4_mmvq_n(ty, d_w, R, K, d_x, d_y, 1.0, 1)            # one row outside a verify scope
    assert not mv.q4_mmvq_n(ty, d_w, R, K, d_x, d_y, 1.0, 9)
    assert not mv.q4_mmvq_n(ty, d_w, R, K + 256, d_x, d_y, 1.0, 2)      # wider than the scratch
    assert not mv.q4_mmvq_n(ty, d_w, R, 2560 - 32, d_x, d_y, 1.0, 2)    # not whole super-blocks
    assert not mv.q4_mmvq_n(12, d_w + 2, R, 2560, d_x, d_y, 1.0, 2)     # Q4_K rows want 16-byte alignment
    assert not mv.q4_mmvq_n(2, d_w, R, 2560, d_x, d_y, 1.0, 2)          # a type outside the product
    mv.q4_mmvq_set(0)
    assert not mv.q4_mmvq_n(ty, d_w, R, K, d_x, d_y, 1.0, 3)
    mv.q4_mmvq_set(1)
    assert lib.q4_cuda_launch_count() == n0
    # hold: the second call on the same rows skips the quantiser, for fewer rows too; once x is
    # rewritten inside the scope the stale quantisation shows, which is the caller's contract
    mv.q4_mmvq_hold(d_x)
    assert mv.q4_mmvq_n(ty, d_w, R, K, d_x, d_y, 1.0, 3)
    n1 = lib.q4_cuda_launch_count()
    assert mv.q4_mmvq_n(ty, d_w, R, K, d_x, d_y, 1.0, 2)
    assert lib.q4_cuda_launch_count() - n1 == 1
    assert np.array_equal(_bits(dev.download(d_y, (2, R), np.float32)), _bits(y[:2]))
    dev.write(d_x, np.zeros_like(xs))
    assert mv.q4_mmvq_n(ty, d_w, R, K, d_x, d_y, 1.0, 3)
    assert np.array_equal(_bits(dev.download(d_y, (3, R), np.float32)), _bits(y))
    mv.q4_mmvq_release()
    assert mv.q4_mmvq_n(ty, d_w, R, K, d_x, d_y, 1.0, 3)
    assert not dev.download(d_y, (3, R), np.float32).any()
    assert lib.q4_cuda_device_error() == 0
