#!/usr/bin/env python3
"""Generate tests/golden/iq3s_moe_small.npz and tests/golden/dense_types_dequant.npz from the
reference's own CPU code.

Needs oracle/_ref/libq4ref.so (built by oracle/build.py from a reference
checkout).  The fixture holds the inputs as bytes, so checking it needs neither
the reference nor any particular random generator.

  python tests/golden/gen_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402
from oracle import pyoracle  # noqa: E402


def main():
    pkg = entry.load_package()
    synth = pkg.synth
    R = pyoracle.reference()
    if R is None:
        raise SystemExit("reference CPU path not built; run oracle/build.py with a checkout")
    H, F, E, K = 256, 256, 2, 2
    rng = np.random.default_rng(20261125)
    packs = synth.expert_packs(rng, E, H, F)
    x = rng.standard_normal(H).astype(np.float32)
    x[32:64] = 0.0                      # an all-zero group: d = 0, q = 0
    x[64] = 3.5                         # exact .5 products after scaling exist below
    wts = np.array([0.625, 0.375], np.float32)
    rb = synth.iq3s_row_bytes(H)
    xq = R.quant8(x)
    gate_dots = np.array([R.dot8(packs[0][r * rb:(r + 1) * rb], xq, H) for r in range(F)],
                         np.float32)
    gate_dots_avx2 = np.array([R.dot8(packs[0][r * rb:(r + 1) * rb], xq, H, avx2=True)
                               for r in range(F)], np.float32)
    assert np.array_equal(gate_dots.view(np.uint32), gate_dots_avx2.view(np.uint32))
    deq = np.stack([R.dequant_row(packs[0][r * rb:(r + 1) * rb], H) for r in range(4)])
    y1 = R.expert_job([packs[0]], [0], [1.0], x, H, F)
    y2 = R.expert_job([packs[0], packs[1]], [0, 1], wts, x, H, F)
    # router pieces
    n_exp = 64
    router = (rng.standard_normal((n_exp, H)) * 0.02).astype(np.float32)
    norm_w = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    xn = R.rms_norm(x, norm_w, 1e-6)
    logits = R.gemv(0, router, n_exp, H, xn)
    logits[7] = logits[3]               # planted tie: the lower index must win
    probs = R.softmax(logits)
    ids, w = R.topk(probs, 6, True)
    # closed-form known answer of the reference's unit test (src/q4_test.c:52-58):
    # all-zero block with d = 1.0 against x = 1 gives 256
    kat_blk = np.zeros(110, np.uint8)
    kat_blk[0:2] = np.array([0x3c00], np.uint16).view(np.uint8)
    kat = R.dot_f32(kat_blk, np.ones(256, np.float32), 256)
    out = os.path.join(HERE, "iq3s_moe_small.npz")
    np.savez(out, H=H, F=F, packs=packs, x=x, wts=wts, xq=xq.view(np.uint8), gate_dots=gate_dots,
             deq=deq, y1=y1, y2=y2, router=router, norm_w=norm_w, xn=xn, logits=logits,
             probs=probs, top_ids=ids, top_w=w, kat=np.float32(kat))
    print("wrote", out, os.path.getsize(out), "bytes")
    dense_types(synth, R)


def dense_types(synth, R):
    """Seeded rows of the five weight types of the dense 8-bit product (Q4_K, Q5_K, Q6_K, IQ4_XS,
    IQ4_NL) with the reference's q4_dequant_row of each: pins the 16-value run decoders."""
    rng = np.random.default_rng(20261126)
    n = 512
    out = {}
    for ty in (12, 13, 14, 23, 20):
        rows = np.stack([synth.blocks_of(rng, ty, synth.row_bytes(ty, n)) for _ in range(3)])
        out["rows_%d" % ty] = rows
        out["deq_%d" % ty] = np.stack([R.dequant_row_t(ty, r, n) for r in rows])
    path = os.path.join(HERE, "dense_types_dequant.npz")
    np.savez(path, n=n, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
