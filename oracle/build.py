#!/usr/bin/env python3
"""Build the CPU checkers.

  oracle/_build/libq4oracle.so   the plain-C restatement (q4_oracle.c); always built
  oracle/_ref/libq4ref.so        the reference engine's own CPU expert path
                                 (src/q4_cpuexp.c + src/q4_quant.c compiled
                                 unmodified, plus ref_shim.c); built only when a
                                 reference checkout is present
  oracle/_ref/q4_moe.o, q4_engine_glue.o   objects of the link check (engine_link_symbols)

Both are test infrastructure: only tests, the smoke check and the benchmark's
CPU-baseline leg load them.  Run `python oracle/build.py [--ref <checkout>]`.
"""
import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CODES_DIR = os.path.join(ROOT, "suzuku-engine-q4_b200", "csrc")
# the reference checkout: named by the environment, else the directory "reference" beside this repository
DEFAULT_REF = os.environ.get("Q4_REFERENCE_DIR", os.path.join(os.path.dirname(ROOT), "reference"))

ORACLE_SO = os.path.join(HERE, "_build", "libq4oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libq4ref.so")


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources if os.path.exists(s))


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("oracle build failed")


def build_oracle(force=False):
    src = [os.path.join(HERE, "q4_oracle.c"), os.path.join(HERE, "q4_oracle.h"),
           os.path.join(CODES_DIR, "iq3s_codes.h"), os.path.join(CODES_DIR, "iq4nl_codes.h"),
           os.path.join(CODES_DIR, "iq3xxs_codes.h"), os.path.join(CODES_DIR, "iq2s_codes.h")]
    if not force and _newer(ORACLE_SO, src):
        return ORACLE_SO
    os.makedirs(os.path.dirname(ORACLE_SO), exist_ok=True)
    # -mfma only so that fmaf() is one instruction; -ffp-contract=off keeps
    # the compiler from fusing anything that is not written as fmaf().
    _run(["gcc", "-O2", "-mfma", "-ffp-contract=off", "-fPIC", "-shared",
          "-I", CODES_DIR, "-o", ORACLE_SO, src[0], "-lm"])
    return ORACLE_SO


def build_ref(ref_dir=DEFAULT_REF, force=False):
    """Returns the .so path, or None when no reference checkout is present and
    no prebuilt library exists."""
    ref_src = os.path.join(ref_dir, "src")
    cpuexp = os.path.join(ref_src, "q4_cpuexp.c")
    quant = os.path.join(ref_src, "q4_quant.c")
    shim = os.path.join(HERE, "ref_shim.c")
    if not (os.path.exists(cpuexp) and os.path.exists(quant)):
        return REF_SO if os.path.exists(REF_SO) else None
    if not force and _newer(REF_SO, [cpuexp, quant, shim]):
        return REF_SO
    out_dir = os.path.dirname(REF_SO)
    os.makedirs(out_dir, exist_ok=True)
    o_shim = os.path.join(out_dir, "ref_shim.o")
    o_quant = os.path.join(out_dir, "q4_quant.o")
    # The reference's own flags for these two objects (its Makefile:6,40-41).
    _run(["gcc", "-O2", "-O3", "-mavx2", "-mfma", "-mf16c", "-pthread", "-fPIC",
          "-w", "-I", ref_src, "-c", "-o", o_shim, shim])
    _run(["gcc", "-O2", "-pthread", "-fopenmp", "-fPIC", "-w", "-I", ref_src, "-c", "-o",
          o_quant, quant])
    _run(["gcc", "-shared", "-pthread", "-fopenmp", "-o", REF_SO, o_shim, o_quant, "-lm"])
    return REF_SO


def engine_link_symbols(ref_dir=DEFAULT_REF):
    """The link check of the drop-in boundary: compile the reference engine's MoE layer code
    (src/q4_moe.c) and the engine-side glue to objects (into oracle/_ref/, nothing is linked
    or run) and return (device symbols q4_moe.o leaves undefined, symbols the glue defines).
    None when no reference checkout is present."""
    ref_src = os.path.join(ref_dir, "src")
    moe = os.path.join(ref_src, "q4_moe.c")
    if not os.path.exists(moe):
        return None
    out_dir = os.path.dirname(REF_SO)
    os.makedirs(out_dir, exist_ok=True)
    o_moe = os.path.join(out_dir, "q4_moe.o")
    o_glue = os.path.join(out_dir, "q4_engine_glue.o")
    glue = os.path.join(ROOT, "suzuku-engine-q4_b200", "host", "q4_engine_glue.c")
    _run(["gcc", "-O1", "-w", "-I", ref_src, "-c", "-o", o_moe, moe])
    _run(["gcc", "-O2", "-Wall", "-Werror", "-I", ref_src, "-c", "-o", o_glue, glue])
    und = subprocess.run(["nm", "-u", o_moe], capture_output=True, text=True, check=True).stdout.split()
    dev = sorted(n for n in und if n.startswith(("q4_hip_", "q4_mmq_", "q4_xg_", "q4_mmvq_", "q4_hgemm_")))
    defs = subprocess.run(["nm", "--defined-only", o_glue], capture_output=True, text=True, check=True).stdout
    glue_syms = sorted(line.split()[-1] for line in defs.splitlines() if " T " in line)
    return dev, glue_syms


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=DEFAULT_REF)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build_oracle(a.force))
    print(build_ref(a.ref, a.force))


if __name__ == "__main__":
    main()
