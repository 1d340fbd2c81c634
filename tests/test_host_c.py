"""The C host mirror: compiles with gcc against include/q4cuda.h (no GPU needed for that), and on
a GPU runs a C program that drives one layer through it and checks it against the C oracle."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "suzuku-engine-q4_b200")
EXE = os.path.join(ROOT, "tests", "host_c", "_build", "q4_moe_host_test")


def _build(pkg):
    os.makedirs(os.path.dirname(EXE), exist_ok=True)
    cmd = ["gcc", "-O2", "-std=c11", "-Wall", "-Werror", "-mfma", "-ffp-contract=off",
           "-I", os.path.join(PKG, "csrc"), "-o", EXE,
           os.path.join(ROOT, "tests", "host_c", "q4_moe_host_test.c"),
           os.path.join(PKG, "host", "q4_moe_b200.c"), os.path.join(PKG, "host", "q4_gguf_experts.c"),
           os.path.join(ROOT, "oracle", "q4_oracle.c"),
           "-L", PKG, "-lq4cuda", "-lm", "-Wl,-rpath," + PKG]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr


def test_c_host_compiles_and_links(pkg):
    _build(pkg)
    assert os.path.exists(EXE)


@pytest.mark.gpu
def test_c_host_layer_on_gpu(pkg):
    _build(pkg)
    r = subprocess.run([EXE], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "PASS" in r.stdout
