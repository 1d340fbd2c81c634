"""The C-ABI library builds, loads without a GPU, exports every symbol the
header declares, and refuses to compute without a device (no CPU fallback)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "q4cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(q4_(?:hip|cuda|mmq|mmvq|xg)_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported(pkg):
    lib = ctypes.CDLL(pkg.capi.LIB_PATH)
    names = _declared()
    assert len(names) > 40
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_ep_library_exports_its_header(pkg):
    text = open(os.path.join(ROOT, "include", "q4cuda_ep.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = sorted(set(re.findall(r"\b(q4_cuda_ep_\w+)\s*\(", text)))
    assert sorted(pkg.capi.EP_SIGNATURES) == names
    lib = pkg.capi.load_ep()
    assert all(hasattr(lib, n) for n in names)
    assert lib.q4_cuda_ep_world() == 1


def test_binding_table_matches_header(pkg):
    assert sorted(pkg.capi.SIGNATURES) == _declared()


def test_no_cpu_fallback(pkg):
    if os.path.exists("/dev/nvidia0"):
        return  # a GPU box: covered by the gpu tests
    lib = pkg.capi.load()
    assert lib.q4_hip_init() is False
    assert lib.q4_hip_ok() is False
    assert lib.q4_hip_malloc(1024) is None
    assert lib.q4_hip_moe_tok_ok(21, 21, 21, 2048, 512) is False
    assert lib.q4_cuda_quant8(None, 32, None, None, None) is False


def test_product_does_not_import_the_oracle():
    pk = os.path.join(ROOT, "suzuku-engine-q4_b200")
    for root, _, files in os.walk(pk):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".c")):
                text = open(os.path.join(root, f)).read()
                assert "pyoracle" not in text and "q4_oracle" not in text, f


def test_reference_moe_layer_code_links_against_the_library(pkg):
    """Every device symbol the reference's src/q4_moe.c references is exported by libq4cuda.so
    or defined by the engine-side glue (host/q4_engine_glue.c).  Needs the reference checkout:
    the file is compiled to an object, nothing of it is linked or run."""
    import pytest
    from oracle import build as obuild
    got = obuild.engine_link_symbols()
    if got is None:
        pytest.skip("no reference checkout on this machine")
    wanted, glue = got
    assert len(wanted) > 90, len(wanted)
    lib = ctypes.CDLL(pkg.capi.LIB_PATH)
    missing = [n for n in wanted if not hasattr(lib, n) and n not in glue]
    assert not missing, missing
    # and the header declares what the library resolves for it
    declared = set(_declared())
    assert not [n for n in wanted if n not in glue and n not in declared]
