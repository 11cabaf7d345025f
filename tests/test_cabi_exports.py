"""CPU: the C-ABI library loads and exports every symbol include/hesper_b200.h declares;
argument validation and the no-GPU failure mode are loud, never a silent CPU fallback."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "hesper_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hb200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_expected_surface():
    syms = declared_symbols()
    for s in ["hb200_ctx_create", "hb200_bitlinear_forward", "hb200_bitlinear_gateup_relu2",
              "hb200_kquant_forward", "hb200_kquant_gateup_gelu", "hb200_attn_decode",
              "hb200_attn_workspace_bytes", "hb200_last_error"]:
        assert s in syms


def test_library_exports_every_declared_symbol():
    from hesper_b200 import _lib
    lib = _lib.load()
    for s in declared_symbols():
        assert hasattr(lib, s), f"{s} is declared in the header but not exported"
        assert s in _lib.SIGNATURES, f"{s} has no ctypes signature"


def test_no_gpu_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import hesper_b200
    with pytest.raises(hesper_b200.HesperB200Error):
        hesper_b200.Context(0)
    from hesper_b200 import _lib
    assert b"CUDA" in _lib.load().hb200_last_error()


def test_null_context_is_rejected_without_touching_the_gpu():
    from hesper_b200 import _lib
    lib = _lib.load()
    rc = lib.hb200_bitlinear_forward(None, None, None, 128, 1, None, 1, None, C.c_float(0), None,
                                     None, None, None, None)
    assert rc == -1 and b"null context" in lib.hb200_last_error()
    rc = lib.hb200_attn_decode(None, None, 0, None, None, None, 1, 1, 1, 64, 1, 0, C.c_float(1),
                               None, 0, None, None)
    assert rc == -1
    assert lib.hb200_version() >= 100


def test_package_has_no_cpu_compute_path():
    """Nothing under hesper_b200/ may import the oracle."""
    pkg = os.path.join(ROOT, "hesper_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src, f
