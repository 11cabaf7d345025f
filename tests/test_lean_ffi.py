"""CPU: the Lean 4 FFI shim (lean/lean_ffi.cpp) covers the whole C ABI and type-checks.

No Lean toolchain is installed where these tests run, so the shim is compiled with
`g++ -fsyntax-only` against a stand-in lean.h that declares the runtime functions it uses with
their real signatures; the real header replaces it on a machine that has Lean."""
import os
import re
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_functions():
    s = open(os.path.join(ROOT, "include", "hesper_b200.h")).read()
    s = re.sub(r"/\*.*?\*/", "", s, flags=re.S)
    return sorted(set(re.findall(r"\b(hb200_\w+)\s*\(", s)))


def test_generated_files_are_up_to_date(tmp_path):
    """Running the generator reproduces the committed shim and extern declarations."""
    work = tmp_path / "lean"
    shutil.copytree(os.path.join(ROOT, "lean"), work)
    os.makedirs(tmp_path / "include")
    shutil.copy(os.path.join(ROOT, "include", "hesper_b200.h"), tmp_path / "include")
    subprocess.run([sys.executable, str(work / "gen_ffi.py")], check=True)
    for name in ("lean_ffi.cpp", "HesperB200Extern.lean"):
        assert open(work / name).read() == open(os.path.join(ROOT, "lean", name)).read(), name


def test_every_exported_function_has_a_wrapper_and_an_extern():
    cpp = open(os.path.join(ROOT, "lean", "lean_ffi.cpp")).read()
    lean = open(os.path.join(ROOT, "lean", "HesperB200Extern.lean")).read()
    wrappers = set(re.findall(r'extern "C" lean_obj_res (lean_hesper_b200_\w+)', cpp))
    externs = set(re.findall(r'@\[extern "(lean_hesper_b200_\w+)"\]', lean))
    assert wrappers == externs
    for fn in _header_functions():
        assert "lean_" + fn.replace("hb200_", "hesper_b200_") in wrappers, fn
        assert re.search(r"\b%s\b\s*[(,]" % fn, cpp), fn  # and the shim really refers to it


def test_shim_type_checks_against_the_lean_runtime_signatures():
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    r = subprocess.run([gxx, "-std=c++17", "-fsyntax-only", "-Wall", "-Werror",
                        "-I", os.path.join(ROOT, "tests", "lean_stub"),
                        "-I", os.path.join(ROOT, "include"),
                        os.path.join(ROOT, "lean", "lean_ffi.cpp")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_hooks_file_uses_only_declared_externs():
    """Every B200 function the hooks file calls is declared in the extern file."""
    lean = open(os.path.join(ROOT, "lean", "HesperB200Extern.lean")).read()
    hooks = open(os.path.join(ROOT, "lean", "HesperB200.lean")).read()
    declared = set(re.findall(r"^opaque (\w+)", lean, flags=re.M))
    for name in ("ctxCreateCurrent", "kquantForward", "bitlinearForward", "bitlinearGateupRelu2",
                 "attnDecode"):
        assert name in declared, name
        assert re.search(r"\b%s\b" % name, hooks), name
