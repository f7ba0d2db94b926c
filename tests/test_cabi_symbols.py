"""The shared library builds for sm_100a, loads without a GPU, and exports every entry point
that include/liteform_b200.h declares (no compute call is made here)."""
import ctypes
import os
import re

from liteform_ae_b200 import _build, _cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "liteform_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lf_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_all_symbols():
    _build.build_library()
    lib = _cabi.load()
    names = _declared()
    assert "lf_spmm_hyb_f32" in names and "lf_hyb_plan" in names
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in the header but not exported"
    assert sorted(_cabi.SIGNATURES) == names, "ctypes signatures and header disagree"
    assert lib.lf_version() >= 100


def test_struct_layout_matches_header():
    # 4 int64 + 2 int32 + 10 pointers + 1 int64
    assert ctypes.sizeof(_cabi.LfHyb) == 4 * 8 + 2 * 4 + 10 * 8 + 8


def test_workspace_queries_are_pure():
    lib = _cabi.load()
    assert lib.lf_hyb_stats_workspace_bytes(10, 1000, 2) >= 4000
    a = lib.lf_hyb_build_workspace_bytes(0, 100000, 4, 20)
    b = lib.lf_hyb_build_workspace_bytes(0, 200000, 4, 20)
    assert 0 < a < b
    assert lib.lf_hyb_fill_scratch_bytes(1000) >= 8000


def test_public_header_is_plain_c():
    """The boundary is a C ABI: the header must compile as C99 on its own (a cgo / JNI / ctypes
    binding generator sees nothing else)."""
    import os
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        import pytest
        pytest.skip("no C compiler")
    header = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "liteform_b200.h")
    res = subprocess.run([gcc, "-fsyntax-only", "-x", "c", "-std=c99", "-Wall", "-Werror", header],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
