"""The C-ABI library builds, loads and exports every symbol the header declares.
No compute calls: this runs on machines without a GPU."""
import ctypes
import os
import re

from float8_experimental_b200 import _native
from float8_experimental_b200.csrc import build as builder

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols(header="f8b200.h"):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(f8b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    path = builder.build()
    assert os.path.exists(path)
    lib = ctypes.CDLL(path)
    names = declared_symbols()
    assert len(names) >= 11
    for name in names:
        assert hasattr(lib, name), name
    assert sorted(_native.EXPORTS) == names


def test_multicast_library_exports_exactly_its_header():
    """libf8b200_mc.so (single-GPU jobs only) exports the two entry points of f8b200_mc.h and
    nothing else: the copy of gemm.cu it carries stays private (hidden visibility), so it cannot
    interpose libf8b200.so's symbols.  Its entry point refuses pointers before any CUDA work."""
    import subprocess

    path = builder.build_mc()
    if path is None:
        import pytest

        pytest.skip("gemm_mc.cu is not part of this checkout")
    names = declared_symbols("f8b200_mc.h")
    assert names == ["f8b200_mc_gemm_fp8", "f8b200_mc_read_device_error"]
    out = subprocess.run(["nm", "-D", "--defined-only", path], capture_output=True, text=True, check=True).stdout
    exported = sorted(line.split()[-1] for line in out.splitlines() if " T " in line)
    assert exported == names, exported
    lib = ctypes.CDLL(path)
    vp = ctypes.c_void_p
    lib.f8b200_mc_gemm_fp8.argtypes = [vp, ctypes.c_int, ctypes.c_int, ctypes.c_int64, vp, ctypes.c_int, ctypes.c_int,
                                       ctypes.c_int64, vp, vp, vp, ctypes.c_int, vp, ctypes.c_int64, ctypes.c_int64,
                                       ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int, vp, ctypes.c_int64, vp]
    # unknown cluster shape: refused before anything touches CUDA
    assert lib.f8b200_mc_gemm_fp8(vp(16), 0, 0, 16, vp(16), 0, 0, 16, vp(4), vp(4), None, 0, vp(16), 16, 4, 4, 16, 3, 1,
                                  None, 0, None) == -1


def test_status_strings_and_argument_validation():
    lib = _native.load()
    assert lib.f8b200_status_string(0) == b"ok"
    for code in range(-7, 0):
        assert lib.f8b200_status_string(code) != b"unknown status"
    # argument checks happen before any CUDA call
    assert lib.f8b200_amax(None, 0, 16, None, None) == -1
    assert lib.f8b200_amax(ctypes.c_void_p(16), 7, 16, ctypes.c_void_p(16), None) == -1
    assert lib.f8b200_gemm_fp8(ctypes.c_void_p(16), 0, 8, ctypes.c_void_p(16), 0, 16, ctypes.c_void_p(4),
                               ctypes.c_void_p(4), None, 0, ctypes.c_void_p(16), 16, 4, 4, 16, 0, None) == -1
    assert lib.f8b200_gemm_fp8(ctypes.c_void_p(16), 0, 24, ctypes.c_void_p(16), 0, 16, ctypes.c_void_p(4),
                               ctypes.c_void_p(4), None, 0, ctypes.c_void_p(16), 16, 4, 4, 16, 0, None) == -2
    # the workspace entry wants an aligned workspace of at least F8B200_GEMM_WORKSPACE_BYTES
    args = (ctypes.c_void_p(16), 0, 0, 16, ctypes.c_void_p(16), 0, 0, 16, ctypes.c_void_p(4), ctypes.c_void_p(4), None,
            0, ctypes.c_void_p(16), 16, 4, 4, 16, 0)
    assert lib.f8b200_gemm_fp8_ws(*args, None, 256, None) == -1
    assert lib.f8b200_gemm_fp8_ws(*args, ctypes.c_void_p(256), 8, None) == -1
    assert lib.f8b200_gemm_fp8_ws(*args, ctypes.c_void_p(260), 256, None) == -2
    # the static-scratch entry validates before it looks anything up or takes a slot
    assert lib.f8b200_gemm_fp8_static_scratch(ctypes.c_void_p(16), 0, 8, ctypes.c_void_p(16), 0, 16, ctypes.c_void_p(4),
                                              ctypes.c_void_p(4), None, 0, ctypes.c_void_p(16), 16, 4, 4, 16, 0,
                                              None) == -1
    assert lib.f8b200_gemm_fp8_static_scratch(None, 0, 16, None, 0, 16, None, None, None, 0, None, 16, 0, 4, 16, 0,
                                              None) == 0  # m == 0: nothing to do
    assert lib.f8b200_cast(ctypes.c_void_p(16), 0, 4, 4, 2, 0, ctypes.c_void_p(4), None, 0, 0, None, 0, None, 0,
                           None, 0, None) == -1


def test_bindings_are_well_formed():
    """Every ctypes binding hands `_check` exactly (status, entry-point name), and the name
    is the entry point it called (a GPU is needed to reach these lines at run time)."""
    import ast
    import inspect

    tree = ast.parse(inspect.getsource(_native))
    calls = [n for n in ast.walk(tree) if isinstance(n, ast.Call) and getattr(n.func, "id", None) == "_check"]
    assert len(calls) >= 14
    for call in calls:
        assert len(call.args) == 2 and not call.keywords, call.lineno
        status, name = call.args
        assert isinstance(name, ast.Constant) and name.value in _native.EXPORTS, call.lineno
        assert isinstance(status, ast.Call) and status.func.attr == name.value, call.lineno


def test_default_gemm_kernel_choice(monkeypatch):
    """Host-side rule behind f8b200_gemm_fp8: CTA pairs on 512x256 tiles for the large long-K products (every
    GEMM of the LLaMa-2-70B step), CTA pairs on 256x256 tiles where the large tiles would fill the last wave
    badly, K is short, or there are at most 256 rows; the environment can force any kernel."""
    for var in ("F8B200_GEMM_MODE", "F8B200_GEMM_WIDE_K", "F8B200_GEMM_SM_MARGIN"):
        monkeypatch.delenv(var, raising=False)
    choice = _native.gemm_kernel_choice
    m = 16384
    for k, n in ((8192, 10240), (8192, 8192), (8192, 57344), (28672, 8192)):
        assert [choice(m, n, k), choice(m, k, n), choice(n, k, m)] == [3, 3, 3], (k, n)
    assert choice(8192, 4096, 4096) == 1      # K = 4096: the exposed part of the drain weighs 7 %
    assert choice(1024, 4096, 8192) == 1      # 32 large tiles would leave most CTA pairs idle
    assert choice(8192, 4096, 14336) == 1     # 256 large tiles: 4 waves for the work of 3.46
    assert choice(4096, 4096, 8192) == 3
    assert choice(256, 8192, 8192) == 1 and choice(257, 8192, 8192) in (1, 3)
    monkeypatch.setenv("F8B200_GEMM_MODE", "wide")
    assert choice(m, 8192, 8192) == 2
    monkeypatch.setenv("F8B200_GEMM_MODE", "pw")
    assert choice(8192, 4096, 4096) == 3
