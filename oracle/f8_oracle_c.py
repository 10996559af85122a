"""ctypes wrapper of the C restatement (`f8_oracle_c.c`).  TEST INFRASTRUCTURE ONLY.

Same arithmetic as `f8_oracle.py`, element-wise parts in C with OpenMP, GEMMs through
numpy's BLAS: the CPU path a user of the reference's `emulate=True` mode would time.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "_build", "libf8oracle.so")
_DT = {"bf16": 0, "fp16": 1, "fp32": 2}
_KIND = {"e4m3fn": 0, "e5m2": 1}
_lib = None


def build() -> str:
    src = os.path.join(HERE, "f8_oracle_c.c")
    if not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE], check=True, capture_output=True)
    return LIB


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(LIB)
        vp, i64, i32, f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
        L.f8o_amax.restype = f32
        L.f8o_amax.argtypes = [vp, i32, i64]
        L.f8o_amax_to_scale.restype = f32
        L.f8o_amax_to_scale.argtypes = [f32, i32, i32, i32]
        L.f8o_cast.restype = None
        L.f8o_cast.argtypes = [vp, i32, i64, f32, i32, i32, vp]
        L.f8o_dequant_f32.restype = None
        L.f8o_dequant_f32.argtypes = [vp, i32, i64, f32, vp]
        L.f8o_round_store.restype = None
        L.f8o_round_store.argtypes = [vp, i64, i32, vp]
        _lib = L
    return _lib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def tensor_to_amax(x: np.ndarray, dtype: str) -> np.float32:
    x = np.ascontiguousarray(x)
    return np.float32(lib().f8o_amax(_ptr(x), _DT[dtype], x.size))


def amax_to_scale(amax, fp8: str, orig_dtype: str, amax_dtype: str) -> np.float32:
    return np.float32(lib().f8o_amax_to_scale(float(amax), _KIND[fp8], _DT[amax_dtype], _DT[orig_dtype]))


def cast_to_fp8(x: np.ndarray, dtype: str, scale, fp8: str, product_dtype: str) -> np.ndarray:
    x = np.ascontiguousarray(x)
    out = np.empty(x.shape, dtype=np.uint8)
    lib().f8o_cast(_ptr(x), _DT[dtype], x.size, float(scale), _KIND[fp8], _DT[product_dtype], _ptr(out))
    return out


def cast_dynamic(x: np.ndarray, dtype: str, fp8: str):
    amax = tensor_to_amax(x, dtype)
    scale = amax_to_scale(amax, fp8, dtype, dtype)
    return cast_to_fp8(x, dtype, scale, fp8, dtype), scale, amax


def dequant_f32(bits: np.ndarray, fp8: str, scale) -> np.ndarray:
    bits = np.ascontiguousarray(bits)
    out = np.empty(bits.shape, dtype=np.float32)
    lib().f8o_dequant_f32(_ptr(bits), _KIND[fp8], bits.size, float(scale), _ptr(out))
    return out


def round_store(v: np.ndarray, dtype: str) -> np.ndarray:
    v = np.ascontiguousarray(v, dtype=np.float32)
    out = np.empty(v.shape, dtype=np.float32 if dtype == "fp32" else np.uint16)
    lib().f8o_round_store(_ptr(v), v.size, _DT[dtype], _ptr(out))
    return out


def float8_linear_fwd_bwd(x, w, go, dtype: str = "bf16"):
    """Float8Linear forward+backward, dynamic scaling, no bias
    (float8_experimental/float8_linear.py:356-373 and :65-95 with the emulated GEMM of
    float8_aten_api.py:16-28).  Outputs in `dtype` storage."""
    x8, sx, _ = cast_dynamic(x, dtype, "e4m3fn")
    w8, sw, _ = cast_dynamic(w, dtype, "e4m3fn")
    g8, sg, _ = cast_dynamic(go, dtype, "e5m2")
    xf, wf, gf = dequant_f32(x8, "e4m3fn", sx), dequant_f32(w8, "e4m3fn", sw), dequant_f32(g8, "e5m2", sg)
    y = round_store(xf @ wf.T, dtype)
    dx = round_store(gf @ wf, dtype)
    dw = round_store(gf.T @ xf, dtype)
    return dict(x8=x8, w8=w8, g8=g8, sx=sx, sw=sw, sg=sg, y=y, dx=dx, dw=dw)
