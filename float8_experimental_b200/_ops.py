"""`torch.library` registration of the sm_100a kernels as opaque custom ops.

The reference registers its one private op the same way
(float8_experimental/float8_aten_api.py:37-49: `Library(...)`, `define`, `impl`).
Only a CUDA implementation (and a Meta/fake one for tracing) is registered: calling an
op with CPU tensors fails in the dispatcher, there is no fallback.

Ops (namespace `f8b200`):
  amax(x) -> fp32 0-dim                                   f8b200_amax
  multi_amax(xs) -> fp32 [n]                              f8b200_multi_amax
  amax_to_scale(amax, kind, amax_dtype, orig_dtype)       f8b200_amax_to_scale
  cast_from_amax(x, amax, kind, with_t) -> (data, data_t, scale)   f8b200_cast, scale_src=1
  cast_with_scale(x, scale, kind, product_fp32, with_t, amax_out!) -> (data, data_t)
  cast_dynamic(x, kind) -> (data, scale)                  f8b200_cast_dynamic (amax + cast, one call)
  multi_cast_with_scales(xs, scales, kind, product_fp32) -> fp8 tensors   f8b200_multi_cast
  transpose_fp8(x) -> x^T contiguous                      f8b200_transpose_u8
  delayed_sync(amax, hist, n_e4m3, orig_dtype, scale_out!, hist_out!)
  scaled_mm(a, b_t, scale_a, scale_b, bias, out_dtype, use_fast_accum) -> out
  rmsnorm_amax(x, weight, eps) -> (rstd fp32 [rows], amax fp32 0-dim)      f8b200_rmsnorm_amax
  rmsnorm_cast(x, weight, rstd, amax, kind) -> (data, scale)               f8b200_rmsnorm_cast
  swiglu_amax(a, b, write_y, approx) -> (amax fp32 0-dim, y or empty)      f8b200_swiglu_amax[_approx]
  swiglu_cast(a, b, amax, kind) -> (data, scale)                           f8b200_swiglu_cast
"""
from __future__ import annotations

from typing import List, Tuple

import torch

from . import _native as N

_lib = torch.library.Library("f8b200", "DEF")

_lib.define("amax(Tensor x) -> Tensor")
_lib.define("multi_amax(Tensor[] xs) -> Tensor")
_lib.define("amax_to_scale(Tensor amax, int fp8_kind, int amax_dtype, int orig_dtype) -> Tensor")
_lib.define("cast_from_amax(Tensor x, Tensor amax, int fp8_kind, bool with_transpose) -> (Tensor, Tensor, Tensor)")
_lib.define(
    "cast_with_scale(Tensor x, Tensor scale, int fp8_kind, bool product_fp32, bool with_transpose, "
    "Tensor(a!)? amax_out) -> (Tensor, Tensor)"
)
_lib.define("cast_dynamic(Tensor x, int fp8_kind) -> (Tensor, Tensor)")
_lib.define("multi_cast_with_scales(Tensor[] xs, Tensor scales, int fp8_kind, bool product_fp32) -> Tensor[]")
_lib.define("transpose_fp8(Tensor x) -> Tensor")
_lib.define(
    "delayed_sync(Tensor amax, Tensor hist, int n_e4m3, int orig_dtype, Tensor(a!) scale_out, "
    "Tensor(b!)? hist_out) -> ()"
)
_lib.define(
    "scaled_mm(Tensor a, Tensor b_t, Tensor scale_a, Tensor scale_b, Tensor? bias, ScalarType out_dtype, "
    "bool use_fast_accum) -> Tensor"
)
_lib.define("rmsnorm_amax(Tensor x, Tensor weight, float eps) -> (Tensor, Tensor)")
_lib.define("rmsnorm_cast(Tensor x, Tensor weight, Tensor rstd, Tensor amax, int fp8_kind) -> (Tensor, Tensor)")
_lib.define("swiglu_amax(Tensor a, Tensor b, bool write_y, bool approx=False) -> (Tensor, Tensor)")
_lib.define("rmsnorm_bwd(Tensor x, Tensor grad_y, Tensor weight, Tensor rstd) -> (Tensor, Tensor)")
_lib.define("swiglu_bwd(Tensor a, Tensor b, Tensor grad_y, bool approx=False) -> (Tensor, Tensor)")
_lib.define("swiglu_cast(Tensor a, Tensor b, Tensor amax, int fp8_kind) -> (Tensor, Tensor)")


def _as_matrix(x: torch.Tensor) -> Tuple[torch.Tensor, int, int, int]:
    """Views `x` as [rows, cols] with unit inner stride; returns (tensor, rows, cols, ld)."""
    cols = x.shape[-1] if x.dim() > 0 else 1
    rows = x.numel() // cols if cols > 0 else 0
    if x.dim() == 2 and x.stride(1) == 1 and x.stride(0) >= max(cols, 1):
        return x, rows, cols, x.stride(0)
    if not x.is_contiguous():
        x = x.contiguous()
    return x, rows, cols, cols


def _empty_like_shape(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    return torch.empty(x.shape, dtype=dtype, device=x.device)


# ---------------------------------------------------------------------------
# CUDA implementations
# ---------------------------------------------------------------------------
def _amax_cuda(x: torch.Tensor) -> torch.Tensor:
    if x.numel() == 0:
        raise RuntimeError("amax of an empty tensor is undefined")
    if not x.is_contiguous():
        x = x.contiguous()
    out = torch.empty((), dtype=torch.float32, device=x.device)
    N.amax(x, out)
    return out


def _multi_amax_cuda(xs: List[torch.Tensor]) -> torch.Tensor:
    xs = [t if t.is_contiguous() else t.contiguous() for t in xs]
    dev = xs[0].device if xs else torch.device("cuda")
    out = torch.empty((len(xs),), dtype=torch.float32, device=dev)
    N.multi_amax(xs, out)
    return out


def _amax_to_scale_cuda(amax: torch.Tensor, fp8_kind: int, amax_dtype: int, orig_dtype: int) -> torch.Tensor:
    a = amax if (amax.dtype == torch.float32 and amax.is_contiguous()) else amax.float().contiguous()
    out = torch.empty(amax.shape, dtype=torch.float32, device=amax.device)
    N.amax_to_scale(a, fp8_kind, amax_dtype, orig_dtype, out)
    return out


def _alloc_cast_outputs(x: torch.Tensor, rows: int, cols: int, fp8_kind: int, with_transpose: bool):
    f8 = N.FP8_DTYPE[fp8_kind]
    data = _empty_like_shape(x, f8)
    if with_transpose:
        data_t = torch.empty((cols, rows), dtype=f8, device=x.device)
    else:
        data_t = torch.empty((0,), dtype=f8, device=x.device)
    return data, data_t


def _cast_from_amax_cuda(x, amax, fp8_kind: int, with_transpose: bool):
    xm, rows, cols, ld = _as_matrix(x)
    data, data_t = _alloc_cast_outputs(x, rows, cols, fp8_kind, with_transpose)
    scale = torch.empty((), dtype=torch.float32, device=x.device)
    N.cast(xm, rows, cols, ld, 1, amax, scale, False, fp8_kind, data, cols,
           data_t if with_transpose else None, rows, None, True)
    return data, data_t, scale


def _cast_with_scale_cuda(x, scale, fp8_kind: int, product_fp32: bool, with_transpose: bool, amax_out):
    xm, rows, cols, ld = _as_matrix(x)
    data, data_t = _alloc_cast_outputs(x, rows, cols, fp8_kind, with_transpose)
    s = scale if scale.dtype == torch.float32 else scale.float()
    N.cast(xm, rows, cols, ld, 0, s, None, product_fp32, fp8_kind, data, cols,
           data_t if with_transpose else None, rows, amax_out, False)
    return data, data_t


def _cast_dynamic_cuda(x, fp8_kind: int):
    """amax + cast with the scale derived from the amax, one host call: (fp8 data, scale)."""
    if not x.is_contiguous():
        x = x.contiguous()
    cols = x.shape[-1] if x.dim() > 0 else 1
    rows = x.numel() // cols if cols > 0 else 0
    if rows == 0 or cols == 0:
        raise RuntimeError("amax of an empty tensor is undefined")
    data = torch.empty(x.shape, dtype=N.FP8_DTYPE[fp8_kind], device=x.device)
    amax_scale = torch.empty(2, dtype=torch.float32, device=x.device)
    N.cast_dynamic(x, rows, cols, fp8_kind, amax_scale[0], amax_scale[1], data)
    return data, amax_scale[1]


def _multi_cast_with_scales_cuda(xs: List[torch.Tensor], scales: torch.Tensor, fp8_kind: int, product_fp32: bool):
    xs = [t if t.is_contiguous() else t.contiguous() for t in xs]
    s = scales if (scales.dtype == torch.float32 and scales.is_contiguous()) else scales.float().contiguous()
    outs = [torch.empty(t.shape, dtype=N.FP8_DTYPE[fp8_kind], device=t.device) for t in xs]
    N.multi_cast(xs, s, product_fp32, fp8_kind, outs)
    return outs


def _transpose_fp8_cuda(x: torch.Tensor) -> torch.Tensor:
    assert x.dim() == 2
    if x.stride(1) != 1:
        x = x.contiguous()
    rows, cols = x.shape
    out = torch.empty((cols, rows), dtype=x.dtype, device=x.device)
    N.transpose_u8(x, rows, cols, x.stride(0), out, rows)
    return out


def _delayed_sync_cuda(amax, hist, n_e4m3: int, orig_dtype: int, scale_out, hist_out) -> None:
    N.delayed_sync(amax, hist, n_e4m3, orig_dtype, scale_out, hist_out)


def _pitch16(n: int) -> int:
    return -(-n // 16) * 16


def _gemm_operand(x: torch.Tensor):
    """How the GEMM can read the logical [rows, K] operand `x` where it lies: (tensor, pitch,
    mn_major).  K contiguous = K-major; rows contiguous (a transposed view of a [K, rows]
    buffer) = MN-major, which the tensor cores read through an MN-major descriptor.  Anything
    else, or a pitch / base address that TMA cannot take, is copied into a K-major buffer
    whose row pitch is rounded up to 16 bytes.  K itself may be any number: TMA zero-fills
    beyond it, so no operand is ever zero-padded along K (the reference pads both operands
    with a copy when K is not a multiple of 16, float8_experimental/float8_ops.py:143-148)."""
    rows, k = x.shape
    if x.stride(1) == 1 and (rows == 1 or (x.stride(0) >= k and x.stride(0) % 16 == 0)) and x.data_ptr() % 16 == 0:
        return x, (x.stride(0) if rows > 1 else _pitch16(k)), False
    if x.stride(0) == 1 and k > 1 and x.stride(1) >= rows and x.stride(1) % 16 == 0 and x.data_ptr() % 16 == 0:
        return x, x.stride(1), True
    buf = torch.empty((rows, _pitch16(k)), dtype=torch.uint8, device=x.device)
    view = buf[:, :k]
    view.copy_(x.view(torch.uint8))
    return view.view(x.dtype), buf.stride(0), False


def _scaled_mm_cuda(a, b_t, scale_a, scale_b, bias, out_dtype, use_fast_accum: bool):
    m, k = a.shape
    n, k2 = b_t.shape
    if k != k2:
        raise RuntimeError(f"scaled_mm: inner dimensions differ ({k} vs {k2})")
    a, lda, a_mn = _gemm_operand(a)
    b_t, ldb, b_mn = _gemm_operand(b_t)
    out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    if bias is not None and bias.dtype != out_dtype:
        bias = bias.to(out_dtype)
    sa = scale_a if scale_a.dtype == torch.float32 else scale_a.float()
    sb = scale_b if scale_b.dtype == torch.float32 else scale_b.float()
    N.gemm_fp8(a, lda, b_t, ldb, sa, sb, bias, out, n, m, n, k, use_fast_accum, a_mn_major=a_mn, b_mn_major=b_mn)
    return out


def _rmsnorm_amax_cuda(x, weight, eps: float):
    xm, rows, cols, ld = _as_matrix(x)
    weight = weight.contiguous()
    if weight.dtype != x.dtype or weight.numel() != cols:
        raise RuntimeError("rmsnorm_amax: the weight must have x's dtype and one element per column")
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    amax = torch.empty((), dtype=torch.float32, device=x.device)
    N.rmsnorm_amax(xm, rows, cols, ld, weight, eps, rstd, amax)
    return rstd, amax


def _rmsnorm_cast_cuda(x, weight, rstd, amax, fp8_kind: int):
    xm, rows, cols, ld = _as_matrix(x)
    weight = weight.contiguous()
    data = _empty_like_shape(x, N.FP8_DTYPE[fp8_kind])
    scale = torch.empty((), dtype=torch.float32, device=x.device)
    N.rmsnorm_cast(xm, rows, cols, ld, weight, rstd, amax, scale, data, cols)
    return data, scale


def _glu_operands(a, b):
    if a.shape != b.shape or a.dtype != b.dtype:
        raise RuntimeError("swiglu: a and b must have one shape and dtype")
    am, rows, cols, lda = _as_matrix(a)
    bm, _, _, ldb = _as_matrix(b)
    return am, bm, rows, cols, lda, ldb


def _swiglu_amax_cuda(a, b, write_y: bool, approx: bool = False):
    am, bm, rows, cols, lda, ldb = _glu_operands(a, b)
    amax = torch.empty((), dtype=torch.float32, device=a.device)
    y = _empty_like_shape(a, a.dtype) if write_y else a.new_empty((0,))
    N.swiglu_amax(am, bm, rows, cols, lda, ldb, y if write_y else None, cols, amax, approx)
    return amax, y


def _swiglu_cast_cuda(a, b, amax, fp8_kind: int):
    am, bm, rows, cols, lda, ldb = _glu_operands(a, b)
    data = _empty_like_shape(a, N.FP8_DTYPE[fp8_kind])
    scale = torch.empty((), dtype=torch.float32, device=a.device)
    N.swiglu_cast(am, bm, rows, cols, lda, ldb, amax, scale, data, cols)
    return data, scale


def _rmsnorm_bwd_cuda(x, grad_y, weight, rstd):
    xm, rows, cols, ld = _as_matrix(x.contiguous())
    gm, _, _, ldg = _as_matrix(grad_y.contiguous())
    dx = torch.empty_like(xm)
    dw = torch.empty_like(weight)
    N.rmsnorm_bwd(xm, gm, rows, cols, ld, ldg, weight.contiguous(), rstd, dx, dw)
    return dx.view(x.shape), dw


def _swiglu_bwd_cuda(a, b, grad_y, approx: bool = False):
    am, bm, rows, cols, lda, ldb = _glu_operands(a, b)
    gm, _, _, ldg = _as_matrix(grad_y.reshape(a.shape).contiguous())
    da = torch.empty(a.shape, dtype=a.dtype, device=a.device)
    db = torch.empty(a.shape, dtype=a.dtype, device=a.device)
    N.swiglu_bwd(am, bm, gm, rows, cols, lda, ldb, ldg, da, db, approx)
    return da, db


_lib.impl("rmsnorm_bwd", _rmsnorm_bwd_cuda, "CUDA")
_lib.impl("swiglu_bwd", _swiglu_bwd_cuda, "CUDA")
_lib.impl("swiglu_amax", _swiglu_amax_cuda, "CUDA")
_lib.impl("swiglu_cast", _swiglu_cast_cuda, "CUDA")
_lib.impl("rmsnorm_amax", _rmsnorm_amax_cuda, "CUDA")
_lib.impl("rmsnorm_cast", _rmsnorm_cast_cuda, "CUDA")
_lib.impl("amax", _amax_cuda, "CUDA")
_lib.impl("multi_amax", _multi_amax_cuda, "CUDA")
_lib.impl("amax_to_scale", _amax_to_scale_cuda, "CUDA")
_lib.impl("cast_from_amax", _cast_from_amax_cuda, "CUDA")
_lib.impl("cast_with_scale", _cast_with_scale_cuda, "CUDA")
_lib.impl("transpose_fp8", _transpose_fp8_cuda, "CUDA")
_lib.impl("multi_cast_with_scales", _multi_cast_with_scales_cuda, "CUDA")
_lib.impl("cast_dynamic", _cast_dynamic_cuda, "CUDA")
_lib.impl("delayed_sync", _delayed_sync_cuda, "CUDA")
_lib.impl("scaled_mm", _scaled_mm_cuda, "CUDA")


# ---------------------------------------------------------------------------
# fake (meta) implementations: shapes and dtypes only, so torch.compile can trace
# around the opaque ops
# ---------------------------------------------------------------------------
@torch.library.register_fake("f8b200::rmsnorm_bwd")
def _rmsnorm_bwd_fake(x, grad_y, weight, rstd):
    return torch.empty_like(x), torch.empty_like(weight)


@torch.library.register_fake("f8b200::swiglu_bwd")
def _swiglu_bwd_fake(a, b, grad_y, approx=False):
    return torch.empty_like(a), torch.empty_like(a)


@torch.library.register_fake("f8b200::swiglu_amax")
def _swiglu_amax_fake(a, b, write_y, approx=False):
    return a.new_empty((), dtype=torch.float32), a.new_empty(a.shape if write_y else (0,))


@torch.library.register_fake("f8b200::swiglu_cast")
def _swiglu_cast_fake(a, b, amax, fp8_kind):
    return a.new_empty(a.shape, dtype=N.FP8_DTYPE[fp8_kind]), a.new_empty((), dtype=torch.float32)


@torch.library.register_fake("f8b200::rmsnorm_amax")
def _rmsnorm_amax_fake(x, weight, eps):
    cols = x.shape[-1]
    return x.new_empty((x.numel() // max(cols, 1),), dtype=torch.float32), x.new_empty((), dtype=torch.float32)


@torch.library.register_fake("f8b200::rmsnorm_cast")
def _rmsnorm_cast_fake(x, weight, rstd, amax, fp8_kind):
    return x.new_empty(x.shape, dtype=N.FP8_DTYPE[fp8_kind]), x.new_empty((), dtype=torch.float32)


@torch.library.register_fake("f8b200::amax")
def _amax_fake(x):
    return x.new_empty((), dtype=torch.float32)


@torch.library.register_fake("f8b200::multi_amax")
def _multi_amax_fake(xs):
    return xs[0].new_empty((len(xs),), dtype=torch.float32)


@torch.library.register_fake("f8b200::amax_to_scale")
def _amax_to_scale_fake(amax, fp8_kind, amax_dtype, orig_dtype):
    return amax.new_empty(amax.shape, dtype=torch.float32)


def _fake_cast_outputs(x, fp8_kind, with_transpose):
    f8 = N.FP8_DTYPE[fp8_kind]
    cols = x.shape[-1] if x.dim() > 0 else 1
    rows = x.numel() // cols if cols > 0 else 0
    data = x.new_empty(x.shape, dtype=f8)
    data_t = x.new_empty((cols, rows) if with_transpose else (0,), dtype=f8)
    return data, data_t


@torch.library.register_fake("f8b200::cast_from_amax")
def _cast_from_amax_fake(x, amax, fp8_kind, with_transpose):
    data, data_t = _fake_cast_outputs(x, fp8_kind, with_transpose)
    return data, data_t, x.new_empty((), dtype=torch.float32)


@torch.library.register_fake("f8b200::cast_with_scale")
def _cast_with_scale_fake(x, scale, fp8_kind, product_fp32, with_transpose, amax_out):
    return _fake_cast_outputs(x, fp8_kind, with_transpose)


@torch.library.register_fake("f8b200::cast_dynamic")
def _cast_dynamic_fake(x, fp8_kind):
    return x.new_empty(x.shape, dtype=N.FP8_DTYPE[fp8_kind]), x.new_empty((), dtype=torch.float32)


@torch.library.register_fake("f8b200::multi_cast_with_scales")
def _multi_cast_with_scales_fake(xs, scales, fp8_kind, product_fp32):
    return [t.new_empty(t.shape, dtype=N.FP8_DTYPE[fp8_kind]) for t in xs]


@torch.library.register_fake("f8b200::transpose_fp8")
def _transpose_fp8_fake(x):
    return x.new_empty((x.shape[1], x.shape[0]))


@torch.library.register_fake("f8b200::delayed_sync")
def _delayed_sync_fake(amax, hist, n_e4m3, orig_dtype, scale_out, hist_out):
    return None


@torch.library.register_fake("f8b200::scaled_mm")
def _scaled_mm_fake(a, b_t, scale_a, scale_b, bias, out_dtype, use_fast_accum):
    return a.new_empty((a.shape[0], b_t.shape[0]), dtype=out_dtype)


ops = torch.ops.f8b200
