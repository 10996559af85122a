"""TEST-ONLY: CPU implementations of the `f8b200::*` ops backed by the numpy oracle.

The package ships CUDA implementations only.  Host-side logic (module swap, autograd
wiring, the Float8Tensor operator table, sync bookkeeping, FSDP2 / DTensor hooks over
gloo) still has to be testable on a machine without a GPU, so the tests register these
stand-ins under the CPU dispatch key.  Nothing outside `tests/` imports this file.
"""
from __future__ import annotations

import numpy as np
import torch

import float8_experimental_b200._ops  # noqa: F401  (defines the op schemas)
from float8_experimental_b200 import _native as N
from oracle import f8_oracle as O

_HP = {torch.bfloat16: O.BF16, torch.float16: O.FP16, torch.float32: O.FP32}
_HP_BY_CODE = {N.BF16: O.BF16, N.FP16: O.FP16, N.FP32: O.FP32}
_F8 = {N.E4M3: O.E4M3, N.E5M2: O.E5M2}
_installed = False


def to_np(t: torch.Tensor) -> np.ndarray:
    # clone: exporting a tensor to numpy pins its storage (it can no longer be resized),
    # which FSDP2 does to the buffers it owns
    t = t.detach().contiguous().clone()
    if t.dtype == torch.float32:
        return t.numpy()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.view(torch.uint8).numpy()


def from_np(a: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    a = np.ascontiguousarray(a)
    if dtype == torch.float32:
        return torch.from_numpy(a.astype(np.float32))
    if dtype in (torch.bfloat16, torch.float16):
        return torch.from_numpy(a.view(np.int16).copy()).view(dtype)
    return torch.from_numpy(a.copy()).view(dtype)


def _amax(x):
    return torch.tensor(float(O.tensor_to_amax(to_np(x), _HP[x.dtype])), dtype=torch.float32)


def _multi_amax(xs):
    return torch.tensor([float(O.tensor_to_amax(to_np(x), _HP[x.dtype])) if x.numel() else 0.0 for x in xs],
                        dtype=torch.float32)


def _amax_to_scale(amax, fp8_kind, amax_dtype, orig_dtype):
    s = O.amax_to_scale(amax.float().numpy(), _F8[fp8_kind], _HP_BY_CODE[orig_dtype], _HP_BY_CODE[amax_dtype])
    return torch.from_numpy(np.asarray(s, dtype=np.float32).reshape(tuple(amax.shape)).copy())


def _cast_outputs(x, bits, fp8_kind, with_transpose):
    f8 = N.FP8_DTYPE[fp8_kind]
    data = from_np(bits.reshape(tuple(x.shape)), f8)
    if with_transpose:
        cols = x.shape[-1]
        data_t = from_np(bits.reshape(-1, cols).T.copy(), f8)
    else:
        data_t = torch.empty((0,), dtype=f8)
    return data, data_t


def _cast_from_amax(x, amax, fp8_kind, with_transpose):
    name = _HP[x.dtype]
    scale = np.float32(O.amax_to_scale(np.float32(amax.item()), _F8[fp8_kind], name, name))
    bits = O.cast_to_fp8(to_np(x), name, scale, _F8[fp8_kind], name)
    data, data_t = _cast_outputs(x, bits, fp8_kind, with_transpose)
    return data, data_t, torch.tensor(float(scale), dtype=torch.float32)


def _cast_with_scale(x, scale, fp8_kind, product_fp32, with_transpose, amax_out):
    name = _HP[x.dtype]
    bits = O.cast_to_fp8(to_np(x), name, np.float32(scale.float().item()), _F8[fp8_kind],
                         O.FP32 if product_fp32 else name)
    if amax_out is not None:
        amax_out.fill_(float(O.tensor_to_amax(to_np(x), name)))
    return _cast_outputs(x, bits, fp8_kind, with_transpose)


def _transpose_fp8(x):
    return x.view(torch.uint8).t().contiguous().view(x.dtype)


def _delayed_sync(amax, hist, n_e4m3, orig_dtype, scale_out, hist_out):
    rows = hist.shape[0]
    kinds = [O.E4M3] * min(n_e4m3, rows) + [O.E5M2] * max(rows - n_e4m3, 0)
    scales, rolled = O.sync_amax_and_scale(amax.numpy(), hist.numpy(), kinds, _HP_BY_CODE[orig_dtype], True)
    scale_out.copy_(torch.from_numpy(scales.copy()))
    if hist_out is not None:
        hist_out.copy_(torch.from_numpy(rolled.copy()))


def _scaled_mm(a, b_t, scale_a, scale_b, bias, out_dtype, use_fast_accum):
    fa = O.E4M3 if a.dtype == torch.float8_e4m3fn else O.E5M2
    fb = O.E4M3 if b_t.dtype == torch.float8_e4m3fn else O.E5M2
    out = O.mm_float8_emulated(to_np(a), fa, scale_a.float().item(), to_np(b_t).T, fb, scale_b.float().item(), O.FP32)
    res = torch.from_numpy(np.ascontiguousarray(out))
    if bias is not None:
        res = res + bias.float()
    return res.to(out_dtype)


def _rmsnorm_amax(x, weight, eps):
    name = _HP[x.dtype]
    cols = x.shape[-1]
    y, rstd = O.rmsnorm(to_np(x).reshape(-1, cols), name, to_np(weight), eps)
    amax = np.float32(np.nan) if np.isnan(y).any() else np.float32(np.abs(y).max())
    return torch.from_numpy(rstd.copy()), torch.tensor(float(amax), dtype=torch.float32)


def _rmsnorm_cast(x, weight, rstd, amax, fp8_kind):
    name = _HP[x.dtype]
    cols = x.shape[-1]
    xf = O.to_f32(to_np(x).reshape(-1, cols), name)
    o = O.round_f32_to(xf * rstd.numpy()[:, None], name)
    y = O.round_f32_to(o * O.to_f32(to_np(weight), name)[None, :], name)
    scale = np.float32(O.amax_to_scale(np.float32(amax.item()), _F8[fp8_kind], name, name))
    bits = O.cast_to_fp8(O.from_f32(y, name), name, scale, _F8[fp8_kind], name)
    return from_np(bits.reshape(tuple(x.shape)), N.FP8_DTYPE[fp8_kind]), torch.tensor(float(scale), dtype=torch.float32)


def _cast_dynamic(x, fp8_kind):
    data, _, scale = _cast_from_amax(x, _amax(x), fp8_kind, False)
    return data, scale


def _multi_cast_with_scales(xs, scales, fp8_kind, product_fp32):
    return [_cast_with_scale(x, scales[i], fp8_kind, product_fp32, False, None)[0] for i, x in enumerate(xs)]


def _rmsnorm_bwd(x, grad_y, weight, rstd):
    """Gradient of `RN_T(RN_T(x * rstd) * w)` as eager autograd evaluates it for a tensor of dtype T
    (float8_experimental/benchmarks/profile_linear_float8.py:69-74), in fp32 from x and 1/rms."""
    cols = x.shape[-1]
    g32 = grad_y.reshape(-1, cols).float()
    n = x.reshape(-1, cols).float() * rstd[:, None]
    dn = (g32 * weight.float()).to(x.dtype).float()
    dx = rstd[:, None] * (dn - n * (dn * n).mean(-1, keepdim=True))
    dw = (g32 * n.to(x.dtype).float()).sum(0)
    return dx.to(x.dtype).reshape(x.shape), dw.to(weight.dtype)


def _swiglu_bwd(a, b, grad_y, approx=False):
    """Gradient of `silu(a) * b` (profile_linear_float8.py:117-118):
    dy/db = silu(a), dy/da = b * sigmoid(a) * (1 + a * (1 - sigmoid(a)))."""
    a32, g32 = a.float(), grad_y.reshape(a.shape).float()
    sig = torch.sigmoid(a32)
    da = (g32 * b.float()).to(a.dtype).float() * (sig * (1 + a32 * (1 - sig)))
    db = g32 * (a32 * sig).to(a.dtype).float()
    return da.to(a.dtype), db.to(b.dtype)


def _swiglu_amax(a, b, write_y, approx=False):
    name = _HP[a.dtype]
    y = O.swiglu(to_np(a), to_np(b), name)
    amax = np.float32(np.nan) if np.isnan(y).any() else np.float32(np.abs(y).max())
    y_t = from_np(O.from_f32(y, name).reshape(tuple(a.shape)), a.dtype) if write_y else a.new_empty((0,))
    return torch.tensor(float(amax), dtype=torch.float32), y_t


def _swiglu_cast(a, b, amax, fp8_kind):
    name = _HP[a.dtype]
    y = O.swiglu(to_np(a), to_np(b), name)
    scale = np.float32(O.amax_to_scale(np.float32(amax.item()), _F8[fp8_kind], name, name))
    bits = O.cast_to_fp8(O.from_f32(y, name), name, scale, _F8[fp8_kind], name)
    return from_np(bits.reshape(tuple(a.shape)), N.FP8_DTYPE[fp8_kind]), torch.tensor(float(scale), dtype=torch.float32)


def install() -> None:
    """Registers the CPU stand-ins once per process."""
    global _installed
    if _installed:
        return
    lib = torch.library.Library("f8b200", "IMPL")
    lib.impl("amax", _amax, "CPU")
    lib.impl("multi_amax", _multi_amax, "CPU")
    lib.impl("amax_to_scale", _amax_to_scale, "CPU")
    lib.impl("cast_from_amax", _cast_from_amax, "CPU")
    lib.impl("cast_with_scale", _cast_with_scale, "CPU")
    lib.impl("transpose_fp8", _transpose_fp8, "CPU")
    lib.impl("delayed_sync", _delayed_sync, "CPU")
    lib.impl("scaled_mm", _scaled_mm, "CPU")
    lib.impl("swiglu_amax", _swiglu_amax, "CPU")
    lib.impl("swiglu_cast", _swiglu_cast, "CPU")
    lib.impl("rmsnorm_amax", _rmsnorm_amax, "CPU")
    lib.impl("rmsnorm_cast", _rmsnorm_cast, "CPU")
    lib.impl("multi_cast_with_scales", _multi_cast_with_scales, "CPU")
    lib.impl("cast_dynamic", _cast_dynamic, "CPU")
    lib.impl("rmsnorm_bwd", _rmsnorm_bwd, "CPU")
    lib.impl("swiglu_bwd", _swiglu_bwd, "CPU")
    install._lib = lib  # keep the registrations alive
    _installed = True
