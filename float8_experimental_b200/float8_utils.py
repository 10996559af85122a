"""amax / scale / saturated-cast helpers with the signatures of
float8_experimental/float8_utils.py, implemented on the sm_100a kernels.

Diagnostics (`compute_error`, `fp8_tensor_statistics`) use plain torch ops; they are
not part of the training step.
"""
from __future__ import annotations

from typing import Iterable, Literal, Tuple, Union

import torch
import torch.distributed as dist

from . import _native as N
from . import config
from ._ops import ops

# float8_experimental/float8_utils.py:19 -- floor for the amax before the reciprocal.
EPS = 1e-12

FP8_TYPES = {
    torch.float8_e4m3fn,
    torch.float8_e5m2,
    torch.float8_e4m3fnuz,
    torch.float8_e5m2fnuz,
}

if config.use_fnuz_dtype:
    raise NotImplementedError("fnuz float8 flavours are ROCm-only; the sm_100a kernels implement e4m3fn / e5m2")
e4m3_dtype = torch.float8_e4m3fn
e5m2_dtype = torch.float8_e5m2


def _kind(float8_dtype: torch.dtype) -> int:
    if float8_dtype is torch.float8_e4m3fn:
        return N.E4M3
    if float8_dtype is torch.float8_e5m2:
        return N.E5M2
    raise ValueError(f"Unsupported float8_dtype: {float8_dtype}")


@torch.no_grad()
def amax_to_scale(amax: torch.Tensor, float8_dtype: torch.dtype, orig_dtype: torch.dtype) -> torch.Tensor:
    """fp32 scale(s) for the given amax(es); same shape as `amax`.

    Mirrors float8_experimental/float8_utils.py:35-57 bit for bit: the arithmetic runs
    in `amax.dtype` as reciprocal-then-multiply with a rounding after every step, and
    the result is clamped to the fp16 maximum when `orig_dtype` is fp16."""
    return ops.amax_to_scale(amax, _kind(float8_dtype), N.hp_code(amax.dtype), N.hp_code(orig_dtype))


@torch.no_grad()
def amax_history_to_scale(
    amax_history: torch.Tensor,
    float8_dtype: torch.dtype,
    orig_dtype: torch.dtype,
    history_to_scale_fn_type: Literal["max"],
) -> torch.Tensor:
    """Scale from one amax history (reference: float8_utils.py:60-77).  Amaxes are
    non-negative, so the max of the history is its amax."""
    if history_to_scale_fn_type != "max":
        raise NotImplementedError()
    return amax_to_scale(ops.amax(amax_history), float8_dtype, orig_dtype)


@torch.no_grad()
def amax_history_to_scale_stack(
    amax_history: torch.Tensor,
    float8_dtype: torch.dtype,
    orig_dtype: torch.dtype,
    history_to_scale_fn_type: Literal["max"],
) -> torch.Tensor:
    """One scale per row of a [rows, history_len] stack (reference: float8_utils.py:80-99)."""
    if history_to_scale_fn_type != "max":
        raise NotImplementedError(
            f"Invalid history_to_scale_fn_type, only 'max' is supported. Got: {history_to_scale_fn_type}"
        )
    _kind(float8_dtype)
    hist = amax_history.float().contiguous()
    rows = hist.shape[0]
    scale = torch.empty((rows,), dtype=torch.float32, device=hist.device)
    # max(last column, first H-1 columns) == max of the whole row
    ops.delayed_sync(hist[:, -1].contiguous(), hist, rows if float8_dtype is e4m3_dtype else 0,
                     N.hp_code(orig_dtype), scale, None)
    return scale


@torch.no_grad()
def tensor_to_amax(x: torch.Tensor, reduce_amax: bool = False) -> torch.Tensor:
    """max(|x|) as a 0-dim tensor of x.dtype (reference: float8_utils.py:102-112)."""
    amax = ops.amax(x)
    if reduce_amax and dist.is_initialized():
        dist.all_reduce(amax, op=dist.ReduceOp.MAX)
    return amax.to(x.dtype)


@torch.no_grad()
def tensor_to_scale(x: torch.Tensor, float8_dtype: torch.dtype, reduce_amax: bool = False) -> torch.Tensor:
    """Dynamic scale of `x` (reference: float8_utils.py:115-120)."""
    return amax_to_scale(tensor_to_amax(x, reduce_amax=reduce_amax), float8_dtype, x.dtype)


def to_fp8_saturated(x: torch.Tensor, float8_dtype: torch.dtype) -> torch.Tensor:
    """clamp to the finite fp8 range, then round to nearest even
    (reference: float8_utils.py:123-139)."""
    one = torch.ones((), dtype=torch.float32, device=x.device)
    data, _ = ops.cast_with_scale(x, one, _kind(float8_dtype), True, False, None)
    return data


def compute_error(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """Signal-to-quantisation-noise ratio in dB (reference: float8_utils.py:142-154)."""
    signal = torch.norm(x)
    noise = torch.norm(x - y)
    return 20 * torch.log10(signal / noise)


def fp8_tensor_statistics(tensor, float8_dtype=e4m3_dtype) -> Tuple[int, ...]:
    """(#zeros, #saturated) of a Float8Tensor (reference: float8_utils.py:157-176)."""
    if float8_dtype not in FP8_TYPES:
        raise ValueError(f"Unsupported float8_dtype: {float8_dtype}")
    top = torch.finfo(float8_dtype).max
    vals = tensor._data.to(dtype=tensor._orig_dtype)
    return ((vals == 0).sum().item(), (torch.abs(vals) == top).sum().item())


def is_row_major(stride) -> bool:
    assert len(stride) == 2, "is_row_major only supports 2D tensors"
    return stride[0] > stride[1] and stride[1] == 1


def _get_min_alignment(size: int, alignment_value: int) -> int:
    """Smallest multiple of `alignment_value` that is >= size."""
    return -(-size // alignment_value) * alignment_value


def pad_tensor_for_matmul(tensor: torch.Tensor, dims: Union[int, Iterable[int]]) -> torch.Tensor:
    """Zero-pads the chosen dims of a 2-D tensor to multiples of 16
    (reference: float8_utils.py:206-247)."""
    assert tensor.dim() == 2
    dims = (dims,) if isinstance(dims, int) else tuple(dims)
    r, c = tensor.shape
    r_pad = _get_min_alignment(r, 16) if 0 in dims else r
    c_pad = _get_min_alignment(c, 16) if 1 in dims else c
    if (r_pad, c_pad) == (r, c):
        return tensor
    return torch.nn.functional.pad(tensor, (0, c_pad - c, 0, r_pad - r))
