"""Dynamic and delayed casts of high-precision tensors to float8, with the entry
points of float8_experimental/float8_scaling_utils.py.
"""
from __future__ import annotations

from typing import Optional

import torch

from ._ops import ops
from .float8_tensor import (
    _DynamicToFloat8Func,
    _want_transposed_copy,
    Float8Tensor,
    GemmInputRole,
    hp_tensor_and_scale_to_float8,
    LinearMMConfig,
    ScaledMMConfig,
    tensor_already_casted_to_fp8,
)
from .float8_utils import amax_history_to_scale, e4m3_dtype, e5m2_dtype, tensor_to_amax, tensor_to_scale

__all__ = [
    "hp_tensor_to_float8_dynamic",
    "hp_tensor_to_float8_delayed",
    "_maybe_initialize_amaxes_scales_for_float8_cast",
    "NoopFwToFloat8E5M2BwDelayed",
    "NoopFwToFloat8E5M2BwDynamic",
]


def hp_tensor_to_float8_dynamic(
    hp_tensor: torch.Tensor,
    float8_dtype: torch.dtype,
    linear_mm_config: LinearMMConfig,
    reduce_amax: bool = False,
    gemm_input_role: GemmInputRole = GemmInputRole.INPUT,
) -> Float8Tensor:
    """amax -> scale -> saturating cast, scale taken from the tensor itself
    (reference: float8_scaling_utils.py:33-62).  Already-fp8 inputs pass through.
    Two kernel launches: the amax reduction and the cast, which computes the scale from
    the amax on the device and also emits the transposed copy for the backward GEMMs."""
    if tensor_already_casted_to_fp8(hp_tensor):
        return hp_tensor
    return _DynamicToFloat8Func.apply(
        hp_tensor, float8_dtype, linear_mm_config, gemm_input_role, reduce_amax, _want_transposed_copy()
    )


def hp_tensor_to_float8_delayed(
    hp_tensor: torch.Tensor,
    s: torch.Tensor,
    float8_dtype: torch.dtype,
    amax_buffer: torch.Tensor,
    linear_mm_config: Optional[LinearMMConfig] = None,
    gemm_input_role: Optional[GemmInputRole] = GemmInputRole.INPUT,
) -> Float8Tensor:
    """Casts with the stored scale `s` and records max|hp_tensor| in `amax_buffer`
    (reference: float8_scaling_utils.py:65-96).  One kernel launch does both from a
    single read of the tensor."""
    return hp_tensor_and_scale_to_float8(
        hp_tensor, s, float8_dtype, linear_mm_config, gemm_input_role, amax_out=amax_buffer
    )


def _maybe_initialize_amaxes_scales_for_float8_cast(
    x, cur_amax, amax_history, scale, scale_fn_name, float8_dtype, is_initialized, reduce_amax
):
    """First-iteration seeding of the delayed-scaling buffers from the data
    (reference: float8_scaling_utils.py:99-125)."""
    if is_initialized:
        return
    with torch.no_grad():
        local = x._local_tensor if hasattr(x, "_local_tensor") else x
        new_amax = tensor_to_amax(local, reduce_amax=reduce_amax)
        cur_amax.fill_(new_amax)
        amax_history[0] = new_amax
        scale.copy_(amax_history_to_scale(amax_history, float8_dtype, local.dtype, scale_fn_name))


@torch._dynamo.allow_in_graph
class NoopFwToFloat8E5M2BwDelayed(torch.autograd.Function):
    """Identity in forward; in backward the incoming gradient is cast to e5m2 with
    delayed scaling, seeding the buffers on first use
    (reference: float8_scaling_utils.py:128-185)."""

    @staticmethod
    def forward(ctx, tensor, fp8_amax_grad_output, fp8_amax_history_grad_output, fp8_scale_grad_output,
                scale_fn_name, is_amax_initialized, linear_mm_config: LinearMMConfig):
        # Plain attributes, not save_for_backward: the buffers are views into slabs shared by
        # all layers (see sync_float8_amax_and_scale_history) and are legitimately written
        # in place by other layers' backward passes before this one runs.
        ctx.f8_buffers = (fp8_amax_grad_output, fp8_amax_history_grad_output, fp8_scale_grad_output)
        ctx.scale_fn_name = scale_fn_name
        ctx.is_amax_initialized = is_amax_initialized
        ctx.linear_mm_config = linear_mm_config
        return tensor

    @staticmethod
    def backward(ctx, go):
        amax_buf, history_buf, scale_buf = ctx.f8_buffers
        _maybe_initialize_amaxes_scales_for_float8_cast(
            go, amax_buf, history_buf, scale_buf, ctx.scale_fn_name, e5m2_dtype, ctx.is_amax_initialized,
            reduce_amax=True,
        )
        res = hp_tensor_and_scale_to_float8(
            go, scale_buf, e5m2_dtype, ctx.linear_mm_config, GemmInputRole.GRAD_OUTPUT, amax_out=amax_buf,
            with_transpose=_want_transposed_copy(),
        )
        return res, None, None, None, None, None, None


@torch._dynamo.allow_in_graph
class NoopFwToFloat8E5M2BwDynamic(torch.autograd.Function):
    """Identity in forward; in backward the incoming gradient is cast to e5m2 with
    dynamic scaling (reference: float8_scaling_utils.py:188-216)."""

    @staticmethod
    def forward(ctx, tensor, linear_mm_config: LinearMMConfig):
        ctx.linear_mm_config = linear_mm_config
        return tensor

    @staticmethod
    def backward(ctx, gradY):
        if tensor_already_casted_to_fp8(gradY):
            return gradY, None
        fp8 = _DynamicToFloat8Func.apply(
            gradY, e5m2_dtype, ctx.linear_mm_config, GemmInputRole.GRAD_OUTPUT, False, _want_transposed_copy()
        )
        return fp8, None
