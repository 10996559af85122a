"""Producers fused into the dynamic fp8 cast of their output: RMSNorm and the SwiGLU gate.

The reference models the start of a transformer block as RMSNorm -> Float8Linear
(float8_experimental/benchmarks/profile_linear_float8.py:52-74,129-149) and leaves it to
torch.compile to fuse the norm with the amax and cast kernels that follow.  Here the fusion
is two hand-written launches: pass A reads x and produces 1/rms per row and the amax of the
normalised tensor, pass B reads x again and writes the fp8 bytes.  The normalised tensor never
reaches memory: 5 bytes of traffic per element instead of 9.

`rms_norm_to_float8_dynamic(x, weight, eps, ...)` returns the `Float8Tensor` that
`hp_tensor_to_float8_dynamic(RMSNorm(x), ...)` would return (same bytes and scale whenever
the two agree on the last bit of 1/rms, see `tests/test_fused_norm_gpu.py`); a `Float8Linear`
takes it as an already-cast input, as it does for tensor-parallel inputs
(float8_experimental/float8_linear.py:240-262).

`swiglu_to_float8_dynamic(a, b, ...)` fuses the FFN gate `silu(a) * b` that feeds the w2
linear (profile_linear_float8.py:117-118) with the amax pass: 9 bytes per element instead of 17.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ._ops import ops
from .float8_tensor import Float8Tensor, GemmInputRole, LinearMMConfig
from .float8_utils import _kind, e4m3_dtype

__all__ = ["rms_norm_to_float8_dynamic", "Float8RMSNorm", "swiglu_to_float8_dynamic"]


class _RMSNormToFloat8(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, float8_dtype, linear_mm_config, gemm_input_role, reduce_amax):
        if weight.dtype != x.dtype:
            raise RuntimeError(f"rms_norm_to_float8_dynamic: weight dtype {weight.dtype} differs from x dtype {x.dtype}")
        rstd, amax = ops.rmsnorm_amax(x, weight, float(eps))
        if reduce_amax and dist.is_initialized():
            dist.all_reduce(amax, op=dist.ReduceOp.MAX)
        data, scale = ops.rmsnorm_cast(x, weight, rstd, amax, _kind(float8_dtype))
        ctx.save_for_backward(x, weight, rstd)
        return Float8Tensor(data, scale, x.dtype, linear_mm_config, gemm_input_role)

    @staticmethod
    def backward(ctx, g):
        # the cast is transparent to autograd (float8_experimental/float8_tensor.py:193-195); what is
        # left is the RMSNorm backward, in fp32 from the saved x and 1/rms
        x, weight, rstd = ctx.saved_tensors
        dx, dw = ops.rmsnorm_bwd(x, g if g.dtype == x.dtype else g.to(x.dtype), weight, rstd)
        return dx, dw, None, None, None, None, None


def rms_norm_to_float8_dynamic(
    x: torch.Tensor,
    weight: torch.Tensor,
    eps: float = 1e-6,
    float8_dtype: torch.dtype = e4m3_dtype,
    linear_mm_config: LinearMMConfig = None,
    gemm_input_role: GemmInputRole = GemmInputRole.INPUT,
    reduce_amax: bool = False,
) -> Float8Tensor:
    """fp8(RMSNorm(x) * weight) with a dynamic per-tensor scale, without materialising the
    normalised tensor.  `x` [..., D] and `weight` [D] share one dtype (bf16 / fp16 / fp32)."""
    if x.numel() == 0:
        raise RuntimeError("rms_norm_to_float8_dynamic: empty input (amax of an empty tensor is undefined)")
    return _RMSNormToFloat8.apply(
        x, weight, eps, float8_dtype, linear_mm_config or LinearMMConfig(), gemm_input_role, reduce_amax
    )


class Float8RMSNorm(torch.nn.Module):
    """RMSNorm whose output is handed to the following `Float8Linear` already cast
    (parameters and formula of RMSNorm in profile_linear_float8.py:52-77).  `linear_mm_config`
    must be the config of the linear that consumes the output (`Float8Linear.linear_mm_config`)."""

    def __init__(self, dim: int, eps: float = 1e-6, linear_mm_config: LinearMMConfig = None,
                 device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.weight = torch.nn.Parameter(torch.ones(dim, device=device, dtype=dtype))
        self.linear_mm_config = linear_mm_config or LinearMMConfig()

    def forward(self, x: torch.Tensor) -> Float8Tensor:
        return rms_norm_to_float8_dynamic(x, self.weight, self.eps, e4m3_dtype, self.linear_mm_config)

    def reset_parameters(self):
        torch.nn.init.ones_(self.weight)


class _SwiGLUToFloat8(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, float8_dtype, linear_mm_config, gemm_input_role, reduce_amax, recompute, approx_gate):
        amax, y = ops.swiglu_amax(a, b, not recompute, approx_gate)
        if reduce_amax and dist.is_initialized():
            dist.all_reduce(amax, op=dist.ReduceOp.MAX)
        if recompute:
            data, scale = ops.swiglu_cast(a, b, amax, _kind(float8_dtype))
        else:
            data, _, scale = ops.cast_from_amax(y, amax, _kind(float8_dtype), False)
            del y  # a temporary: nothing keeps it for backward
        ctx.save_for_backward(a, b)
        ctx.approx_gate = approx_gate
        return Float8Tensor(data, scale, a.dtype, linear_mm_config, gemm_input_role)

    @staticmethod
    def backward(ctx, g):
        # y = silu(a) * b:  dy/db = silu(a),  dy/da = b * sigmoid(a) * (1 + a * (1 - sigmoid(a)))
        a, b = ctx.saved_tensors
        da, db = ops.swiglu_bwd(a, b, g if g.dtype == a.dtype else g.to(a.dtype), ctx.approx_gate)
        return da, db, None, None, None, None, None, None


def swiglu_to_float8_dynamic(
    a: torch.Tensor,
    b: torch.Tensor,
    float8_dtype: torch.dtype = e4m3_dtype,
    linear_mm_config: LinearMMConfig = None,
    gemm_input_role: GemmInputRole = GemmInputRole.INPUT,
    reduce_amax: bool = False,
    recompute: bool = False,
    approx_gate: bool = False,
) -> Float8Tensor:
    """fp8(silu(a) * b) with a dynamic per-tensor scale in two launches and 9 bytes of traffic
    per element (17 unfused).  `a` and `b` share shape and dtype; they may be column slices of one
    fused w1|w3 output.  By default the first launch writes the gate output once (a temporary in
    the input dtype, freed on return) while it takes the amax, and the second is the plain cast;
    `recompute=True` never writes it and evaluates the gate in both launches instead (no
    temporary, same bytes moved, more arithmetic: slower).  Both give the same bytes.

    `approx_gate=True` (opt-in; 16-bit inputs whose last dimension is a multiple of 8, not with
    `recompute`) evaluates the sigmoid with the hardware's approximate exp2 and reciprocal in forward and
    backward: the gate output, its amax and the gradients are within one ulp of the input dtype of the exact
    path's, hence every fp8 byte within one fp8 step; shapes the approximate kernels do not cover raise."""
    if a.numel() == 0:
        raise RuntimeError("swiglu_to_float8_dynamic: empty input (amax of an empty tensor is undefined)")
    if approx_gate and recompute:
        raise RuntimeError("swiglu_to_float8_dynamic: approx_gate needs the gate output written once (recompute=False)")
    return _SwiGLUToFloat8.apply(
        a, b, float8_dtype, linear_mm_config or LinearMMConfig(), gemm_input_role, reduce_amax, recompute,
        approx_gate
    )
