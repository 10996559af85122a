"""Unwrapped scaled GEMM entry point, signature of
float8_experimental/float8_python_api.py:24-64.

The reference takes the reciprocal of both scales with two tiny kernels and calls
`torch._scaled_mm` (cuBLASLt).  Here one launch of the tcgen05 kernel does all of it:
the reciprocals, the fp32-accumulated product, the bias add and the conversion to the
output dtype happen in the kernel's epilogue.
"""
from __future__ import annotations

from typing import Optional

import torch

from ._ops import ops


def addmm_float8_unwrapped(
    a_data: torch.Tensor,
    a_scale: torch.Tensor,
    b_data: torch.Tensor,
    b_scale: torch.Tensor,
    output_dtype: torch.dtype,
    output_scale: Optional[torch.Tensor] = None,
    bias: Optional[torch.Tensor] = None,
    use_fast_accum: bool = False,
) -> torch.Tensor:
    """out = (a_data @ b_data) / (a_scale * b_scale) [+ bias], in `output_dtype`.

    a_data: [M, K] fp8, row-major.  b_data: [K, N] fp8, column-major (a transposed view of
    an [N, K] row-major buffer).  Scales are the factors the operands were multiplied by
    when cast.  `output_scale` (fp8 output) is not supported, as in the reference's call
    sites (float8_ops.py:186,223 always pass None)."""
    if output_scale is not None:
        raise NotImplementedError("fp8 output (output_scale) is not implemented")
    if a_data.dim() != 2 or b_data.dim() != 2:
        raise RuntimeError("addmm_float8_unwrapped expects 2-D operands")
    return ops.scaled_mm(a_data, b_data.t(), a_scale, b_scale, bias, output_dtype, use_fast_accum)
