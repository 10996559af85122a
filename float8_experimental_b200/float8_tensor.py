"""`Float8Tensor`: fp8 bytes + scale travelling through PyTorch as one tensor.

Same fields and construction signature as float8_experimental/float8_tensor.py:243-363
(`_data`, `_scale`, `_orig_dtype`, `_linear_mm_config`, `_gemm_input_role`).  One
addition: `_alt`, an optional second copy of the same 2-D values in the opposite memory
order (column-major when `_data` is row-major).  The cast kernel emits it from the same
read of the high-precision tensor, so the backward GEMMs find K-major operands without
the transpose copies the reference makes in float8_ops.py:150-153.
"""
from __future__ import annotations

import os

import enum
from collections import namedtuple
from typing import Dict, Optional

import torch
import torch.distributed as dist
import torch.distributed._functional_collectives as funcol
from torch.distributed._tensor import DTensor

from ._ops import ops
from .float8_utils import _kind, e4m3_dtype

aten = torch.ops.aten

# Per-GEMM switches (reference: float8_tensor.py:55-59).  `emulate` is carried but has
# no effect here: there is no emulated GEMM.
ScaledMMConfig = namedtuple(
    "ScaledMMConfig",
    ["emulate", "use_fast_accum", "fp8_output", "pad_inner_dim"],
    defaults=[False, False, False, False],
)

# The three GEMMs of a linear layer (reference: float8_tensor.py:66-74).
LinearMMConfig = namedtuple(
    "LinearMMConfig",
    ["output", "grad_input", "grad_weight"],
    defaults=[
        ScaledMMConfig(False, True, False, False),
        ScaledMMConfig(False, False, False, False),
        ScaledMMConfig(False, False, False, False),
    ],
)


class GemmInputRole(enum.Enum):
    """Which operand of the linear layer a Float8Tensor is (reference: float8_tensor.py:77-87)."""

    INPUT = "input"
    WEIGHT = "weight"
    GRAD_OUTPUT = "grad_output"


_GEMM_OF_ROLES = {
    (GemmInputRole.INPUT, GemmInputRole.WEIGHT): "output",
    (GemmInputRole.GRAD_OUTPUT, GemmInputRole.WEIGHT): "grad_input",
    (GemmInputRole.GRAD_OUTPUT, GemmInputRole.INPUT): "grad_weight",
}


def choose_scaled_mm_config(a_role, a_linear_mm_config, b_role, b_linear_mm_config) -> ScaledMMConfig:
    """Picks the GEMM config from the operand roles and checks both operands agree
    (reference: float8_tensor.py:91-113; the assertion texts are part of the contract)."""
    which = _GEMM_OF_ROLES.get((a_role, b_role))
    if which is None:
        raise AssertionError(f"unexpected a_role {a_role} and b_role {b_role}")
    a_cfg, b_cfg = getattr(a_linear_mm_config, which), getattr(b_linear_mm_config, which)
    assert a_cfg == b_cfg, f"linear_mm_config.{which} mismatch: {a_cfg} vs {b_cfg}"
    return a_cfg


def tensor_already_casted_to_fp8(tensor: torch.Tensor) -> bool:
    """True for a Float8Tensor, also when wrapped in a DTensor or an in-flight
    functional collective (reference: float8_tensor.py:116-128)."""
    if isinstance(tensor, Float8Tensor):
        return True
    if isinstance(tensor, DTensor):
        return tensor_already_casted_to_fp8(tensor._local_tensor)
    if isinstance(tensor, funcol.AsyncCollectiveTensor):
        return tensor_already_casted_to_fp8(tensor.elem)
    return False


def _want_transposed_copy() -> bool:
    """Whether casts also emit the transposed fp8 copy (`Float8Tensor._alt`).  The GEMM reads
    an operand in either memory order, so nothing needs that copy any more and the default is
    no; F8B200_CAST_TRANSPOSED=1 in the environment brings the copies back (the backward GEMMs
    then run on K-major operands only) for comparisons."""
    return os.environ.get("F8B200_CAST_TRANSPOSED", "0") == "1"


def _wrap_cast_result(data, data_t, scale, orig_dtype, linear_mm_config, gemm_input_role):
    out = Float8Tensor(data, scale, orig_dtype, linear_mm_config, gemm_input_role)
    if data_t.numel() == data.numel() and data.numel() > 0:
        # data_t is [cols, rows] row-major == the flattened [rows, cols] matrix column-major
        out._alt = data_t.t()
    return out


def _mesh_max_(amax: torch.Tensor, dt: DTensor) -> None:
    """All-reduce MAX of a local amax over every mesh dimension `dt` is sharded on."""
    for dim, placement in enumerate(dt.placements):
        if placement.is_shard():
            dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=dt.device_mesh.get_group(dim))
        elif placement.is_partial():
            raise NotImplementedError("cannot cast a Partial DTensor to float8")


def _rewrap_like(dt: DTensor, local_fp8: "Float8Tensor") -> DTensor:
    return DTensor.from_local(
        local_fp8, dt.device_mesh, dt.placements, run_check=False, shape=dt.size(), stride=dt.stride()
    )


@torch._dynamo.allow_in_graph
class _ToFloat8ConstrFunc(torch.autograd.Function):
    """high precision + given scale -> Float8Tensor; gradient passes through unchanged
    (reference: float8_tensor.py:131-195).

    Rounding of `tensor * scale` follows PyTorch type promotion, which the reference gets
    implicitly: with a 0-dim scale the product is rounded to the tensor's dtype before
    the clamp, with a [1]-shaped scale (delayed-scaling buffers) it stays fp32."""

    @staticmethod
    def forward(ctx, tensor, scale, float8_dtype=e4m3_dtype, linear_mm_config=None,
                gemm_input_role=GemmInputRole.INPUT, amax_out=None, with_transpose=False):
        kind = _kind(float8_dtype)
        if isinstance(tensor, DTensor):
            local = tensor._local_tensor
            local_scale = scale._local_tensor if isinstance(scale, DTensor) else scale
        else:
            local, local_scale = tensor, scale
        prod_dtype = torch.result_type(local, local_scale)
        if prod_dtype not in (local.dtype, torch.float32):
            raise NotImplementedError(f"tensor*scale would be computed in {prod_dtype}")
        data, data_t = ops.cast_with_scale(
            local, local_scale, kind, prod_dtype == torch.float32, with_transpose, amax_out
        )
        out = _wrap_cast_result(data, data_t, local_scale, local.dtype, linear_mm_config, gemm_input_role)
        return _rewrap_like(tensor, out) if isinstance(tensor, DTensor) else out

    @staticmethod
    def backward(ctx, g):
        return g, None, None, None, None, None, None


@torch._dynamo.allow_in_graph
class _DynamicToFloat8Func(torch.autograd.Function):
    """Dynamic scaling in two launches: amax reduction, then a cast that derives the
    scale from the amax word on the device (no host round trip, no scale kernels).
    Covers tensor_to_scale + hp_tensor_and_scale_to_float8 of
    float8_experimental/float8_scaling_utils.py:33-62; for a DTensor the local amax is
    all-reduced (MAX) over the mesh between the two launches."""

    @staticmethod
    def forward(ctx, tensor, float8_dtype, linear_mm_config, gemm_input_role, reduce_amax, with_transpose):
        kind = _kind(float8_dtype)
        is_dt = isinstance(tensor, DTensor)
        local = tensor._local_tensor if is_dt else tensor
        amax = ops.amax(local)
        if is_dt:
            _mesh_max_(amax, tensor)
        elif reduce_amax and dist.is_initialized():
            dist.all_reduce(amax, op=dist.ReduceOp.MAX)
        data, data_t, scale = ops.cast_from_amax(local, amax, kind, with_transpose)
        out = _wrap_cast_result(data, data_t, scale, local.dtype, linear_mm_config, gemm_input_role)
        return _rewrap_like(tensor, out) if is_dt else out

    @staticmethod
    def backward(ctx, g):
        return g, None, None, None, None, None


@torch._dynamo.allow_in_graph
class _FromFloat8ConstrFunc(torch.autograd.Function):
    """Float8Tensor -> original precision: `_data.to(orig) / _scale`
    (reference: float8_tensor.py:198-212)."""

    @staticmethod
    def forward(ctx, tensor):
        return tensor._data.to(tensor._orig_dtype) / tensor._scale

    @staticmethod
    def backward(ctx, g):
        return g, None, None


def hp_tensor_and_scale_to_float8(
    hp_tensor: torch.Tensor,
    s: torch.Tensor,
    float8_dtype=e4m3_dtype,
    linear_mm_config: Optional[LinearMMConfig] = None,
    gemm_input_role: Optional[GemmInputRole] = GemmInputRole.INPUT,
    amax_out: Optional[torch.Tensor] = None,
    with_transpose: Optional[bool] = None,
):
    """Casts `hp_tensor` with a precomputed scale (reference: float8_tensor.py:215-240).

    `amax_out` (an fp32 buffer) additionally receives max|hp_tensor| from the same read;
    delayed scaling uses it to record the current amax while casting.  `with_transpose`
    asks for the second (transposed) layout; default: `_want_transposed_copy()`."""
    if with_transpose is None:
        with_transpose = _want_transposed_copy()
    return _ToFloat8ConstrFunc.apply(
        hp_tensor, s, float8_dtype, linear_mm_config, gemm_input_role, amax_out, with_transpose
    )


class Float8Tensor(torch.Tensor):
    """Wrapper subclass that presents as a tensor of `_orig_dtype` and holds
    `_data` (fp8 bytes), `_scale` (fp32, one element; data = hp * scale),
    `_orig_dtype`, `_linear_mm_config`, `_gemm_input_role`, and optionally `_alt`.
    Only the ops in `float8_ops.FLOAT8_OPS_TABLE` are defined on it."""

    __slots__ = ["_data", "_scale", "_orig_dtype", "_linear_mm_config", "_gemm_input_role", "_alt"]

    def __new__(cls, data, scale, orig_dtype, linear_mm_config, gemm_input_role=GemmInputRole.INPUT):
        assert scale.numel() == 1, "Scale should contain a single value, but got: {} elements".format(scale.numel())
        self = torch.Tensor._make_wrapper_subclass(
            cls,
            data.size(),
            strides=data.stride(),
            storage_offset=data.storage_offset(),
            dtype=orig_dtype,
            layout=data.layout,
            requires_grad=data.requires_grad,
            device=data.device,
        )
        self._data = data
        self._scale = scale
        self._orig_dtype = orig_dtype
        self._linear_mm_config = linear_mm_config if linear_mm_config is not None else LinearMMConfig()
        self._gemm_input_role = gemm_input_role
        self._alt = None
        return self

    def __repr__(self):
        return (
            f"Float8Tensor(dtype={self._data.dtype}, scale={self._scale}, "
            f"linear_mm_config={self._linear_mm_config}\ngemm_input_role={self._gemm_input_role}\n"
            f"as_orig_prec={self.to_original_precision()}"
        )

    def __tensor_flatten__(self):
        meta = {
            "_orig_dtype": self._orig_dtype,
            "_linear_mm_config": self._linear_mm_config,
            "_gemm_input_role": self._gemm_input_role,
        }
        return ["_data", "_scale"], meta

    @staticmethod
    def __tensor_unflatten__(inner_tensors: Dict, metadata, outer_size, outer_stride):
        assert len(inner_tensors) == 2
        return Float8Tensor(
            inner_tensors["_data"],
            inner_tensors["_scale"],
            metadata["_orig_dtype"],
            metadata["_linear_mm_config"],
            metadata["_gemm_input_role"],
        )

    def to_original_precision(self):
        return _FromFloat8ConstrFunc.apply(self)

    @classmethod
    def __torch_dispatch__(cls, func, types, args, kwargs=None):
        from .float8_ops import FLOAT8_OPS_TABLE

        # ops mixing Float8Tensor with another subclass are left to that subclass
        def compatible(t):
            return (
                issubclass(cls, t)
                or issubclass(torch._subclasses.fake_tensor.FakeTensor, t)
                or issubclass(torch._subclasses.functional_tensor.FunctionalTensor, t)
            )

        if not all(compatible(t) for t in types):
            return NotImplemented
        handler = FLOAT8_OPS_TABLE.get(func)
        if handler is None:
            raise NotImplementedError(f"attempting to run {func}, this is not supported")
        return handler(func, args, kwargs)

    # user-level torch functions must not re-wrap results as Float8Tensor
    __torch_function__ = torch._C._disabled_torch_function_impl
