"""Operator table of `Float8Tensor` (`__torch_dispatch__` handlers).

Covers the same aten / c10d ops as float8_experimental/float8_ops.py:33-363.  The
matrix products go to the tcgen05 GEMM (`f8b200::scaled_mm`), which reads an operand in
either memory order (K contiguous or rows contiguous), so the transposed fp8 copies of the
reference's `preprocess_addmm` are not made; only an operand that is contiguous in neither
order, or misaligned for TMA, is copied.
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch
from torch.utils._pytree import tree_map

from .float8_python_api import addmm_float8_unwrapped
from .float8_tensor import choose_scaled_mm_config, Float8Tensor

aten = torch.ops.aten
c10d_functional = torch.ops.c10d_functional
_c10d_functional = torch.ops._c10d_functional
FLOAT8_OPS_TABLE: Dict[Any, Any] = {}


def implements(aten_ops):
    """Decorator: route the listed ops to the decorated handler."""

    def register(fn):
        FLOAT8_OPS_TABLE.update({op: fn for op in aten_ops})
        return fn

    return register


def _like(src: Float8Tensor, data: torch.Tensor, alt: Optional[torch.Tensor] = None, **over) -> Float8Tensor:
    out = Float8Tensor(
        data,
        over.get("scale", src._scale),
        over.get("orig_dtype", src._orig_dtype),
        src._linear_mm_config,
        src._gemm_input_role,
    )
    out._alt = alt
    return out


def _flat_rows_cols(t: torch.Tensor):
    cols = t.shape[-1] if t.dim() > 0 else 1
    return (t.numel() // cols if cols else 0), cols


# ---------------------------------------------------------------------------
# metadata-only ops: applied to the bytes, scale and config carried over
# ---------------------------------------------------------------------------
@implements(
    [
        aten.view.default,
        aten._unsafe_view.default,
        aten.t.default,
        aten.as_strided.default,
        aten.clone.default,
        aten.detach.default,
        aten.slice.Tensor,
        aten.transpose.int,
        aten.fill_.Scalar,
    ]
)
def float8_desugar_op(aten_op, args, kwargs=None):
    src = args[0]
    kwargs = kwargs or {}
    data = aten_op(src._data, *args[1:], **kwargs)
    alt = None
    if src._alt is not None:
        if aten_op is aten.detach.default:
            alt = src._alt
        elif aten_op is aten.t.default and src._data.dim() == 2:
            alt = src._alt.t()
        elif aten_op is aten.transpose.int and src._data.dim() == 2 and {args[1] % 2, args[2] % 2} == {0, 1}:
            alt = src._alt.t()
        elif aten_op in (aten.view.default, aten._unsafe_view.default):
            # a reshape that keeps the last dimension keeps the flattened [rows, cols] matrix
            if src._data.is_contiguous() and data.is_contiguous() and _flat_rows_cols(data) == _flat_rows_cols(src._data):
                alt = src._alt
    return _like(src, data, alt)


@implements([aten.split.Tensor])
def float8_split(aten_op, args, kwargs=None):
    src = args[0]
    return [_like(src, piece) for piece in aten_op(src._data, *args[1:], **(kwargs or {}))]


@implements([aten.cat.default])
def float8_cat(aten_op, args, kwargs=None):
    chunks = args[0]
    head = chunks[0]
    for c in chunks:
        assert isinstance(c, Float8Tensor), "Expecting all chunks to be of type Float8Tensor"
        assert c._orig_dtype == head._orig_dtype, "Expecting all chunks to be of the same dtype"
        assert c._scale is head._scale, "Expecting all chunks to have thee same scale as a result of a split"
        assert (
            c._linear_mm_config is head._linear_mm_config
        ), "Expecting all chunks to have thee same mm config as a result of a split"
        assert c._data.dtype == head._data.dtype, "Expecting all chunks to be of the same dtype as a result of a split"
        assert (
            c._gemm_input_role is head._gemm_input_role
        ), "Expecting all chunks to have the same gemm_input_role as a result of a split"
    # concatenate as bytes: aten.cat has no fp8 kernel
    joined = aten_op([c._data.view(torch.uint8) for c in chunks], *args[1:], **(kwargs or {}))
    return _like(head, joined.view(head._data.dtype))


@implements([aten.sum.dim_IntList])
def float8_cast_up_op(aten_op, args, kwargs=None):
    """Reductions run in the original precision (needed for the bias gradient when
    grad_output arrives as fp8; reference: float8_ops.py:111-128)."""

    def up(x):
        return x.to_original_precision() if isinstance(x, Float8Tensor) else x

    return aten_op(*tree_map(up, args), **tree_map(up, kwargs or {}))


# ---------------------------------------------------------------------------
# matrix products
# ---------------------------------------------------------------------------
def _k_major(data: torch.Tensor) -> bool:
    return data.dim() == 2 and data.stride(1) == 1 and data.stride(0) >= data.shape[1]


def _mn_major(data: torch.Tensor) -> bool:
    """A transposed view of a row-major [K, rows] buffer that TMA can address."""
    return (
        data.dim() == 2
        and data.stride(0) == 1
        and data.shape[1] > 1
        and data.stride(1) >= data.shape[0]
        and data.stride(1) % 16 == 0
        and data.data_ptr() % 16 == 0
    )


def _gemm_readable(t: Float8Tensor, logical: torch.Tensor, alt: Optional[torch.Tensor]) -> torch.Tensor:
    """`logical` is the [rows, K] operand as a view of `t._data`.  Returned as it lies when
    the GEMM can read it (K contiguous, or rows contiguous: the kernels take both), else the
    pre-emitted copy in the other memory order when there is one, else a K-major copy."""
    if _k_major(logical) or _mn_major(logical):
        return logical
    if alt is not None and (_k_major(alt) or _mn_major(alt)):
        return alt
    return logical.contiguous()


def _row_major_operand(t: Float8Tensor) -> torch.Tensor:
    """The [M, K] operand."""
    return _gemm_readable(t, t._data, t._alt)


def _col_major_operand_as_nk(t: Float8Tensor) -> torch.Tensor:
    """The [K, N] operand returned as its transpose [N, K]."""
    return _gemm_readable(t, t._data.t(), t._alt.t() if t._alt is not None else None)


def preprocess_addmm(a: Float8Tensor, b: Float8Tensor):
    """Operands as the GEMM can read them: A [M,K] and B (returned as a [K,N] view of its [N,K]
    form), each K-major or MN-major as it lies; the inner-dimension contract of the reference
    (float8_ops.py:131-155) without its padding copies."""
    cfg = choose_scaled_mm_config(a._gemm_input_role, a._linear_mm_config, b._gemm_input_role, b._linear_mm_config)
    a_data = _row_major_operand(a)
    b_nk = _col_major_operand_as_nk(b)
    if cfg.pad_inner_dim:
        assert a._data.size(1) == b._data.size(
            0
        ), f"Inner dims must match for mm, got {a._data.size(1)} and {b._data.size(0)}"
    if a_data.shape[1] % 16 != 0 and not cfg.pad_inner_dim:
        # same contract as the reference, whose cuBLASLt path needs K % 16 == 0 unless it pads
        raise RuntimeError(
            f"float8 GEMM needs the inner dimension to be a multiple of 16, got {a_data.shape[1]}; "
            "set Float8LinearConfig.pad_inner_dim=True"
        )
    # with pad_inner_dim nothing is padded here: the GEMM takes any K (TMA zero-fills the tail) and
    # `scaled_mm` gives an operand whose row pitch TMA cannot take a pitch-aligned copy
    return a_data, a._scale, b_nk.t(), b._scale


def _mm_impl(a: Float8Tensor, b: Float8Tensor, bias):
    assert isinstance(a, Float8Tensor) and isinstance(
        b, Float8Tensor
    ), "Expecting  both Float8Tensor for mm inputs but found {} and {}".format(type(a), type(b))
    a_data, a_scale, b_data, b_scale = preprocess_addmm(a, b)
    cfg = choose_scaled_mm_config(a._gemm_input_role, a._linear_mm_config, b._gemm_input_role, b._linear_mm_config)
    return addmm_float8_unwrapped(
        a_data, a_scale, b_data, b_scale, a._orig_dtype, output_scale=None, bias=bias,
        use_fast_accum=cfg.use_fast_accum,
    )


@implements([aten.mm.default, aten.matmul.default])
def float8_mm(aten_op, args, kwargs=None):
    return _mm_impl(args[0], args[1], None)


@implements([aten.addmm.default])
def float8_addmm(aten_op, args, kwargs=None):
    bias, a, b = args[0], args[1], args[2]
    assert isinstance(bias, torch.Tensor) and isinstance(a, Float8Tensor) and isinstance(b, Float8Tensor)
    assert bias.dtype == a._orig_dtype, "bias dtype must match output dtype"
    return _mm_impl(a, b, bias)


@implements([aten.is_same_size.default])
def float8_is_same_size(aten_op, args, kwargs=None):
    return args[0].shape == args[1].shape


@implements([aten._to_copy.default])
def autocast_to_copy(aten_op, args, kwargs=None):
    """Under autocast a Float8Tensor is only re-tagged with the autocast dtype; the
    bytes stay (reference: float8_ops.py:235-255)."""
    src = args[0]
    assert isinstance(src, Float8Tensor)
    assert len(kwargs) == 1 and "dtype" in kwargs, "Only support dtype kwarg for autocast"
    assert kwargs["dtype"] in {
        torch.float16,
        torch.bfloat16,
    }, "Only support floating point conversion for autocast w/ Float8Tensor"
    return _like(src, src._data, src._alt, orig_dtype=kwargs["dtype"])


# ---------------------------------------------------------------------------
# functional collectives: move bytes, keep the scale on the side
# ---------------------------------------------------------------------------
@implements(
    [
        c10d_functional.all_gather_into_tensor.default,
        _c10d_functional.all_gather_into_tensor.default,
    ]
)
def allgather_fp8(aten_op, args, kwargs=None):
    """All-gather of the fp8 bytes, 1 byte per element on the wire.  The payload is
    viewed as uint8 so that every backend can carry it (reference: float8_ops.py:258-282)."""
    src = args[0]
    assert isinstance(src, Float8Tensor), f"expecting a Float8Tensor for allgather but found {type(src)}"
    payload = src._data.contiguous().view(torch.uint8)
    gathered = aten_op(payload, *args[1:], **(kwargs or {}))
    return _like(src, gathered.view(src._data.dtype))


@implements([c10d_functional.wait_tensor.default, _c10d_functional.wait_tensor.default])
def wait_tensor_fp8(aten_op, args, kwargs=None):
    src = args[0]
    assert isinstance(src, Float8Tensor)
    done = aten_op(src._data.view(torch.uint8), *args[1:], **(kwargs or {}))
    return _like(src, done.view(src._data.dtype))


if hasattr(_c10d_functional, "_wrap_tensor_autograd"):

    @implements([_c10d_functional._wrap_tensor_autograd.default])
    def wrap_tensor_autograd_fp8(aten_op, args, kwargs=None):
        """Newer DTensor redistribute passes the local tensor through this op to attach
        autograd to the pending collective; the fp8 payload needs no such wrapping
        beyond the usual async handle."""
        from torch.distributed._functional_collectives import AsyncCollectiveTensor

        return AsyncCollectiveTensor(args[0])


@implements([aten.index_put_.default])
def index_put_fp8(aten_op, args, kwargs=None):
    dst, values = args[0], args[2]
    assert isinstance(dst, Float8Tensor)
    assert isinstance(values, Float8Tensor)
    assert dst._scale == values._scale
    assert dst.dtype == values.dtype
    assert dst._orig_dtype == values._orig_dtype
    out = aten_op(dst._data, args[1], values._data, *args[3:], **(kwargs or {}))
    return _like(dst, out)


@implements([aten.copy_.default])
def copy_fp8(aten_op, args, kwargs=None):
    """copy_ into a high-precision tensor dequantises; between two Float8Tensors it
    needs identical metadata; anything else is rejected (reference: float8_ops.py:323-363)."""
    dst, src = args[0], args[1]
    kwargs = kwargs or {}
    if isinstance(src, Float8Tensor) and not isinstance(dst, Float8Tensor):
        return aten_op(dst, src.to_original_precision(), *args[2:], **kwargs)
    if isinstance(src, Float8Tensor) and isinstance(dst, Float8Tensor):
        assert dst._orig_dtype == src._orig_dtype, "Expecting both Float8Tensors to be of the same dtype"
        assert dst._scale == src._scale, "Expecting both Float8Tensors to have thee same scale"
        assert dst._linear_mm_config == src._linear_mm_config, "Expecting both Float8Tensors to have thee same mm config"
        assert dst._data.dtype == src._data.dtype, "Expecting both Float8Tensors to be of the same dtypet"
        assert dst._gemm_input_role == src._gemm_input_role, "Expecting both Float8Tensors to have the same gemm_input_role"
        return _like(dst, aten_op(dst._data, src._data, *args[2:], **kwargs))
    raise RuntimeError("Unsupported semantics for copy_ in Float8Tensor")
