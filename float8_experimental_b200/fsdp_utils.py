"""FSDP2 integration: weight wrappers whose `fsdp_pre_all_gather` casts the local
shard to e4m3 so the all-gather moves 1 byte per element, and the one-collective
precompute of all dynamic weight scales
(API of float8_experimental/fsdp_utils.py).

The all-gather payload is handed to FSDP as a uint8 view of the fp8 bytes so that any
process-group backend can carry it; `fsdp_post_all_gather` views it back.
"""
from __future__ import annotations

from typing import Any, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.utils._pytree as pytree
from torch._prims_common import suggest_memory_format

from . import _native as N
from ._ops import ops
from .float8_scaling_utils import (
    _maybe_initialize_amaxes_scales_for_float8_cast,
    hp_tensor_to_float8_delayed,
    hp_tensor_to_float8_dynamic,
)
from .float8_tensor import Float8Tensor, GemmInputRole, hp_tensor_and_scale_to_float8, LinearMMConfig
from .float8_utils import e4m3_dtype, EPS


@torch.no_grad()
def precompute_float8_dynamic_scale_for_fsdp(module: nn.Module, cast_now: bool = False) -> None:
    """Computes the dynamic scale of every FSDP-sharded float8 weight after an optimizer
    step with ONE multi-tensor amax launch over all local shards, ONE all-reduce (MAX)
    over the [n_weights] amax vector and ONE scale kernel
    (reference: fsdp_utils.py:29-72).  The scale arithmetic runs in the weights' dtype,
    as in the reference.

        model(input).sum().backward(); optim.step()
        precompute_float8_dynamic_scale_for_fsdp(model)

    `cast_now=True` (not in the reference) also casts every local shard right away, all of them
    in one multi-tensor launch (per 96 weights), and keeps the fp8 bytes on the weight wrappers:
    the all-gathers of the following forward AND backward then hand over those bytes without
    launching anything, where the reference casts each weight once per all-gather
    (fsdp_utils.py:168-185).  Same bytes and scales.  The cached bytes belong to the weights as
    they are at this call, exactly like the precomputed scales: call it after every optimizer
    step, before the next forward."""
    from torch.distributed._tensor import DTensor

    from .config import ScalingType
    from .float8_linear import Float8Linear

    linears = [m for m in module.modules() if isinstance(m, Float8Linear)]
    if any(m.scaling_type_weight is ScalingType.DELAYED for m in linears):
        # message kept from the reference (it means: dynamic weight scaling only)
        raise NotImplementedError("Only supports delayed scaling")
    targets: List[Float8Linear] = [
        m
        for m in linears
        if isinstance(m.weight, DTensor) and isinstance(m.weight._local_tensor, WeightWithDynamicFloat8CastTensor)
    ]
    if not targets:
        return
    shards = [m.weight._local_tensor._tensor for m in targets]
    w_dtype = shards[0].dtype
    amaxes = ops.multi_amax(shards)  # fp32 [n]; exact values of the weights' dtype
    mesh = targets[0].weight.device_mesh
    for dim in range(mesh.ndim):
        dist.all_reduce(amaxes, op=dist.ReduceOp.MAX, group=mesh.get_group(dim))
    code = N.hp_code(w_dtype)
    scales = ops.amax_to_scale(amaxes, N.E4M3, code, code)  # fp32 [n]
    if w_dtype != torch.float32:
        scales = scales.to(w_dtype)  # the reference's scale tensor has the weights' dtype
    fp8_shards = None
    if cast_now:
        # product rounded to the weights' dtype: the precomputed scale is a 0-dim tensor of that dtype
        fp8_shards = ops.multi_cast_with_scales(shards, scales.float(), N.E4M3, False)
    for i, m in enumerate(targets):
        w = m.weight._local_tensor
        w._precomputed_scale = scales[i]
        w._precomputed_fp8 = fp8_shards[i] if fp8_shards is not None else None
    N.poll_errors_if_enabled()


# FSDP pads, slices and copies its local shards; these ops must hand back the wrapper
# type so that the padded / moved shard still knows how to cast itself.
_ops_to_preserve_subclass = {
    torch.ops.aten.empty_like.default,
    torch.ops.aten.new_zeros.default,
    torch.ops.aten.slice.Tensor,
    torch.ops.aten.copy_.default,
    torch.ops.aten.view.default,
    torch.ops.aten.as_strided.default,
    torch.ops.aten._to_copy.default,
    torch.ops.aten._pin_memory.default,
}


def _make_outer(cls, tensor: torch.Tensor):
    return torch.Tensor._make_wrapper_subclass(
        cls,
        tensor.size(),
        strides=tensor.stride(),
        storage_offset=tensor.storage_offset(),
        memory_format=suggest_memory_format(tensor),
        dtype=tensor.dtype,
        layout=tensor.layout,
        device=tensor.device,
        pin_memory=tensor.is_pinned(),
        requires_grad=tensor.requires_grad,
    )


def _payload(fp8: Float8Tensor) -> Tuple[Tuple[torch.Tensor, ...], Tuple[torch.Tensor, ...]]:
    return (fp8._data.view(torch.uint8),), (fp8._scale,)


def _post_all_gather(self, all_gather_outputs, metadata, param_dtype, out):
    (raw,) = all_gather_outputs
    (scale,) = metadata
    if out is not None:
        assert isinstance(out, Float8Tensor), f"{type(out)}"
        out._scale = scale  # bytes were gathered in place into out._data's storage
        out._alt = None
        return
    data = raw.view(e4m3_dtype)
    return Float8Tensor(data, scale, param_dtype, self._linear_mm_config, gemm_input_role=GemmInputRole.WEIGHT), (raw,)


class WeightWithDynamicFloat8CastTensor(torch.Tensor):
    """High-precision weight shard that FSDP2 all-gathers as e4m3 bytes, dynamic
    scaling (reference: fsdp_utils.py:90-207).  `_precomputed_scale`, when set by
    `precompute_float8_dynamic_scale_for_fsdp`, saves the per-weight amax all-reduce."""

    @staticmethod
    def __new__(cls, tensor: torch.Tensor, linear_mm_config: LinearMMConfig,
                precomputed_scale: Optional[torch.Tensor] = None):
        return _make_outer(cls, tensor)

    def __init__(self, tensor: torch.Tensor, linear_mm_config: LinearMMConfig,
                 precomputed_scale: Optional[torch.Tensor] = None):
        self._tensor = tensor
        self._linear_mm_config = linear_mm_config
        self._precomputed_scale = precomputed_scale
        # fp8 bytes of `tensor` under `precomputed_scale`, set by precompute(cast_now=True); like the
        # scale it lives on this wrapper object only (every op that makes a new wrapper drops it)
        self._precomputed_fp8 = None

    @classmethod
    def __torch_dispatch__(cls, func, types, args, kwargs=None):
        if func == torch.ops.aten.detach.default:
            return cls(args[0]._tensor, args[0]._linear_mm_config)
        seen_cfg: List[LinearMMConfig] = []

        def unwrap(t):
            if seen_cfg:
                assert t._linear_mm_config == seen_cfg[0]
            else:
                seen_cfg.append(t._linear_mm_config)
            return t._tensor

        args, kwargs = pytree.tree_map_only(cls, unwrap, (args, kwargs or {}))
        out = func(*args, **kwargs)
        if func not in _ops_to_preserve_subclass:
            return out
        return pytree.tree_map_only(torch.Tensor, lambda x: cls(x, seen_cfg[0]), out)

    def __tensor_flatten__(self):
        if self._precomputed_scale is not None:
            return ["_tensor", "_precomputed_scale"], self._linear_mm_config
        return ["_tensor"], self._linear_mm_config

    @staticmethod
    def __tensor_unflatten__(inner_tensors, flatten_spec, outer_size, outer_stride):
        return WeightWithDynamicFloat8CastTensor(
            inner_tensors["_tensor"], flatten_spec, inner_tensors.get("_precomputed_scale", None)
        )

    def __repr__(self):
        return f"WeightWithDynamicFloat8CastTensor(tensor={self._tensor}, linear_mm_config={self._linear_mm_config})"

    @torch.no_grad()  # the transposed copy for backward GEMMs is pointless on a shard
    def fsdp_pre_all_gather(self, mesh):
        if self._precomputed_scale is not None and self._precomputed_fp8 is not None:
            return (self._precomputed_fp8.view(torch.uint8),), (self._precomputed_scale,)
        if self._precomputed_scale is not None:
            fp8 = hp_tensor_and_scale_to_float8(
                self._tensor, self._precomputed_scale, torch.float8_e4m3fn, self._linear_mm_config,
                GemmInputRole.WEIGHT,
            )
        else:
            fp8 = hp_tensor_to_float8_dynamic(
                self._tensor, e4m3_dtype, self._linear_mm_config, reduce_amax=True,
                gemm_input_role=GemmInputRole.WEIGHT,
            )
        return _payload(fp8)

    def fsdp_post_all_gather(self, all_gather_outputs: Tuple[torch.Tensor, ...], metadata: Any,
                             param_dtype: torch.dtype, *, out: Optional[torch.Tensor] = None):
        return _post_all_gather(self, all_gather_outputs, metadata, param_dtype, out)


class WeightWithDelayedFloat8CastTensor(torch.Tensor):
    """Same for delayed scaling: carries the owning layer's amax / history / scale
    buffers and updates them in `fsdp_pre_all_gather` (reference: fsdp_utils.py:210-388)."""

    @staticmethod
    def __new__(cls, tensor, amax_buffer, amax_history_buffer, scale_buffer, linear_mm_config, is_amax_initialized):
        return _make_outer(cls, tensor)

    def __init__(self, tensor, amax_buffer, amax_history_buffer, scale_buffer, linear_mm_config,
                 is_amax_initialized: bool):
        self._tensor = tensor
        self._amax_buffer = amax_buffer
        self._amax_history_buffer = amax_history_buffer
        self._scale_buffer = scale_buffer
        self._linear_mm_config = linear_mm_config
        self.is_amax_initialized = is_amax_initialized

    def _clone_with(self, tensor):
        return WeightWithDelayedFloat8CastTensor(
            tensor, self._amax_buffer, self._amax_history_buffer, self._scale_buffer, self._linear_mm_config,
            self.is_amax_initialized,
        )

    @classmethod
    def __torch_dispatch__(cls, func, types, args, kwargs=None):
        if func == torch.ops.aten.detach.default:
            return args[0]._clone_with(args[0]._tensor)
        first: List["WeightWithDelayedFloat8CastTensor"] = []

        def unwrap(t):
            if first:
                assert t._linear_mm_config == first[0]._linear_mm_config
            else:
                first.append(t)
            return t._tensor

        args, kwargs = pytree.tree_map_only(cls, unwrap, (args, kwargs or {}))
        out = func(*args, **kwargs)
        if func not in _ops_to_preserve_subclass:
            return out
        return pytree.tree_map_only(torch.Tensor, lambda x: first[0]._clone_with(x), out)

    def __tensor_flatten__(self):
        names = ["_tensor", "_amax_buffer", "_amax_history_buffer", "_scale_buffer"]
        return names, {"mm_config": self._linear_mm_config, "is_amax_initialized": self.is_amax_initialized}

    @staticmethod
    def __tensor_unflatten__(inner_tensors, metadata, outer_size, outer_stride):
        return WeightWithDelayedFloat8CastTensor(
            inner_tensors["_tensor"], inner_tensors["_amax_buffer"], inner_tensors["_amax_history_buffer"],
            inner_tensors["_scale_buffer"], metadata["mm_config"], metadata["is_amax_initialized"],
        )

    def __repr__(self):
        return (
            f"WeightWithDelayedFloat8CastTensor(tensor={self._tensor}, amax_buffer={self._amax_buffer}, "
            f"scale_buffer={self._scale_buffer}, mm_config={self._linear_mm_config})"
        )

    @torch.no_grad()
    def fsdp_pre_all_gather(self, mesh):
        if not self.is_amax_initialized:
            _maybe_initialize_amaxes_scales_for_float8_cast(
                self._tensor, self._amax_buffer, self._amax_history_buffer, self._scale_buffer, "max", e4m3_dtype,
                self.is_amax_initialized, reduce_amax=True,
            )
            self.is_amax_initialized = True
        fp8 = hp_tensor_to_float8_delayed(
            self._tensor, self._scale_buffer, e4m3_dtype, self._amax_buffer, self._linear_mm_config,
            GemmInputRole.WEIGHT,
        )
        return _payload(fp8)

    def fsdp_post_all_gather(self, all_gather_outputs: Tuple[torch.Tensor, ...], metadata: Any,
                             param_dtype: torch.dtype, *, out: Optional[torch.Tensor] = None):
        return _post_all_gather(self, all_gather_outputs, metadata, param_dtype, out)
