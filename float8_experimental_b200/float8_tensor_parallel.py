"""DTensor tensor/sequence-parallel styles that cast to float8 BEFORE redistributing,
so sequence-sharded activations cross NVLink as 1 byte per element
(API of float8_experimental/float8_tensor_parallel.py).

Only dynamic scaling of input and grad_output is supported, as in the reference.
"""
from __future__ import annotations

import torch
import torch.nn as nn
from torch.distributed._tensor import DTensor
from torch.distributed.device_mesh import DeviceMesh
from torch.distributed.tensor.parallel import ColwiseParallel, PrepareModuleInput, RowwiseParallel

from .config import ScalingType
from .float8_scaling_utils import hp_tensor_to_float8_dynamic, NoopFwToFloat8E5M2BwDynamic
from .float8_tensor import GemmInputRole
from .float8_utils import e4m3_dtype


def _float8_linear_supports_float8_allgather(m) -> bool:
    return m.scaling_type_input == ScalingType.DYNAMIC and m.scaling_type_grad_output == ScalingType.DYNAMIC


def _check_module(module: nn.Module) -> None:
    from .float8_linear import Float8Linear

    if not isinstance(module, Float8Linear):
        raise ValueError(f"Expecting module to be Float8Linear but found {type(module)}")
    if not _float8_linear_supports_float8_allgather(module):
        raise AssertionError("unsupported")


def _cast_then_redistribute(input_layouts, desired_input_layouts, mod, inputs, device_mesh):
    """Annotate the local activation as a DTensor, cast it to e4m3 (the local amax is
    all-reduced over the mesh inside the cast), then redistribute the fp8 bytes."""
    x = inputs[0]
    if not isinstance(x, DTensor):
        x = DTensor.from_local(x, device_mesh, input_layouts, run_check=False)
    x = hp_tensor_to_float8_dynamic(x, e4m3_dtype, mod.linear_mm_config, gemm_input_role=GemmInputRole.INPUT)
    if input_layouts != desired_input_layouts:
        x = x.redistribute(placements=desired_input_layouts, async_op=True)
    return x


def _redistribute_then_mark_for_bw_cast(output_layouts, use_local_output, mod, outputs, device_mesh):
    if outputs.placements != output_layouts:
        outputs = outputs.redistribute(placements=output_layouts, async_op=True)
    # identity now; casts the incoming gradient (a DTensor) to e5m2 in backward
    outputs = NoopFwToFloat8E5M2BwDynamic.apply(outputs, mod.linear_mm_config)
    return outputs.to_local() if use_local_output else outputs


class Float8ColwiseParallel(ColwiseParallel):
    """Column-parallel Float8Linear (reference: float8_tensor_parallel.py:37-89)."""

    @staticmethod
    def _prepare_input_fn(input_layouts, desired_input_layouts, mod, inputs, device_mesh):
        return _cast_then_redistribute(input_layouts, desired_input_layouts, mod, inputs, device_mesh)

    @staticmethod
    def _prepare_output_fn(output_layouts, use_local_output, mod, outputs, device_mesh):
        return _redistribute_then_mark_for_bw_cast(output_layouts, use_local_output, mod, outputs, device_mesh)

    def _apply(self, module: nn.Module, device_mesh: DeviceMesh) -> nn.Module:
        _check_module(module)
        return super()._apply(module, device_mesh)


class Float8RowwiseParallel(RowwiseParallel):
    """Row-parallel Float8Linear; the partial outputs are reduced in high precision
    (reference: float8_tensor_parallel.py:92-142).

    `fused_reduce_scatter` (not in the reference): a `fused_reduce_scatter.GemmReduceScatter` over
    the mesh's process group.  With a sharded `output_layouts` the forward GEMM then stores its
    partial product straight into the owners' receive buffers (peer memory) and the bf16
    reduce-scatter of the reference disappears into the GEMM; the backward is unchanged."""

    def __init__(self, *, input_layouts=None, output_layouts=None, use_local_output=True, fused_reduce_scatter=None):
        super().__init__(input_layouts=input_layouts, output_layouts=output_layouts, use_local_output=use_local_output)
        self.fused_reduce_scatter = fused_reduce_scatter

    @staticmethod
    def _prepare_input_fn(input_layouts, desired_input_layouts, mod, inputs, device_mesh):
        return _cast_then_redistribute(input_layouts, desired_input_layouts, mod, inputs, device_mesh)

    @staticmethod
    def _prepare_output_fn(output_layouts, use_local_output, mod, outputs, device_mesh):
        return _redistribute_then_mark_for_bw_cast(output_layouts, use_local_output, mod, outputs, device_mesh)

    def _apply(self, module: nn.Module, device_mesh: DeviceMesh) -> nn.Module:
        _check_module(module)
        if self.fused_reduce_scatter is not None:
            (layout,) = self.output_layouts
            if device_mesh.ndim != 1 or not layout.is_shard():
                raise ValueError("fused_reduce_scatter needs a 1-D mesh and a sharded output layout")
            module._rowwise_reduce_scatter = (self.fused_reduce_scatter, layout.dim)
        return super()._apply(module, device_mesh)


class _CastAllGatherInput(torch.autograd.Function):
    """Sequence-parallel input -> replicated float8 DTensor through `CastAllGatherPool`: the cast
    kernel's stores are the all-gather (peer memory), in place of cast + redistribute
    (float8_experimental/float8_tensor_parallel.py:202-209).  Backward is the backward of that
    redistribute: the gradient (partial sums of the column-parallel consumers) is reduce-scattered
    back onto the input's sharding."""

    @staticmethod
    def forward(ctx, dt: DTensor, pool, linear_mm_config, shard_dim: int):
        from torch.distributed._tensor import Replicate

        ctx.placements = dt.placements
        y8 = pool.gather_dim(dt.to_local(), shard_dim, linear_mm_config=linear_mm_config,
                             gemm_input_role=GemmInputRole.INPUT)
        return DTensor.from_local(y8, dt.device_mesh, (Replicate(),), run_check=False)

    @staticmethod
    def backward(ctx, grad):
        return grad.redistribute(placements=ctx.placements), None, None, None


class PrepareFloat8ModuleInput(PrepareModuleInput):
    """`PrepareModuleInput` that casts the (sequence-sharded) input to e4m3 before the
    all-gather, so several float8 consumers share one 1-byte-per-element gather
    (reference: float8_tensor_parallel.py:145-235).

    Extra keywords: `float8_dtype` (only e4m3fn) and `fwd_config_submodule_fqn`, the
    submodule whose `linear_mm_config` tags the cast; when omitted every Float8Linear
    below the module must share one config.  `cast_all_gather` (not in the reference): a
    `fp8_all_gather.CastAllGatherPool` over the mesh's process group; a sharded -> replicated
    input then goes through the cast whose stores are the all-gather (peer memory over NVLink)
    instead of cast + NCCL all-gather.  Same bytes and scale; the pool's `depth` bounds how many
    gathered inputs may be alive at once."""

    def __init__(self, *, input_layouts=None, desired_input_layouts=None, input_kwarg_layouts=None,
                 desired_input_kwarg_layouts=None, use_local_output=False, float8_dtype=torch.float8_e4m3fn,
                 fwd_config_submodule_fqn=None, cast_all_gather=None):
        super().__init__(
            input_layouts=input_layouts,
            desired_input_layouts=desired_input_layouts,
            input_kwarg_layouts=input_kwarg_layouts,
            desired_input_kwarg_layouts=desired_input_kwarg_layouts,
            use_local_output=use_local_output,
        )
        if float8_dtype != torch.float8_e4m3fn:
            raise NotImplementedError("PrepareFloat8ModuleInput only support casting to float8_e4m3fn for now")
        self.float8_dtype = float8_dtype
        self.linear_mm_config = None
        self.fwd_config_submodule_fqn = fwd_config_submodule_fqn
        self.cast_all_gather = cast_all_gather

    def _prepare_input_arg(self, input, mesh, input_layout, desired_layout):
        if input_layout is None:
            return input
        if isinstance(input, DTensor):
            dt = input
        else:
            assert isinstance(input, torch.Tensor), "expecting input to be a torch.Tensor!"
            dt = DTensor.from_local(input, mesh, (input_layout,), run_check=False)
        if (self.cast_all_gather is not None and mesh.ndim == 1 and desired_layout is not None
                and desired_layout.is_replicate() and input_layout.is_shard() and dt.is_cuda
                and input_layout.dim < dt.dim() - 1):
            dt = _CastAllGatherInput.apply(dt, self.cast_all_gather, self.linear_mm_config, input_layout.dim)
            return dt.to_local() if self.use_local_output else dt
        dt = hp_tensor_to_float8_dynamic(dt, e4m3_dtype, self.linear_mm_config, gemm_input_role=GemmInputRole.INPUT)
        if desired_layout is not None and input_layout != desired_layout:
            dt = dt.redistribute(placements=(desired_layout,))
        return dt.to_local() if self.use_local_output else dt

    def _apply(self, module: nn.Module, device_mesh: DeviceMesh) -> nn.Module:
        from .float8_linear import Float8Linear

        if self.fwd_config_submodule_fqn is not None:
            fwd_linear = module.get_submodule(self.fwd_config_submodule_fqn)
            assert isinstance(fwd_linear, Float8Linear)
            self.linear_mm_config = fwd_linear.linear_mm_config
        else:
            for mod in module.modules():
                if not isinstance(mod, Float8Linear):
                    continue
                if self.linear_mm_config is None:
                    self.linear_mm_config = mod.linear_mm_config
                else:
                    assert (
                        self.linear_mm_config == mod.linear_mm_config
                    ), "All the Float8Linear modules should have same linear_mm_config!"
        assert self.linear_mm_config is not None
        super()._apply(module, device_mesh)
        return module
