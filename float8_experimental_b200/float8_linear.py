"""`Float8Linear`: an `nn.Linear` whose three GEMMs run in float8 on the sm_100a
kernels.  Public surface, buffer names and guard messages follow
float8_experimental/float8_linear.py:43-438.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _native as N
from ._ops import ops
from .config import Float8LinearConfig, ScalingType
from .float8_scaling_utils import (
    _maybe_initialize_amaxes_scales_for_float8_cast,
    hp_tensor_to_float8_delayed,
    hp_tensor_to_float8_dynamic,
    NoopFwToFloat8E5M2BwDelayed,
    NoopFwToFloat8E5M2BwDynamic,
)
from .float8_tensor import Float8Tensor, GemmInputRole, LinearMMConfig, ScaledMMConfig
from .float8_utils import e4m3_dtype, e5m2_dtype, tensor_to_amax
from .fsdp_utils import WeightWithDelayedFloat8CastTensor, WeightWithDynamicFloat8CastTensor

_TENSORS = ("input", "weight", "grad_output")


@torch._dynamo.allow_in_graph
class manual_float8_matmul(torch.autograd.Function):
    """`input_fp8 @ weight_fp8_t` with both backward products also taken in float8
    (reference: float8_linear.py:43-95).  Each `torch.mm` below lands in the Float8Tensor
    operator table and from there in the tcgen05 GEMM."""

    @staticmethod
    def forward(ctx, input_fp8, weight_fp8_t):
        ctx.save_for_backward(input_fp8, weight_fp8_t)
        lead = input_fp8.shape[:-1]
        out = torch.mm(input_fp8.reshape(-1, input_fp8.shape[-1]), weight_fp8_t)
        return out.reshape(*lead, out.shape[-1])

    @staticmethod
    def backward(ctx, grad_output_fp8):
        input_fp8, weight_fp8_t = ctx.saved_tensors
        lead = grad_output_fp8.shape[:-1]
        go2d = grad_output_fp8.reshape(-1, grad_output_fp8.shape[-1])
        # dX = dY @ W
        grad_input = torch.mm(go2d, weight_fp8_t.t())
        grad_input = grad_input.reshape(*lead, grad_input.shape[-1])
        # dW = dY^T @ X  (returned as dW^T because the forward took W^T)
        x2d = input_fp8.reshape(-1, input_fp8.shape[-1])
        grad_weight = torch.mm(go2d.t(), x2d)
        return grad_input, grad_weight.t()


def _inner_dim_ok(k: int, mm_cfg: ScaledMMConfig) -> None:
    if k % 16 != 0 and not mm_cfg.pad_inner_dim:
        # same contract as the reference, whose cuBLASLt path needs K % 16 == 0 unless it pads
        raise RuntimeError(
            f"float8 GEMM needs the inner dimension to be a multiple of 16, got {k}; "
            "set Float8LinearConfig.pad_inner_dim=True"
        )


@torch._dynamo.allow_in_graph
class _float8_linear_dynamic(torch.autograd.Function):
    """Forward + backward of a Float8Linear whose three tensors use dynamic scaling, for plain CUDA
    tensors: the same kernels with the same arguments in the same order as the general route
    (amax, cast, GEMM for the output; amax, cast and two GEMMs for the gradients), launched from
    ONE autograd node on raw tensors.  The general route builds three `Float8Tensor`s, runs
    three extra autograd nodes and goes through `__torch_dispatch__` for every product; with
    hundreds of small layers per step that host work, not the GPU, sets the step time.  Results
    are bit-identical to the general route (`test_fast_path_matches_general_route`)."""

    @staticmethod
    def forward(ctx, x, weight, mm_cfg: LinearMMConfig):
        lead, k = x.shape[:-1], x.shape[-1]
        x2 = x.reshape(-1, k)
        _inner_dim_ok(k, mm_cfg.output)
        x8, sx = ops.cast_dynamic(x2, N.E4M3)  # amax + cast: two launches, one host call
        if isinstance(weight, Float8Tensor):  # FSDP2 delivered fp8 bytes and their scale
            w8, sw = weight._data, weight._scale
        else:
            w8, sw = ops.cast_dynamic(weight, N.E4M3)
        y = ops.scaled_mm(x8, w8, sx, sw, None, x.dtype, mm_cfg.output.use_fast_accum)
        ctx.save_for_backward(x8, sx, w8, sw)
        ctx.mm_cfg = mm_cfg
        return y.reshape(*lead, y.shape[-1])

    @staticmethod
    def backward(ctx, go):
        x8, sx, w8, sw = ctx.saved_tensors
        cfg = ctx.mm_cfg
        lead, n = go.shape[:-1], go.shape[-1]
        go2 = go.reshape(-1, n)
        g8, sg = ops.cast_dynamic(go2, N.E5M2)
        dx = dw = None
        if ctx.needs_input_grad[0]:  # dX = dY @ W: W [N, K] read as the transposed operand it is
            _inner_dim_ok(n, cfg.grad_input)
            dx = ops.scaled_mm(g8, w8.t(), sg, sw, None, go.dtype, cfg.grad_input.use_fast_accum)
            dx = dx.reshape(*lead, dx.shape[-1])
        if ctx.needs_input_grad[1]:  # dW = dY^T @ X: both operands read where they lie
            _inner_dim_ok(g8.shape[0], cfg.grad_weight)
            dw = ops.scaled_mm(g8.t(), x8.t(), sg, sx, None, go.dtype, cfg.grad_weight.use_fast_accum)
        return dx, dw, None


class Float8Linear(torch.nn.Linear):
    """Drop-in for `nn.Linear` (created through `from_float` / `convert_to_float8_training`).

    input and weight are cast to e4m3, the gradient of the output to e5m2, each with
    dynamic or delayed per-tensor scaling as configured."""

    def __init__(self, *args, **kwargs):
        """Takes `nn.Linear`'s arguments plus the keyword `config: Float8LinearConfig`."""
        self.always_float32_buffers = set()
        config = kwargs.pop("config")
        super().__init__(*args, **kwargs)
        self.config = config
        self.scaling_type_input = config.cast_config_input.scaling_type
        self.scaling_type_weight = config.cast_config_weight.scaling_type
        self.scaling_type_grad_output = config.cast_config_grad_output.scaling_type
        self.has_any_delayed_scaling = ScalingType.DELAYED in (
            self.scaling_type_input,
            self.scaling_type_weight,
            self.scaling_type_grad_output,
        )
        self.create_buffers()

        def mm_cfg(gemm_cfg):
            return ScaledMMConfig(config.emulate, gemm_cfg.use_fast_accum, False, config.pad_inner_dim)

        self.linear_mm_config = LinearMMConfig(
            mm_cfg(config.gemm_config_output),
            mm_cfg(config.gemm_config_grad_input),
            mm_cfg(config.gemm_config_grad_weight),
        )
        # plain attributes (not buffers): no data-dependent control flow on the device
        self.is_amax_initialized = not config.enable_amax_init
        self.amax_and_scale_synced = not config.enable_amax_init
        self.last_seen_input_dtype = None
        self.enable_pre_and_post_forward = config.enable_pre_and_post_forward
        # (GemmReduceScatter, output shard dimension), set by Float8RowwiseParallel(fused_reduce_scatter=...)
        self._rowwise_reduce_scatter = None

    # -- delayed-scaling state --------------------------------------------
    def create_buffers(self):
        """fp8_amax_* [1], fp8_amax_history_* [history_len], fp8_scale_* [1], fp32, for
        all three tensors as soon as one of them uses delayed scaling; initial amax is the
        format's maximum, initial scale 1 (reference: float8_linear.py:180-222)."""
        if not self.has_any_delayed_scaling:
            return
        hist_len = self.config.delayed_scaling_config.history_len
        dev = self.weight.device
        start_amax = {
            "input": torch.finfo(torch.float8_e4m3fn).max,
            "weight": torch.finfo(torch.float8_e4m3fn).max,
            "grad_output": torch.finfo(torch.float8_e5m2).max,
        }
        for name in _TENSORS:
            self.register_always_float32_buffer(f"fp8_amax_{name}", torch.tensor([start_amax[name]], device=dev))
            self.register_always_float32_buffer(f"fp8_amax_history_{name}", torch.zeros(hist_len, device=dev))
            self.register_always_float32_buffer(f"fp8_scale_{name}", torch.tensor([1.0], device=dev))

    def register_always_float32_buffer(self, name: str, tensor: Optional[torch.Tensor], persistent: bool = True) -> None:
        self.register_buffer(name=name, tensor=tensor, persistent=persistent)
        self.always_float32_buffers.add(name)

    def _apply(self, fn, recurse=True):
        ret = super()._apply(fn, recurse)
        self.convert_amax_buffer_to_float32()
        # buffers may have been replaced: the batched sync must re-pack its slabs
        self._f8_sync_slot = None
        return ret

    def convert_amax_buffer_to_float32(self):
        for key in self.always_float32_buffers:
            if self._buffers[key] is not None:
                self._buffers[key] = self._buffers[key].to(torch.float32)

    # -- casts ---------------------------------------------------------------
    def cast_input_to_float8(self, input: torch.Tensor, is_amax_initialized: bool) -> torch.Tensor:
        if torch.is_autocast_enabled():
            # same rule F.linear applies, so the output keeps the autocast dtype
            input = input.to(torch.get_autocast_dtype("cuda"))
        if self.scaling_type_input is ScalingType.DELAYED:
            _maybe_initialize_amaxes_scales_for_float8_cast(
                input, self.fp8_amax_input, self.fp8_amax_history_input, self.fp8_scale_input,
                self.config.delayed_scaling_config.scale_fn_name, e4m3_dtype, is_amax_initialized, reduce_amax=True,
            )
            return hp_tensor_to_float8_delayed(
                input, self.fp8_scale_input, e4m3_dtype, self.fp8_amax_input,
                linear_mm_config=self.linear_mm_config, gemm_input_role=GemmInputRole.INPUT,
            )
        assert self.scaling_type_input is ScalingType.DYNAMIC
        return hp_tensor_to_float8_dynamic(input, e4m3_dtype, self.linear_mm_config)

    def cast_weight_to_float8(self, weight: torch.Tensor, is_amax_initialized: bool) -> torch.Tensor:
        if isinstance(self.weight, Float8Tensor):
            return self.weight  # FSDP2 already delivered fp8 bytes
        if self.scaling_type_weight is ScalingType.DELAYED:
            _maybe_initialize_amaxes_scales_for_float8_cast(
                weight, self.fp8_amax_weight, self.fp8_amax_history_weight, self.fp8_scale_weight,
                self.config.delayed_scaling_config.scale_fn_name, e4m3_dtype, is_amax_initialized, reduce_amax=False,
            )
            return hp_tensor_to_float8_delayed(
                weight, self.fp8_scale_weight, e4m3_dtype, self.fp8_amax_weight,
                linear_mm_config=self.linear_mm_config, gemm_input_role=GemmInputRole.WEIGHT,
            )
        assert self.scaling_type_weight is ScalingType.DYNAMIC
        return hp_tensor_to_float8_dynamic(
            self.weight, e4m3_dtype, self.linear_mm_config, gemm_input_role=GemmInputRole.WEIGHT
        )

    def cast_output_to_float8_in_bw(self, output: torch.Tensor) -> torch.Tensor:
        if self.scaling_type_grad_output is ScalingType.DELAYED:
            return NoopFwToFloat8E5M2BwDelayed.apply(
                output, self.fp8_amax_grad_output, self.fp8_amax_history_grad_output, self.fp8_scale_grad_output,
                self.config.delayed_scaling_config.scale_fn_name, self.is_amax_initialized, self.linear_mm_config,
            )
        assert self.scaling_type_grad_output is ScalingType.DYNAMIC
        return NoopFwToFloat8E5M2BwDynamic.apply(output, self.linear_mm_config)

    # -- guards --------------------------------------------------------------
    def float8_pre_forward(self, input):
        if not self.enable_pre_and_post_forward:
            return
        if self.is_amax_initialized and not self.amax_and_scale_synced and torch.is_grad_enabled():
            raise AssertionError(
                "amaxes and scales not synced, please call `sync_float8_amax_and_scale_history` before forward"
            )
        self.last_seen_input_dtype = input.dtype

    def float8_post_forward(self):
        if not self.enable_pre_and_post_forward:
            return
        # the next training forward must be preceded by a sync
        self.is_amax_initialized = True
        self.amax_and_scale_synced = False

    def _single_node_route(self, input: torch.Tensor) -> bool:
        """Whether this call can take `_float8_linear_dynamic`: dynamic scaling throughout, a plain
        tensor as input (not a DTensor, not already float8), a plain or FSDP2-delivered float8 weight,
        no autocast, no transposed copies asked for.  F8B200_LINEAR_SINGLE_NODE=0 switches it off."""
        if self.has_any_delayed_scaling or self._rowwise_reduce_scatter is not None:
            return False
        if type(input) is not torch.Tensor or torch.is_autocast_enabled(input.device.type):
            return False
        w = self.weight
        if not (type(w) in (torch.nn.Parameter, torch.Tensor) or isinstance(w, Float8Tensor)):
            return False
        if isinstance(w, Float8Tensor) and (w._data.dim() != 2 or w._orig_dtype != input.dtype):
            return False
        if not isinstance(w, Float8Tensor) and w.dtype != input.dtype:
            return False
        import os

        return os.environ.get("F8B200_LINEAR_SINGLE_NODE", "1") != "0" and \
            os.environ.get("F8B200_CAST_TRANSPOSED", "0") != "1"

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        if self._single_node_route(input):
            output = _float8_linear_dynamic.apply(input, self.weight, self.linear_mm_config)
            if self.bias is not None:
                output = output + self.bias.to(output.dtype)
            return output
        if self.has_any_delayed_scaling:
            self.float8_pre_forward(input)
        input_fp8 = self.cast_input_to_float8(input, self.is_amax_initialized)
        weight_fp8 = self.cast_weight_to_float8(self.weight, self.is_amax_initialized)
        if self._rowwise_reduce_scatter is not None and type(input_fp8).__name__ == "DTensor":
            from .fused_reduce_scatter import rowwise_matmul_reduce_scatter

            output = rowwise_matmul_reduce_scatter(input_fp8, weight_fp8.t(), *self._rowwise_reduce_scatter)
        else:
            output = manual_float8_matmul.apply(input_fp8, weight_fp8.t())
        output = self.cast_output_to_float8_in_bw(output)
        if self.bias is not None:
            output = output + self.bias.to(output.dtype)
        if self.has_any_delayed_scaling:
            self.float8_post_forward()
        return output

    def scaling_repr(self):
        parts = zip(("i", "w", "go"), (self.scaling_type_input, self.scaling_type_weight, self.scaling_type_grad_output))
        return ",".join(f"{tag}:{st.short_str()}" for tag, st in parts)

    def extra_repr(self):
        return f'{super().extra_repr()}, scaling="{self.scaling_repr()}"'

    @classmethod
    def from_float(cls, mod, config: Optional[Float8LinearConfig] = None):
        """Builds a Float8Linear that shares `mod`'s weight and bias
        (reference: float8_linear.py:384-438)."""
        if config is None:
            config = Float8LinearConfig()
        with torch.device("meta"):
            new_mod = cls(mod.in_features, mod.out_features, bias=False, config=config)
        new_mod.weight = mod.weight
        new_mod.bias = mod.bias
        new_mod.create_buffers()  # again, now on the weight's real device
        if config.enable_fsdp_float8_all_gather:
            # last, because the delayed wrapper captures the buffers created above
            if config.cast_config_weight.scaling_type is ScalingType.DYNAMIC:
                wrapped = WeightWithDynamicFloat8CastTensor(new_mod.weight, new_mod.linear_mm_config)
            else:
                assert config.cast_config_weight.scaling_type is ScalingType.DELAYED
                wrapped = WeightWithDelayedFloat8CastTensor(
                    new_mod.weight, new_mod.fp8_amax_weight, new_mod.fp8_amax_history_weight,
                    new_mod.fp8_scale_weight, new_mod.linear_mm_config, new_mod.is_amax_initialized,
                )
            new_mod.weight = torch.nn.Parameter(wrapped)
        return new_mod
