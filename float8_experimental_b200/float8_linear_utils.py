"""Module conversion and the delayed-scaling sync step
(API of float8_experimental/float8_linear_utils.py).

`sync_float8_amax_and_scale_history` is where this implementation departs most from
the reference's mechanics: instead of ~9 small tensor ops per layer it keeps every
layer's amax / history / scale buffers as views into three contiguous slabs and
updates all rows with ONE kernel launch, preceded (when torch.distributed is
initialised) by ONE all-reduce over the amax slab.
"""
from __future__ import annotations

import logging
from typing import Callable, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from . import _native as N
from ._ops import ops
from .config import Float8LinearConfig, ScalingType
from .float8_linear import Float8Linear
from .float8_utils import amax_history_to_scale_stack, e4m3_dtype, e5m2_dtype

log = logging.getLogger(__name__)
log.addHandler(logging.NullHandler())

# The reference rolls a stacked COPY of the per-layer histories and never writes it
# back (float8_linear_utils.py:287-302), so the module buffers `fp8_amax_history_*`
# keep their initial contents and each new scale is computed from
# max(current amax, history[0..H-2]) with a static history.  False reproduces those
# scales exactly; True persists the rolled history (what the recipe intends).
WRITE_BACK_AMAX_HISTORY = False

_KINDS = ("input", "weight", "grad_output")


def linear_requires_sync(config: Float8LinearConfig) -> bool:
    """True when any of the three casts uses delayed scaling (reference: :26-34)."""
    casts = (config.cast_config_input, config.cast_config_weight, config.cast_config_grad_output)
    return any(c.scaling_type is ScalingType.DELAYED for c in casts)


def _update_history_stack(new_amax: torch.Tensor, amax_history_stack: torch.Tensor) -> None:
    """In place: shift every row right by one and put `new_amax` in column 0
    (reference: :37-56)."""
    assert amax_history_stack.dim() == 2, f"Expected amat_history_stack to be 2D, got {amax_history_stack.shape}"
    assert new_amax.size(0) == amax_history_stack.size(0), (
        "Expected new_amax to have the same size as the first dimension of amax_history_stack, "
        f"got {new_amax.size(0)} and {amax_history_stack.size(0)}"
    )
    rolled = torch.roll(amax_history_stack, 1, dims=1)
    rolled[:, 0] = new_amax.squeeze(-1)
    amax_history_stack.copy_(rolled)


def swap_linear_layers(
    module: nn.Module,
    from_float_func: Callable[[nn.Linear], nn.Linear],
    *,
    module_filter_fn: Optional[Callable[[nn.Module, str], bool]] = None,
) -> nn.Module:
    """Replaces every `nn.Linear` accepted by `module_filter_fn(module, fqn)` with
    `from_float_func(linear)`, children before parents.  A bare `nn.Linear` root is
    converted and returned (not modified in place); one with children is rejected
    (reference: :59-122)."""

    def wanted(m: nn.Module, fqn: str) -> bool:
        return isinstance(m, nn.Linear) and (module_filter_fn is None or module_filter_fn(m, fqn))

    if wanted(module, ""):
        if any(True for _ in module.children()):
            raise AssertionError(f"Does not support a root nn.Linear with children: {module}")
        return from_float_func(module)

    def visit(mod: nn.Module, fqn: str, parent: Optional[nn.Module]) -> None:
        for name, child in mod.named_children():
            visit(child, f"{fqn}.{name}" if fqn else name, mod)
        if wanted(mod, fqn):
            assert parent is not None, f"Linear root module should return early: {mod}"
            setattr(parent, fqn.rsplit(".", 1)[-1], from_float_func(mod))

    visit(module, "", None)
    return module


def convert_to_float8_training(
    module: nn.Module,
    *,
    module_filter_fn: Optional[Callable[[nn.Module, str], bool]] = None,
    config: Float8LinearConfig = None,
) -> nn.Module:
    """Swaps `nn.Linear` for `Float8Linear` throughout `module` (reference: :125-154)."""
    cfg = config if config is not None else Float8LinearConfig()
    return swap_linear_layers(
        module, lambda m: Float8Linear.from_float(m, config=cfg), module_filter_fn=module_filter_fn
    )


def get_float8_layers(model: torch.nn.Module) -> List[Float8Linear]:
    """All Float8Linear modules of `model`, in `modules()` order (reference: :157-169)."""
    return [m for m in model.modules() if isinstance(m, Float8Linear)]


class _SyncSlabs:
    """amax [3L], history [3L, H] and scale [3L] for L layers, rows ordered
    inputs | weights | grad_outputs; the layers' nine buffers are views into them."""

    def __init__(self, layers: List[Float8Linear]):
        n = len(layers)
        dev = layers[0].fp8_amax_input.device
        hist_len = layers[0].fp8_amax_history_input.numel()
        self.token = object()
        self.n_layers = n
        self.amax = torch.empty(3 * n, dtype=torch.float32, device=dev)
        self.hist = torch.empty(3 * n, hist_len, dtype=torch.float32, device=dev)
        self.scale = torch.empty(3 * n, dtype=torch.float32, device=dev)
        # gather the current values with three small cats each, then rebind the views
        for k, kind in enumerate(_KINDS):
            rows = slice(k * n, (k + 1) * n)
            self.amax[rows] = torch.cat([getattr(m, f"fp8_amax_{kind}").reshape(1) for m in layers])
            self.hist[rows] = torch.stack([getattr(m, f"fp8_amax_history_{kind}") for m in layers])
            self.scale[rows] = torch.cat([getattr(m, f"fp8_scale_{kind}").reshape(1) for m in layers])
        for i, m in enumerate(layers):
            for k, kind in enumerate(_KINDS):
                r = k * n + i
                m._buffers[f"fp8_amax_{kind}"] = self.amax[r : r + 1]
                m._buffers[f"fp8_amax_history_{kind}"] = self.hist[r]
                m._buffers[f"fp8_scale_{kind}"] = self.scale[r : r + 1]
            m._f8_sync_slot = (self.token, i)
            _rebind_fsdp_weight_buffers(m)

    def matches(self, layers: List[Float8Linear]) -> bool:
        if len(layers) != self.n_layers:
            return False
        tok = self.token
        return all(getattr(m, "_f8_sync_slot", None) == (tok, i) for i, m in enumerate(layers))


def _rebind_fsdp_weight_buffers(m: Float8Linear) -> None:
    from .fsdp_utils import WeightWithDelayedFloat8CastTensor

    w = m.weight
    inner = getattr(w, "_local_tensor", w)
    for t in (w, inner, getattr(inner, "data", None)):
        if isinstance(t, WeightWithDelayedFloat8CastTensor):
            t._amax_buffer = m.fp8_amax_weight
            t._amax_history_buffer = m.fp8_amax_history_weight
            t._scale_buffer = m.fp8_scale_weight


_SLABS_ATTR = "_f8_sync_slabs"


@torch.no_grad()
def sync_float8_amax_and_scale_history(model: torch.nn.Module, fp8_layers=None) -> None:
    """Delayed-scaling bookkeeping between iterations (reference: :172-327):
    1. cross-rank MAX of every current amax (one all-reduce over the amax slab),
    2. per (layer, tensor): scale = amax_to_scale(max(amax, history[0..H-2])) in fp32,
       e4m3 range for inputs and weights, e5m2 for grad_outputs, fp16 clamp keyed on
       the dtype of the last input seen -- one kernel launch for all rows,
    3. marks every layer as synced.
    Pass `fp8_layers=get_float8_layers(model)` to skip the module walk."""
    if fp8_layers is None:
        fp8_layers = get_float8_layers(model)
    if len(fp8_layers) == 0:
        log.warning("Calling sync_float8_amax_and_scale_history on a module with no Float8Linear layers")
        return

    anchor = fp8_layers[0]
    slabs: Optional[_SyncSlabs] = getattr(anchor, _SLABS_ATTR, None)
    tok = slabs.token if slabs is not None else None
    # one pass over the layers: recipe / dtype agreement and slab membership
    x_dtype = anchor.last_seen_input_dtype
    recipe = anchor.config.delayed_scaling_config.scale_fn_name
    uniform, packed = True, slabs is not None and slabs.n_layers == len(fp8_layers)
    for i, m in enumerate(fp8_layers):
        if m.last_seen_input_dtype is not x_dtype or m.config.delayed_scaling_config.scale_fn_name != recipe:
            uniform = False
        if packed and getattr(m, "_f8_sync_slot", None) != (tok, i):
            packed = False
    if not uniform:
        x_dtypes = {m.last_seen_input_dtype for m in fp8_layers}
        if len(x_dtypes) != 1:
            raise ValueError(f"All layers must have the same last seen input_dtype, got {x_dtypes}")
        recipes = {m.config.delayed_scaling_config.scale_fn_name for m in fp8_layers}
        raise ValueError(f"All layers must have the same scale_fn recipe, got {recipes}")
    # None (no forward seen yet) behaves like any non-fp16 dtype: no fp16 clamp of the scale
    orig_code = N.hp_code(x_dtype) if x_dtype is not None else N.FP32
    if not packed:
        slabs = _SyncSlabs(list(fp8_layers))
        object.__setattr__(anchor, _SLABS_ATTR, slabs)

    if dist.is_initialized():
        dist.all_reduce(slabs.amax, op=dist.ReduceOp.MAX)

    ops.delayed_sync(
        slabs.amax, slabs.hist, 2 * slabs.n_layers, orig_code, slabs.scale,
        slabs.hist if WRITE_BACK_AMAX_HISTORY else None,
    )
    for m in fp8_layers:
        m.amax_and_scale_synced = True
    N.poll_errors_if_enabled()
