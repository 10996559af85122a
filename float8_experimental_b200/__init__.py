"""B200-native float8 training path with the public API of float8_experimental
(reference: float8_experimental/__init__.py:7-46)."""
from .config import CastConfig, DelayedScalingConfig, Float8GemmConfig, Float8LinearConfig, ScalingType
from .float8_linear import Float8Linear
from .float8_linear_utils import (
    convert_to_float8_training,
    linear_requires_sync,
    sync_float8_amax_and_scale_history,
)
from .float8_tensor import Float8Tensor, GemmInputRole, LinearMMConfig, ScaledMMConfig
from .fsdp_utils import precompute_float8_dynamic_scale_for_fsdp

from torch.serialization import add_safe_globals

# lets torch.load(weights_only=True) rebuild Float8Tensor state
add_safe_globals([Float8Tensor, ScaledMMConfig, GemmInputRole, LinearMMConfig])

__all__ = [
    "DelayedScalingConfig",
    "ScalingType",
    "Float8GemmConfig",
    "Float8LinearConfig",
    "CastConfig",
    "convert_to_float8_training",
    "linear_requires_sync",
    "sync_float8_amax_and_scale_history",
    "precompute_float8_dynamic_scale_for_fsdp",
]
