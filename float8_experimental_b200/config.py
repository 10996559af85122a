"""Configuration objects of the float8 training path.

Field names, defaults and value strings match float8_experimental/config.py:12-129 so
that existing user code keeps working.  All objects are immutable and hashable.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field


class ScalingType(enum.Enum):
    """How the per-tensor scale of a cast is obtained (reference: config.py:12-21)."""

    DELAYED = "delayed"  # scale comes from a history of earlier amaxes
    DYNAMIC = "dynamic"  # scale comes from the amax of the tensor being cast

    def short_str(self) -> str:
        return {"delayed": "del", "dynamic": "dyn"}[self.value]


@dataclass(frozen=True)
class CastConfig:
    """Cast recipe of one of the three tensors of a linear layer (reference: config.py:24-30)."""

    scaling_type: ScalingType = ScalingType.DYNAMIC


@dataclass(frozen=True)
class DelayedScalingConfig:
    """Delayed-scaling recipe (reference: config.py:33-54).

    `history_len` amaxes are remembered per tensor; the scale is derived from their
    maximum ("max" is the only supported `scale_fn_name`).  One recipe is shared by
    every layer of a model."""

    history_len: int = 16
    scale_fn_name: str = "max"

    def __post_init__(self):
        if self.scale_fn_name != "max":
            raise AssertionError(
                f"{self.scale_fn_name} is not implemented yet. Only max is supported for now."
            )


@dataclass(frozen=True)
class Float8GemmConfig:
    """Options of one of the three GEMMs (reference: config.py:57-65).

    `use_fast_accum` is a Hopper cuBLASLt hint.  The sm_100a kernel always accumulates
    in fp32 tensor memory; the flag is carried for API compatibility and ignored."""

    use_fast_accum: bool = False


@dataclass(frozen=True)
class Float8LinearConfig:
    """Everything `convert_to_float8_training` needs (reference: config.py:68-123)."""

    # casts of input / weight / grad_output
    cast_config_input: CastConfig = CastConfig()
    cast_config_weight: CastConfig = CastConfig()
    cast_config_grad_output: CastConfig = CastConfig()

    # GEMMs producing output / grad_input / grad_weight
    gemm_config_output: Float8GemmConfig = Float8GemmConfig(use_fast_accum=True)
    gemm_config_grad_input: Float8GemmConfig = Float8GemmConfig()
    gemm_config_grad_weight: Float8GemmConfig = Float8GemmConfig()

    # delayed scaling: seed amax/history/scale from the first batch seen
    enable_amax_init: bool = True
    # delayed scaling: run the "did you sync?" guards around forward
    enable_pre_and_post_forward: bool = True
    # wrap weights so that FSDP2 all-gathers fp8 bytes instead of high precision
    enable_fsdp_float8_all_gather: bool = False
    # zero-pad the contraction dimension to a multiple of 16 before the GEMM
    pad_inner_dim: bool = False
    # Accepted for compatibility.  This package has no emulated (fp32, CPU-capable)
    # GEMM: every GEMM runs the sm_100a kernel whatever this flag says.
    emulate: bool = False

    delayed_scaling_config: DelayedScalingConfig = field(default_factory=DelayedScalingConfig)


# ROCm-only "fnuz" float8 flavours are not supported by the sm_100a kernels; the flag
# exists because reference code reads it (config.py:126-129).
use_fnuz_dtype = False
