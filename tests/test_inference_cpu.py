"""Inference flows on CPU (oracle-backed stand-ins for the kernels): the three activation
casting modes, module swap, and save -> load -> quantize bit-equality
(the reference pins these in test/test_inference_flows.py:51-58,190-236)."""
import copy
import io

import pytest
import torch
import torch.nn as nn

import oracle_backend

oracle_backend.install()

from float8_experimental_b200.float8_tensor import Float8Tensor  # noqa: E402
from float8_experimental_b200.float8_utils import compute_error  # noqa: E402
from float8_experimental_b200.inference import (  # noqa: E402
    ActivationCasting,
    Float8InferenceLinear,
    QuantConfig,
    quantize_to_float8,
)


class FFN(nn.Module):
    def __init__(self):
        super().__init__()
        self.w1 = nn.Linear(64, 128, bias=True)
        self.w2 = nn.Linear(128, 64, bias=False)

    def forward(self, x):
        return self.w2(torch.relu(self.w1(x)))


class FeedForward(nn.Module):
    """The model of the reference's inference tests (test/test_inference_flows.py:35-49: w1, w3,
    w2 without bias around a SiLU gate, default nn.Linear init) at a quarter of its width."""

    def __init__(self, dim=256, hidden=896):
        super().__init__()
        self.w1 = nn.Linear(dim, hidden, bias=False)
        self.w3 = nn.Linear(dim, hidden, bias=False)
        self.w2 = nn.Linear(hidden, dim, bias=False)

    def forward(self, x):
        return self.w2(nn.functional.silu(self.w1(x)) * self.w3(x))


def configs():
    # the static scale of the reference's test (test/test_inference_flows.py:105-110)
    return [
        QuantConfig(ActivationCasting.WEIGHT_ONLY),
        QuantConfig(ActivationCasting.DYNAMIC),
        QuantConfig(ActivationCasting.STATIC, static_quantization_scale=torch.tensor([1.0])),
    ]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32], ids=["bf16", "fp32"])
@pytest.mark.parametrize("cfg", configs(), ids=["weight_only", "dynamic", "static"])
def test_modes_track_the_high_precision_model(cfg, dtype):
    """SQNR against the high-precision model above 20 dB, the reference's own bar
    (test/test_inference_flows.py:51-58), for the three activation-casting modes."""
    torch.manual_seed(0)
    ref = FeedForward().to(dtype)
    q = quantize_to_float8(copy.deepcopy(ref), cfg)
    assert isinstance(q.w1, Float8InferenceLinear) and isinstance(q.w1.weight, Float8Tensor)
    assert not q.w1.weight.requires_grad
    x = torch.randn(4, 64, 256, dtype=dtype)
    with torch.no_grad():
        y_ref, y = ref(x), q(x)
    assert y.shape == y_ref.shape and y.dtype == y_ref.dtype
    assert compute_error(y_ref, y) > 20.0


def test_bias_is_carried_through_the_quantised_linear():
    torch.manual_seed(0)
    ref = FFN()
    q = quantize_to_float8(copy.deepcopy(ref), QuantConfig(ActivationCasting.DYNAMIC))
    x = torch.randn(4, 16, 64)
    with torch.no_grad():
        assert compute_error(ref.w1(x), q.w1(x)) > 20.0


def test_static_config_needs_a_scale_and_double_quantize_is_rejected():
    with pytest.raises(AssertionError, match="activation_scale must be a tensor"):
        QuantConfig(ActivationCasting.STATIC)
    lin = Float8InferenceLinear.from_float(nn.Linear(32, 32), QuantConfig(ActivationCasting.DYNAMIC), True)
    with pytest.raises(AssertionError, match="already been quantized"):
        lin.quantize_weight()


def test_save_load_quantize_gives_the_same_bytes():
    torch.manual_seed(1)
    ref = FFN()
    q1 = quantize_to_float8(copy.deepcopy(ref), QuantConfig(ActivationCasting.DYNAMIC))
    buf = io.BytesIO()
    torch.save(ref.state_dict(), buf)
    buf.seek(0)
    fresh = FFN()
    fresh.load_state_dict(torch.load(buf, weights_only=True))
    q2 = quantize_to_float8(fresh, QuantConfig(ActivationCasting.DYNAMIC))
    for a, b in ((q1.w1, q2.w1), (q1.w2, q2.w2)):
        assert torch.equal(a.weight._data.view(torch.uint8), b.weight._data.view(torch.uint8))
        assert torch.equal(a.weight._scale, b.weight._scale)
    x = torch.randn(8, 64)
    with torch.no_grad():
        assert torch.equal(q1(x), q2(x))
