"""Host logic of the fused RMSNorm -> fp8 cast (autograd wiring, composition with
Float8Linear), on the CPU stand-ins; and the oracle's restatement of the fused arithmetic
against the unfused composition the reference's benchmark model performs."""
import pytest
import torch

import oracle_backend

oracle_backend.install()

import float8_experimental_b200 as f8  # noqa: E402
from float8_experimental_b200.float8_linear import Float8Linear  # noqa: E402
from float8_experimental_b200.float8_scaling_utils import hp_tensor_to_float8_dynamic  # noqa: E402
from float8_experimental_b200.float8_tensor import Float8Tensor, LinearMMConfig  # noqa: E402
from float8_experimental_b200.fused_norm import (  # noqa: E402
    Float8RMSNorm,
    rms_norm_to_float8_dynamic,
    swiglu_to_float8_dynamic,
)
from oracle import f8_oracle as O  # noqa: E402


def reference_rmsnorm(x, weight, eps):
    """RMSNorm.forward of float8_experimental/benchmarks/profile_linear_float8.py:69-74."""
    xf = x.float()
    n = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return n.type_as(x) * weight


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(8, 4096), (33, 520), (5, 7), (3, 4, 256)])
def test_oracle_fused_norm_equals_unfused_composition(dtype, shape):
    torch.manual_seed(shape[-1])
    x = (torch.randn(shape) * 2.5).to(dtype)
    w = (1 + 0.2 * torch.randn(shape[-1])).to(dtype)
    fused = rms_norm_to_float8_dynamic(x, w, 1e-6)
    unfused = hp_tensor_to_float8_dynamic(reference_rmsnorm(x, w, 1e-6), torch.float8_e4m3fn, LinearMMConfig())
    assert isinstance(fused, Float8Tensor) and fused.shape == x.shape and fused.dtype == dtype
    a, b = fused._data.view(torch.uint8), unfused._data.view(torch.uint8)
    # the only freedom is the last bit of 1/rms (summation order of the mean, rsqrt vs 1/sqrt):
    # it moves few values across a rounding boundary, each by one fp8 step
    assert (a != b).float().mean().item() <= 2e-3
    assert (a.int() - b.int()).abs().max().item() <= 1
    assert abs(fused._scale.item() / unfused._scale.item() - 1) <= 2 ** -7


def test_fused_norm_feeds_float8_linear_and_backward_matches_autograd():
    torch.manual_seed(1)
    dim, out = 256, 128
    lin = torch.nn.Linear(dim, out, bias=False, dtype=torch.bfloat16)
    m = Float8Linear.from_float(lin, f8.Float8LinearConfig())
    norm = Float8RMSNorm(dim, 1e-6, m.linear_mm_config, dtype=torch.bfloat16)
    with torch.no_grad():
        norm.weight.copy_((1 + 0.1 * torch.randn(dim)).to(torch.bfloat16))
    x = torch.randn(32, dim).to(torch.bfloat16).requires_grad_(True)
    go = (torch.randn(32, out) * 0.01).to(torch.bfloat16)
    y = m(norm(x))
    y.backward(go)
    # unfused: the reference's RMSNorm in eager mode, then the same Float8Linear
    x2 = x.detach().clone().requires_grad_(True)
    w2 = norm.weight.detach().clone().requires_grad_(True)
    m.weight.grad = None
    y2 = m(reference_rmsnorm(x2, w2, 1e-6))
    y2.backward(go)
    assert O.sqnr_db(y2.detach().float().numpy(), y.detach().float().numpy()) > 40
    assert O.sqnr_db(x2.grad.float().numpy(), x.grad.float().numpy()) > 35
    assert O.sqnr_db(w2.grad.float().numpy(), norm.weight.grad.float().numpy()) > 35


def test_fused_norm_rejects_mismatched_weight_dtype_and_empty_input():
    x = torch.randn(4, 64).to(torch.bfloat16)
    with pytest.raises(RuntimeError):
        rms_norm_to_float8_dynamic(x, torch.ones(64), 1e-6)
    with pytest.raises(RuntimeError):
        rms_norm_to_float8_dynamic(x[:0], torch.ones(64, dtype=torch.bfloat16), 1e-6)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_oracle_fused_swiglu_equals_unfused_composition(dtype):
    torch.manual_seed(9)
    h = torch.randn(24, 2 * 264).mul(3).to(dtype)
    a, b = h[:, :264], h[:, 264:]  # the two halves of one fused w1|w3 output
    fused = swiglu_to_float8_dynamic(a, b)
    unfused = hp_tensor_to_float8_dynamic(torch.nn.functional.silu(a) * b, torch.float8_e4m3fn, LinearMMConfig())
    x, y = fused._data.view(torch.uint8), unfused._data.view(torch.uint8)
    assert fused.shape == a.shape and fused.dtype == dtype
    assert (x != y).float().mean().item() <= 2e-3 and (x.int() - y.int()).abs().max().item() <= 1
    assert abs(fused._scale.item() / unfused._scale.item() - 1) <= 2 ** -7


def test_fused_swiglu_backward_matches_autograd():
    torch.manual_seed(4)
    a = torch.randn(16, 128).to(torch.bfloat16).requires_grad_(True)
    b = torch.randn(16, 128).to(torch.bfloat16).requires_grad_(True)
    lin = torch.nn.Linear(128, 64, bias=False, dtype=torch.bfloat16)
    m = Float8Linear.from_float(lin, f8.Float8LinearConfig())
    go = (torch.randn(16, 64) * 0.01).to(torch.bfloat16)
    m(swiglu_to_float8_dynamic(a, b, linear_mm_config=m.linear_mm_config)).backward(go)
    a2, b2 = a.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    m(torch.nn.functional.silu(a2) * b2).backward(go)
    assert O.sqnr_db(a2.grad.float().numpy(), a.grad.float().numpy()) > 35
    assert O.sqnr_db(b2.grad.float().numpy(), b.grad.float().numpy()) > 35
