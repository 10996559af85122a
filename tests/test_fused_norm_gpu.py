"""The fused RMSNorm -> fp8 cast kernels against the oracle (bit-exact: 1/rms, amax, scale and
every fp8 byte) and, at full size, against the unfused composition on the GPU."""
import numpy as np
import pytest
import torch

from float8_experimental_b200._ops import ops
from float8_experimental_b200.float8_scaling_utils import hp_tensor_to_float8_dynamic
from float8_experimental_b200.float8_tensor import LinearMMConfig
from float8_experimental_b200.fused_norm import rms_norm_to_float8_dynamic, swiglu_to_float8_dynamic
from oracle import f8_oracle as O

pytestmark = pytest.mark.gpu

_HP = {torch.bfloat16: O.BF16, torch.float16: O.FP16, torch.float32: O.FP32}


def host_bits(t):
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.float32:
        return t.numpy()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.view(torch.uint8).numpy()


def reference_rmsnorm(x, weight, eps):
    xf = x.float()
    n = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return n.type_as(x) * weight


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(64, 8192), (7, 4096), (33, 520), (5, 7), (3, 4, 264), (300, 2048 + 8), (2, 16384 + 24)])
@pytest.mark.parametrize("fp8", [torch.float8_e4m3fn, torch.float8_e5m2])
def test_fused_norm_kernels_match_oracle_bit_for_bit(dtype, shape, fp8):
    g = torch.Generator().manual_seed(shape[-1] * 3 + shape[0])
    x = (torch.randn(shape, generator=g) * 3).to(dtype)
    x.view(-1)[::97] *= 40  # outliers: the amax sits on few elements
    w = (1 + 0.2 * torch.randn(shape[-1], generator=g)).to(dtype)
    name, kind = _HP[dtype], (O.E4M3 if fp8 == torch.float8_e4m3fn else O.E5M2)
    bits, scale, amax, rstd = O.rmsnorm_cast_dynamic(host_bits(x).reshape(-1, shape[-1]), name, host_bits(w), 1e-6, kind)
    xc, wc = x.cuda(), w.cuda()
    rstd_g, amax_g = ops.rmsnorm_amax(xc, wc, 1e-6)
    assert np.array_equal(rstd_g.cpu().numpy().view(np.uint32), rstd.view(np.uint32))
    assert amax_g.item() == float(amax)
    out = rms_norm_to_float8_dynamic(xc, wc, 1e-6, fp8)
    assert out._scale.item() == float(scale)
    assert out._data.shape == x.shape
    assert np.array_equal(host_bits(out._data).reshape(-1), bits.reshape(-1))


def test_fused_norm_strided_rows_and_nan():
    base = torch.randn(40, 1024 + 64, device="cuda").to(torch.bfloat16)
    x = base[:, :1024]  # row pitch 1088 elements
    w = torch.ones(1024, device="cuda", dtype=torch.bfloat16)
    a = rms_norm_to_float8_dynamic(x, w, 1e-6)
    b = rms_norm_to_float8_dynamic(x.contiguous(), w, 1e-6)
    assert torch.equal(a._data.view(torch.uint8), b._data.view(torch.uint8)) and a._scale.item() == b._scale.item()
    x2 = x.contiguous().clone()
    x2[3, 5] = float("nan")
    c = rms_norm_to_float8_dynamic(x2, w, 1e-6)
    assert torch.isnan(c._scale).item()  # NaN amax -> NaN scale, as in the unfused path
    assert (c._data.view(torch.uint8)[3] & 0x7F == 0x7F).all().item()


def test_fused_norm_full_size_against_unfused_composition():
    """16384 x 8192 bf16 (the activation of the LLaMa-2-70B shapes): the oracle is too slow, so
    compare with RMSNorm in eager mode followed by the unfused dynamic cast.  The two differ only
    through the last bit of 1/rms."""
    torch.manual_seed(11)
    x = torch.randn(16384, 8192, device="cuda", dtype=torch.bfloat16) * 1.7
    w = (1 + 0.1 * torch.randn(8192, device="cuda")).to(torch.bfloat16)
    fused = rms_norm_to_float8_dynamic(x, w, 1e-6)
    unfused = hp_tensor_to_float8_dynamic(reference_rmsnorm(x, w, 1e-6), torch.float8_e4m3fn, LinearMMConfig())
    a, b = fused._data.view(torch.uint8), unfused._data.view(torch.uint8)
    assert fused._scale.item() == unfused._scale.item()
    assert (a != b).float().mean().item() <= 1e-3
    assert (a.int() - b.int()).abs().max().item() <= 1
    # idempotence of the cast half: casting the dequantised result with the same scale returns the bytes
    again = hp_tensor_to_float8_dynamic(fused.to_original_precision(), torch.float8_e4m3fn, LinearMMConfig())
    assert again._scale.item() == fused._scale.item()


def _close_fp8(a, b, frac):
    a, b = a.view(torch.uint8), b.view(torch.uint8)
    assert (a != b).float().mean().item() <= frac
    assert (a.int() - b.int()).abs().max().item() <= 1


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(64, 4096), (33, 520), (5, 7), (3, 4, 264)])
@pytest.mark.parametrize("fp8", [torch.float8_e4m3fn, torch.float8_e5m2])
def test_fused_swiglu_kernels_match_oracle(dtype, shape, fp8):
    """exp comes from two math libraries (device expf, numpy), so a last-bit difference of
    silu(a) may move an element across a rounding boundary: at most one fp8 step, on a
    vanishing fraction of elements; amax and scale agree to a bf16 ulp."""
    g = torch.Generator().manual_seed(shape[-1] + shape[0])
    a = (torch.randn(shape, generator=g) * 3).to(dtype)
    b = (torch.randn(shape, generator=g) * 2).to(dtype)
    name, kind = _HP[dtype], (O.E4M3 if fp8 == torch.float8_e4m3fn else O.E5M2)
    bits, scale, amax = O.swiglu_cast_dynamic(host_bits(a), host_bits(b), name, kind)
    out = swiglu_to_float8_dynamic(a.cuda(), b.cuda(), fp8)
    assert abs(out._scale.item() / float(scale) - 1) <= 2 ** -7
    if out._scale.item() == float(scale):
        _close_fp8(out._data.cpu(), torch.from_numpy(bits.reshape(shape)), 2e-3)
    # evaluating the gate in both launches instead of writing it once gives the same bytes
    again = swiglu_to_float8_dynamic(a.cuda(), b.cuda(), fp8, recompute=True)
    assert again._scale.item() == out._scale.item()
    assert torch.equal(again._data.view(torch.uint8), out._data.view(torch.uint8))


def test_fused_swiglu_full_size_against_unfused_composition_on_gpu():
    """The w2 input of the LLaMa-2-70B FFN: a, b = halves of the [16384, 57344] w1|w3 output.
    Same math library on both sides, so the bytes agree."""
    torch.manual_seed(12)
    h = torch.randn(16384, 57344, device="cuda", dtype=torch.bfloat16) * 2
    a, b = h[:, :28672], h[:, 28672:]
    ref = hp_tensor_to_float8_dynamic(torch.nn.functional.silu(a) * b, torch.float8_e4m3fn, LinearMMConfig())
    for recompute in (False, True):
        fused = swiglu_to_float8_dynamic(a, b, recompute=recompute)
        assert fused._scale.item() == ref._scale.item()
        _close_fp8(fused._data, ref._data, 1e-4)


def _fp8_code_steps(x, y):
    """Distance in fp8 codes along the real line (sign-magnitude bytes made monotonic)."""
    def key(t):
        u = t.view(torch.uint8).to(torch.int16)
        return torch.where(u >= 128, 127 - u, u)  # -0 -> -1, negative codes descend
    return (key(x) - key(y)).abs()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(2048, 4096), (3, 40, 264), (512, 28672)])
def test_fused_swiglu_approximate_gate_is_within_one_step_of_the_exact_one(dtype, shape):
    """`approx_gate=True`: sigmoid from the approximate exp2 and reciprocal.  The stated bound: the amax (and
    with it the scale) within one ulp of the input dtype of the exact path's, every fp8 byte within one
    fp8 step, gradients within one ulp of the input dtype.  Most bytes are identical."""
    torch.manual_seed(shape[-1] + 7)
    h = (torch.randn(*shape[:-1], 2 * shape[-1], device="cuda") * 3).to(dtype)
    a = h[..., : shape[-1]].detach().requires_grad_(True)
    b = h[..., shape[-1]:].detach().requires_grad_(True)
    a2, b2 = a.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    g = torch.randn(shape, device="cuda").to(dtype)
    exact = swiglu_to_float8_dynamic(a, b)
    fast = swiglu_to_float8_dynamic(a2, b2, approx_gate=True)
    ulp = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
    rel = abs(fast._scale.item() / exact._scale.item() - 1.0)
    assert rel <= 2.0 * ulp, rel
    steps = _fp8_code_steps(fast._data, exact._data)
    assert steps.max().item() <= 1
    if fast._scale.item() == exact._scale.item():
        assert (steps != 0).float().mean().item() <= 2e-3
    exact.backward(g)
    fast.backward(g)
    for got, ref in ((a2.grad, a.grad), (b2.grad, b.grad)):
        assert got.dtype == dtype
        err = (got.float() - ref.float()).abs()
        assert bool((err <= 2.0 * ulp * ref.float().abs() + 1e-5).all())  # (1 + a (1 - sig)) cancels near a = -1.28
        assert (got != ref).float().mean().item() <= 2e-3


def test_fused_swiglu_approximate_gate_refuses_what_it_does_not_cover():
    a = torch.randn(8, 40, device="cuda", dtype=torch.float32)
    with pytest.raises(RuntimeError):
        swiglu_to_float8_dynamic(a, a, approx_gate=True)          # fp32
    h = torch.randn(8, 36, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        swiglu_to_float8_dynamic(h, h, approx_gate=True)          # columns not a multiple of 8
    c = torch.randn(8, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        swiglu_to_float8_dynamic(c, c, approx_gate=True, recompute=True)


def _sqnr(ref, got):
    ref, got = ref.double(), got.double()
    return 20 * torch.log10(ref.norm() / (ref - got).norm()).item()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(512, 8192), (3, 40, 4096), (77, 264), (16, 2048)])
def test_fused_norm_backward_kernel_matches_eager_autograd(dtype, shape):
    torch.manual_seed(shape[-1])
    x = (torch.randn(shape, device="cuda") * 2).to(dtype).requires_grad_(True)
    w = (1 + 0.2 * torch.randn(shape[-1], device="cuda")).to(dtype).requires_grad_(True)
    g = torch.randn(shape, device="cuda").to(dtype)
    y8 = rms_norm_to_float8_dynamic(x, w, 1e-6)
    y8.backward(g)  # the cast passes the gradient through; RMSNorm backward runs in the CUDA kernel
    x2, w2 = x.detach().clone().requires_grad_(True), w.detach().clone().requires_grad_(True)
    reference_rmsnorm(x2, w2, 1e-6).backward(g)
    assert x.grad.dtype == dtype and w.grad.dtype == dtype and x.grad.shape == x.shape
    assert _sqnr(x2.grad, x.grad) > (45 if dtype == torch.bfloat16 else 60)
    assert _sqnr(w2.grad, w.grad) > (40 if dtype == torch.bfloat16 else 55)


@pytest.mark.parametrize("dtype,shape", [(torch.float32, (64, 1024)), (torch.float32, (5, 33)),
                                         (torch.bfloat16, (40, 1001)), (torch.float16, (9, 12288)),
                                         (torch.bfloat16, (24, 8200))])
def test_fused_norm_backward_generic_shapes(dtype, shape):
    """fp32 tensors, column counts that are not multiples of 8 and rows wider than 8192 run on the
    element-wise backward kernels: same formulas, same tolerances (fp32: only summation order differs)."""
    torch.manual_seed(shape[-1])
    x = (torch.randn(shape, device="cuda") * 2).to(dtype).requires_grad_(True)
    w = (1 + 0.2 * torch.randn(shape[-1], device="cuda")).to(dtype).requires_grad_(True)
    g = torch.randn(shape, device="cuda").to(dtype)
    rms_norm_to_float8_dynamic(x, w, 1e-6).backward(g)
    x2, w2 = x.detach().clone().requires_grad_(True), w.detach().clone().requires_grad_(True)
    reference_rmsnorm(x2, w2, 1e-6).backward(g)
    floor = {torch.float32: 100, torch.bfloat16: 40, torch.float16: 55}[dtype]
    assert x.grad.dtype == dtype and w.grad.dtype == dtype
    assert _sqnr(x2.grad, x.grad) > floor + (5 if dtype != torch.float32 else 0)
    assert _sqnr(w2.grad, w.grad) > floor
    # the gate's backward on the same kinds of shapes
    a = (torch.randn(shape, device="cuda") * 2).to(dtype).requires_grad_(True)
    b = torch.randn(shape, device="cuda").to(dtype).requires_grad_(True)
    swiglu_to_float8_dynamic(a, b).backward(g)
    a2, b2 = a.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    (torch.nn.functional.silu(a2) * b2).backward(g)
    for got, ref in ((a.grad, a2.grad), (b.grad, b2.grad)):
        assert got.dtype == dtype and _sqnr(ref, got) > floor + (10 if dtype != torch.float32 else 0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(512, 4096), (3, 40, 264)])
def test_fused_swiglu_backward_kernel_matches_eager_autograd(dtype, shape):
    torch.manual_seed(shape[-1] + 1)
    h = (torch.randn(*shape[:-1], 2 * shape[-1], device="cuda") * 2).to(dtype)
    a = h[..., : shape[-1]].detach().requires_grad_(True)   # halves of one tensor: strided rows
    b = h[..., shape[-1]:].detach().requires_grad_(True)
    g = torch.randn(shape, device="cuda").to(dtype)
    swiglu_to_float8_dynamic(a, b).backward(g)
    a2, b2 = a.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    (torch.nn.functional.silu(a2) * b2).backward(g)
    # same formulas with the same roundings as eager autograd; exp and the fp32 expression order may
    # differ in the last bit
    for got, ref in ((a.grad, a2.grad), (b.grad, b2.grad)):
        assert got.dtype == dtype
        assert _sqnr(ref, got) > (50 if dtype == torch.bfloat16 else 65)
    assert (b.grad != b2.grad).float().mean().item() <= 1e-3


def test_ffn_fragment_with_fused_producers_matches_unfused_float8_model():
    """RMSNorm -> w1|w3 -> SwiGLU -> w2 (the FFN of the reference's benchmark model,
    float8_experimental/benchmarks/profile_linear_float8.py:52-149) with both producers fused
    into the casts of the linears that follow them, forward and backward, against the same
    float8 linears fed by eager RMSNorm and silu * mul."""
    import copy

    import torch.nn as nn

    import float8_experimental_b200 as f8
    from float8_experimental_b200.float8_linear import Float8Linear

    torch.manual_seed(3)
    dim, hidden, tokens = 1024, 2816, 512
    w13 = Float8Linear.from_float(nn.Linear(dim, 2 * hidden, bias=False, device="cuda", dtype=torch.bfloat16),
                                  f8.Float8LinearConfig())
    w2 = Float8Linear.from_float(nn.Linear(hidden, dim, bias=False, device="cuda", dtype=torch.bfloat16),
                                 f8.Float8LinearConfig())
    norm_w = (1 + 0.1 * torch.randn(dim, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    x = torch.randn(tokens, dim, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    go = torch.randn(tokens, dim, device="cuda", dtype=torch.bfloat16) * 1e-2

    def fused(xi, nw, l13, l2):
        h = l13(rms_norm_to_float8_dynamic(xi, nw, 1e-6, linear_mm_config=l13.linear_mm_config))
        return xi + l2(swiglu_to_float8_dynamic(h[:, :hidden], h[:, hidden:], linear_mm_config=l2.linear_mm_config))

    def unfused(xi, nw, l13, l2):
        h = l13(reference_rmsnorm(xi, nw, 1e-6))
        return xi + l2(torch.nn.functional.silu(h[:, :hidden]) * h[:, hidden:])

    y = fused(x, norm_w, w13, w2)
    y.backward(go)
    got = [y.detach(), x.grad, norm_w.grad, w13.weight.grad, w2.weight.grad]
    x2, nw2 = x.detach().clone().requires_grad_(True), norm_w.detach().clone().requires_grad_(True)
    l13b, l2b = copy.deepcopy(w13), copy.deepcopy(w2)
    l13b.weight.grad = None
    l2b.weight.grad = None
    y2 = unfused(x2, nw2, l13b, l2b)
    y2.backward(go)
    want = [y2.detach(), x2.grad, nw2.grad, l13b.weight.grad, l2b.weight.grad]
    for name, a, b in zip(("y", "dx", "dnorm_w", "dw13", "dw2"), got, want):
        assert _sqnr(b, a) > 40, name
