"""The single-GPU cluster-multicast GEMM (optional library libf8b200_mc.so) must return the
bits of the kernels in libf8b200.so: every output tile is accumulated the same way, only the
route the operand tiles take into shared memory differs."""
import pytest
import torch

from float8_experimental_b200 import _native as N

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _need_mc_library():
    if N.load_mc() is None:
        pytest.skip("libf8b200_mc.so is not part of this run")


def _gemm(a, b, sa, sb, m, n, k, out_dtype, bias, a_mn, b_mn):
    out = torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda")
    N.gemm_fp8(a, a.stride(0), b, b.stride(0), sa, sb, bias, out, n, m, n, k, False, a_mn_major=a_mn, b_mn_major=b_mn)
    torch.cuda.synchronize()
    assert N.read_device_error() == 0
    return out


@pytest.mark.parametrize("cluster", ["21", "22", "41"])
@pytest.mark.parametrize("mnk", [(512, 512, 256), (4096, 2048, 1024), (300, 520, 272), (8192, 4096 + 48, 512 + 16),
                                 (1280, 768, 128), (256, 256, 64), (4096, 8192, 16384 + 128)])
@pytest.mark.parametrize("layouts", [(False, False), (False, True), (True, True)])
def test_multicast_gemm_matches_plain_kernels(cluster, mnk, layouts, monkeypatch):
    m, n, k = mnk
    a_mn, b_mn = layouts
    if (a_mn and m % 16) or (b_mn and n % 16):
        pytest.skip("an MN-major operand needs a row count that is a multiple of 16")
    g = torch.Generator(device="cuda").manual_seed(m + 3 * n + 7 * k)
    a = torch.randn(m, k, device="cuda", generator=g).to(torch.float8_e5m2)
    b = torch.randn(n, k, device="cuda", generator=g).to(torch.float8_e4m3fn)
    sa, sb = torch.tensor(2.0, device="cuda"), torch.tensor(0.5, device="cuda")
    a_arg = a.view(torch.uint8).t().contiguous().view(a.dtype) if a_mn else a
    b_arg = b.view(torch.uint8).t().contiguous().view(b.dtype) if b_mn else b
    monkeypatch.setenv("F8B200_GEMM_MC", "0")
    want = _gemm(a_arg, b_arg, sa, sb, m, n, k, torch.bfloat16, None, a_mn, b_mn)
    monkeypatch.setenv("F8B200_GEMM_MC", cluster)
    for _ in range(2):
        got = _gemm(a_arg, b_arg, sa, sb, m, n, k, torch.bfloat16, None, a_mn, b_mn)
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("cluster", ["21", "22", "41"])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.float16])
def test_multicast_gemm_bias_and_output_types(cluster, out_dtype, monkeypatch):
    m, n, k = 768, 640, 512
    a = torch.randn(m, k, device="cuda").to(torch.float8_e4m3fn)
    b = torch.randn(n, k, device="cuda").to(torch.float8_e4m3fn)
    bias = torch.randn(n, device="cuda").to(out_dtype)
    one = torch.tensor(1.0, device="cuda")
    monkeypatch.setenv("F8B200_GEMM_MC", "0")
    want = _gemm(a, b, one, one, m, n, k, out_dtype, bias, False, False)
    monkeypatch.setenv("F8B200_GEMM_MC", cluster)
    got = _gemm(a, b, one, one, m, n, k, out_dtype, bias, False, False)
    assert torch.equal(got, want)
