"""Parity at the full sizes of the LLaMa-2-70B configuration (M = 16384 tokens; (K, N) = wqkv
(8192, 10240), wo (8192, 8192), w13 (8192, 57344), w2 (28672, 8192)).

Casts: every tensor of every layer (input, weight, grad_output) is cast on the GPU and by the C
restatement of the reference's arithmetic (`oracle/f8_oracle_c.c`, OpenMP) and compared byte for
byte, amax and scale included.  GEMMs: the products whose K or N is long (the ones the small-shape
tests never reach: 57344 columns, K up to 57344) are checked on sampled rows and columns, tile
edges included, against an fp32 product of the dequantised operands, through every kernel that can
run them."""
import numpy as np
import pytest
import torch

from float8_experimental_b200 import _native as N
from oracle import f8_oracle_c as C

pytestmark = pytest.mark.gpu

M = 16384
LAYERS = {"wqkv": (8192, 10240), "wo": (8192, 8192), "w13": (8192, 57344), "w2": (28672, 8192)}
GEMM_SQNR_DB = 25.0
GEMM_MAX_REL = 2e-2


def _bits(t):
    return t.contiguous().cpu().view(torch.int16).numpy().view(np.uint16)


def _tensor(shape, sigma, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(shape, device="cuda", dtype=torch.bfloat16, generator=g).mul_(sigma)


@pytest.mark.parametrize("layer", list(LAYERS))
def test_dynamic_casts_of_a_whole_layer_are_bit_exact(layer):
    """amax, scale and every fp8 byte of x (e4m3), W (e4m3) and grad_output (e5m2) at full size."""
    k, n = LAYERS[layer]
    cases = [("x", (M, k), 1.0, N.E4M3, "e4m3fn"), ("w", (n, k), 0.02, N.E4M3, "e4m3fn"),
             ("go", (M, n), 1e-3, N.E5M2, "e5m2")]
    for i, (name, shape, sigma, kind, oname) in enumerate(cases):
        x = _tensor(shape, sigma, 1000 * (list(LAYERS).index(layer) + 1) + i)
        rows, cols = shape
        out = torch.empty(rows, cols, dtype=torch.uint8, device="cuda")
        amax, scale = torch.zeros((), device="cuda"), torch.zeros((), device="cuda")
        N.amax(x, amax)
        N.cast(x, rows, cols, cols, 1, amax, scale, False, kind, out, cols, None, 0, None, True)
        torch.cuda.synchronize()
        want, want_scale, want_amax = C.cast_dynamic(_bits(x), "bf16", oname)
        assert amax.item() == float(want_amax), (layer, name)
        assert scale.item() == float(want_scale), (layer, name)
        got = out.cpu().numpy()
        assert np.array_equal(got, want), (layer, name, int((got != want).sum()))
        del x, out, got, want


def _check(out, ref, what):
    out, ref = out.double(), ref.double()
    sqnr = 20 * torch.log10(ref.norm() / (ref - out).norm()).item()
    peak = ref.abs().max()
    max_rel = ((ref - out).abs().max() / peak).item()
    assert sqnr >= GEMM_SQNR_DB, (what, sqnr)
    assert max_rel <= GEMM_MAX_REL, (what, max_rel)
    # element by element, on every element that is not small against the largest one
    big = ref.abs() >= 1e-2 * peak
    rel = ((ref - out).abs()[big] / ref.abs()[big]).max().item()
    assert rel <= GEMM_MAX_REL, (what, rel)


FULL_GEMMS = {
    # name: (m, n, k, A format)
    "w13.fwd": (M, 57344, 8192, torch.float8_e4m3fn),
    "w13.dgrad": (M, 8192, 57344, torch.float8_e5m2),
    "w13.wgrad": (57344, 8192, M, torch.float8_e5m2),
    "w2.fwd": (M, 8192, 28672, torch.float8_e4m3fn),
    "w2.wgrad": (8192, 28672, M, torch.float8_e5m2),
}


@pytest.mark.parametrize("mode", ["2cta", "wide", "pw", "pw-smem"])
@pytest.mark.parametrize("name", list(FULL_GEMMS))
def test_long_gemms_on_sampled_rows_and_columns(name, mode, monkeypatch):
    monkeypatch.setenv("F8B200_GEMM_MODE", mode.split("-")[0])
    monkeypatch.setenv("F8B200_GEMM_STORE", "smem" if mode.endswith("-smem") else "")
    m, n, k, a_dt = FULL_GEMMS[name]
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = torch.randn(m, k, device="cuda", generator=g).mul_(0.5).to(a_dt)
    b = torch.randn(n, k, device="cuda", generator=g).mul_(0.5).to(torch.float8_e4m3fn)
    sa, sb = torch.tensor(4.0, device="cuda"), torch.tensor(0.5, device="cuda")
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    N.gemm_fp8(a, k, b, k, sa, sb, None, out, n, m, n, k, False)
    torch.cuda.synchronize()
    assert N.read_device_error() == 0
    assert not bool(torch.isnan(out).any())
    inv = 1.0 / (4.0 * 0.5)
    rows = torch.tensor(sorted({0, 127, 128, 255, 256, 511, 512, m // 2 + 3, m - 257, m - 1}), device="cuda")
    cols = torch.tensor(sorted({0, 127, 128, 255, 256, n // 2 + 5, n - 129, n - 1}), device="cuda")
    _check(out[rows].float(), (a[rows].float() @ b.float().t()) * inv, (name, mode, "rows"))
    del_b = b[cols].float()
    _check(out[:, cols].float(), (a.float() @ del_b.t()) * inv, (name, mode, "cols"))


def test_gemm_runs_on_every_device_of_the_process():
    """The shared-memory opt-in of the GEMM kernels is a per-device attribute: a process that drives
    two GPUs gets correct products on both (needs two visible GPUs)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from oracle import f8_oracle as O

    for dev in (0, 1):
        for mode_k in (512, 16384 + 128):  # pair kernel, then the long-K kernel
            g = torch.Generator().manual_seed(dev * 7 + mode_k)
            a = torch.randn(300, mode_k, generator=g).to(torch.float8_e4m3fn).to(f"cuda:{dev}")
            b = torch.randn(272, mode_k, generator=g).to(torch.float8_e4m3fn).to(f"cuda:{dev}")
            sa = torch.tensor(3.0, device=f"cuda:{dev}")
            sb = torch.tensor(0.25, device=f"cuda:{dev}")
            out = torch.full((300, 272), float("nan"), dtype=torch.bfloat16, device=f"cuda:{dev}")
            N.gemm_fp8(a, mode_k, b, mode_k, sa, sb, None, out, 272, 300, 272, mode_k, False)
            torch.cuda.synchronize(dev)
            ref = O.mm_float8_emulated(a.cpu().view(torch.uint8).numpy(), O.E4M3, 3.0,
                                       b.cpu().view(torch.uint8).numpy().T, O.E4M3, 0.25, O.FP32)
            _check(out.float().cpu(), torch.from_numpy(ref), ("device", dev, mode_k))
    with torch.cuda.device(1):
        assert N.read_device_error() == 0
    assert N.read_device_error() == 0
