"""Parity of the CUDA kernels, called through the C ABI, against the oracle and the
reference's recorded outputs.  Casts, amaxes and scales: bit-exact.  GEMM: SQNR >= 25 dB
and max relative error <= 2e-2 against the emulated fp32 product."""
import os

import numpy as np
import pytest
import torch

from float8_experimental_b200 import _native as N
from oracle import f8_oracle as O

pytestmark = pytest.mark.gpu

DT = {O.BF16: torch.bfloat16, O.FP16: torch.float16, O.FP32: torch.float32}
KIND = {O.E4M3: N.E4M3, O.E5M2: N.E5M2}
TF8 = {O.E4M3: torch.float8_e4m3fn, O.E5M2: torch.float8_e5m2}
GEMM_SQNR_DB = 25.0
GEMM_MAX_REL = 2e-2


def dev_tensor(arr, dname):
    if dname == O.FP32:
        return torch.from_numpy(np.ascontiguousarray(arr)).cuda()
    return torch.from_numpy(np.ascontiguousarray(arr).view(np.int16)).cuda().view(DT[dname])


def host_bits(t):
    t = t.contiguous()
    if t.dtype == torch.float32:
        return t.cpu().numpy()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.cpu().view(torch.int16).numpy().view(np.uint16)
    return t.cpu().view(torch.uint8).numpy()


def nan_class_equal(a, b):
    an, bn = (a & 0x7F) == 0x7F, (b & 0x7F) == 0x7F
    return bool(np.all((a == b) | (an & bn)))


def run_cast(x, fname, *, scale=None, product_fp32=False, transpose=True, want_amax=False, reverse=False):
    x2 = x.reshape(-1, x.shape[-1])
    rows, cols = x2.shape
    out = torch.full((rows, cols), 0x55, dtype=torch.uint8, device="cuda")
    ld_t = (rows + 15) // 16 * 16
    out_t = torch.full((cols, ld_t), 0x55, dtype=torch.uint8, device="cuda") if transpose else None
    amax = torch.zeros((), device="cuda")
    sc = torch.zeros((), device="cuda")
    amax2 = torch.full((1,), -1.0, device="cuda") if want_amax else None
    if scale is None:
        N.amax(x2.contiguous(), amax)  # the C entry point reduces a contiguous range
        N.cast(x2, rows, cols, x2.stride(0), 1, amax, sc, product_fp32, KIND[fname], out, cols, out_t, ld_t, amax2,
               reverse)
    else:
        sc.fill_(float(scale))
        N.cast(x2, rows, cols, x2.stride(0), 0, sc, None, product_fp32, KIND[fname], out, cols, out_t, ld_t, amax2,
               reverse)
    torch.cuda.synchronize()
    return (out.cpu().numpy(), out_t[:, :rows].cpu().numpy() if transpose else None, amax.item(), sc.item(),
            amax2.item() if want_amax else None)


def test_device_is_supported():
    assert N.load().f8b200_device_check() == 0


def test_casts_match_reference_fixture(golden_dir):
    g = np.load(os.path.join(golden_dir, "casts.npz"))
    for i in range(int(g["n"])):
        dname, fname = [str(s) for s in g[f"c{i}_meta"]]
        x = dev_tensor(g[f"c{i}_x"], dname)
        bits, bits_t, amax, scale, _ = run_cast(x, fname, reverse=bool(i & 1))
        ref = g[f"c{i}_dyn_bits"].reshape(bits.shape)
        assert scale == g[f"c{i}_dyn_scale"], (i, dname, fname)
        assert np.array_equal(bits, ref), (i, dname, fname)
        assert np.array_equal(bits_t, ref.T), (i, dname, fname)
        dbits, dbits_t, _, _, damax = run_cast(x, fname, scale=g[f"c{i}_del_scale"][0], product_fp32=True,
                                               want_amax=True)
        dref = g[f"c{i}_del_bits"].reshape(bits.shape)
        assert np.array_equal(dbits, dref) and np.array_equal(dbits_t, dref.T), (i, dname, fname)
        assert damax == g[f"c{i}_del_amax"][0]


def test_every_bf16_pattern(golden_dir):
    g = np.load(os.path.join(golden_dir, "exhaustive_bf16.npz"))
    pat = np.arange(65536, dtype=np.uint16).reshape(256, 256)
    x = dev_tensor(pat, O.BF16)
    for fname in (O.E4M3, O.E5M2):
        for si, s in enumerate(g["scales"]):
            for tag, pf32 in (("dim0", False), ("dim1", True)):
                bits, bits_t, *_ = run_cast(x, fname, scale=s, product_fp32=pf32)
                ref = g[f"{fname}_{si}_{tag}"].reshape(256, 256)
                assert nan_class_equal(bits, ref), (fname, s, tag)
                assert nan_class_equal(bits_t, ref.T), (fname, s, tag)


@pytest.mark.parametrize("dname", [O.BF16, O.FP16, O.FP32])
@pytest.mark.parametrize("shape", [(1, 1), (3, 5), (17, 36), (128, 128), (129, 260), (1000, 12), (7, 4096)])
def test_cast_shapes_against_oracle(dname, shape):
    g = torch.Generator(device="cpu").manual_seed(hash((dname, shape)) % 2**31)
    x = (torch.randn(shape, generator=g) * torch.exp(2 * torch.randn(shape, generator=g))).to(DT[dname]).cuda()
    xb = host_bits(x)
    for fname in (O.E4M3, O.E5M2):
        bits, bits_t, amax, scale, _ = run_cast(x, fname)
        rbits, rscale, ramax = O.cast_dynamic(xb, dname, fname)
        assert amax == float(ramax) and scale == float(rscale)
        assert np.array_equal(bits, rbits) and np.array_equal(bits_t, rbits.T)
        bits, bits_t, _, _, amax2 = run_cast(x, fname, scale=0.731, product_fp32=True, want_amax=True)
        rbits, ramax = O.cast_delayed(xb, dname, np.float32(0.731), fname)
        assert amax2 == float(ramax)
        assert np.array_equal(bits, rbits) and np.array_equal(bits_t, rbits.T)


def test_cast_strided_rows_and_special_values():
    torch.manual_seed(11)
    base = torch.randn(64, 200, dtype=torch.bfloat16, device="cuda")
    x = base[:, 8:136]  # ld 200, 128 columns, 16-byte aligned start
    bits, bits_t, amax, scale, _ = run_cast(x, O.E4M3)
    rbits, rscale, ramax = O.cast_dynamic(host_bits(x), O.BF16, O.E4M3)
    assert np.array_equal(bits, rbits) and np.array_equal(bits_t, rbits.T) and scale == float(rscale)
    y = torch.tensor([[0.0, -0.0, float("inf"), -float("inf")], [1e-30, -1e-30, 448.0, -449.0]], device="cuda")
    bits, *_ = run_cast(y, O.E4M3, scale=1.0, product_fp32=True, transpose=False)
    assert np.array_equal(bits, O.cast_to_fp8(y.cpu().numpy(), O.FP32, 1.0, O.E4M3, O.FP32))
    z = torch.zeros(33, 8, dtype=torch.float16, device="cuda")  # amax 0 -> fp16 scale clamps to 65504
    _, _, amax, scale, _ = run_cast(z, O.E5M2)
    assert amax == 0.0 and scale == 65504.0


def test_amax_nan_heads_tails_and_errors():
    out = torch.zeros((), device="cuda")
    x = torch.randn(100003, dtype=torch.bfloat16, device="cuda")
    for off in (0, 1, 3, 7):
        N.amax(x[off:], out)
        assert out.item() == x[off:].abs().max().item()
    xf = torch.randn(50001, device="cuda")
    N.amax(xf[1:], out)
    assert out.item() == xf[1:].abs().max().item()
    x[4321] = float("nan")
    N.amax(x, out)
    assert np.isnan(out.item())
    with pytest.raises(N.F8B200Error):
        N.amax(x[:0], out)


def test_multi_amax():
    sizes = [5, 0, 1000, 123457, 1 << 22] + [257] * 200
    xs = [torch.randn(n, device="cuda") * (1 + i % 7) for i, n in enumerate(sizes)]
    out = torch.full((len(xs),), -1.0, device="cuda")
    N.multi_amax(xs, out)
    ref = [t.abs().max().item() if t.numel() else 0.0 for t in xs]
    assert out.tolist() == ref


def test_amax_to_scale_every_pattern(golden_dir):
    g = np.load(os.path.join(golden_dir, "exhaustive_bf16.npz"))
    pat = np.arange(32768, dtype=np.uint16)
    for dname, code in ((O.BF16, N.BF16), (O.FP16, N.FP16)):
        a = torch.from_numpy(O.to_f32(pat, dname)).cuda()
        for fname in (O.E4M3, O.E5M2):
            out = torch.empty_like(a)
            N.amax_to_scale(a, KIND[fname], code, code, out)
            got = out.cpu().numpy()
            ref = g[f"scale_{dname}_{fname}"].view(np.float32)
            same = (got.view(np.uint32) == ref.view(np.uint32)) | (np.isnan(got) & np.isnan(ref))
            assert same.all(), (dname, fname)


def test_delayed_sync_matches_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "sync.npz"))
    for dname, code in ((O.BF16, N.BF16), (O.FP16, N.FP16), (O.FP32, N.FP32)):
        amax, hist = g[f"{dname}_amax"], g[f"{dname}_hist"]
        L = amax.shape[1]
        a = torch.from_numpy(amax.reshape(-1).copy()).cuda()
        h = torch.from_numpy(hist.reshape(3 * L, -1).copy()).cuda()
        s = torch.zeros(3 * L, device="cuda")
        N.delayed_sync(a, h, 2 * L, code, s, None)
        assert np.array_equal(s.cpu().numpy().reshape(3, L), g[f"{dname}_scales"])
        assert np.array_equal(h.cpu().numpy().reshape(hist.shape), hist)
        N.delayed_sync(a, h, 2 * L, code, s, h)  # in place roll
        _, rolled = O.sync_amax_and_scale(amax.reshape(-1), hist.reshape(3 * L, -1), [O.E4M3] * 3 * L, dname, True)
        assert np.array_equal(h.cpu().numpy(), rolled)


@pytest.mark.parametrize("dname", [O.BF16, O.FP16, O.FP32])
def test_multi_tensor_cast_matches_single_casts(dname):
    """One launch casting many contiguous tensors, each with its own scale, returns the bytes of
    one f8b200_cast per tensor (which are pinned against the reference): every size class (empty,
    shorter than a vector, ragged tails, large), more tensors than one launch holds, both
    product-rounding routes."""
    g = torch.Generator(device="cuda").manual_seed(11)
    sizes = [0, 1, 7, 8, 9, 1000, 4096, 12345, 1 << 20, 3 * 1024 * 512 + 5] + [257 + 13 * i for i in range(100)]
    xs = [(torch.randn(n, device="cuda", generator=g) * (1 + i % 5)).to(DT[dname]) for i, n in enumerate(sizes)]
    scales = (torch.rand(len(sizes), device="cuda", generator=g) * 100 + 0.5).to(DT[dname]).float()
    for product_fp32 in (False, True):
        outs = [torch.full((n,), 0x55, dtype=torch.uint8, device="cuda") for n in sizes]
        N.multi_cast(xs, scales, product_fp32, N.E4M3, outs)
        torch.cuda.synchronize()
        for i, (x, n) in enumerate(zip(xs, sizes)):
            if n == 0:
                continue
            want = torch.empty(1, n, dtype=torch.uint8, device="cuda")
            N.cast(x.view(1, n), 1, n, n, 0, scales[i:i + 1], None, product_fp32, N.E4M3, want, n, None, 0, None, False)
            assert torch.equal(outs[i], want[0]), (dname, product_fp32, i, n)
        # and against the oracle directly on one of them
        i = 5
        ref = O.cast_to_fp8(host_bits(xs[i]), dname, np.float32(scales[i].item()), O.E4M3, O.FP32 if product_fp32 else dname)
        assert nan_class_equal(outs[i].cpu().numpy(), ref)


@pytest.mark.parametrize("dname", [O.BF16, O.FP16, O.FP32])
@pytest.mark.parametrize("shape", [(256, 512), (77, 264), (5, 3), (4096, 4096)])
def test_one_call_dynamic_cast_matches_the_oracle(dname, shape):
    """f8b200_cast_dynamic (amax + cast in one host call): amax, scale and bytes of the oracle."""
    g = torch.Generator(device="cuda").manual_seed(shape[0] + shape[1])
    x = (torch.randn(shape, device="cuda", generator=g) * 3).to(DT[dname])
    for fname in (O.E4M3, O.E5M2):
        out = torch.full(shape, 0x55, dtype=torch.uint8, device="cuda")
        amax, scale = torch.zeros((), device="cuda"), torch.zeros((), device="cuda")
        N.cast_dynamic(x, shape[0], shape[1], KIND[fname], amax, scale, out)
        torch.cuda.synchronize()
        bits, rscale, ramax = O.cast_dynamic(host_bits(x), dname, fname)
        assert amax.item() == float(ramax) and scale.item() == float(rscale)
        assert np.array_equal(out.cpu().numpy(), bits)


def test_transpose_u8():
    for shape in ((128, 128), (130, 260), (5, 3), (1024, 16), (16, 1024)):
        x = torch.randint(0, 256, shape, dtype=torch.uint8, device="cuda")
        out = torch.zeros(shape[1], shape[0], dtype=torch.uint8, device="cuda")
        N.transpose_u8(x, shape[0], shape[1], shape[1], out, shape[0])
        assert torch.equal(out, x.t().contiguous())


# ---------------------------------------------------------------------------
@pytest.fixture(params=["2cta", "1cta", "wide", "pw", "2cta-direct", "1cta-direct", "wide-direct", "pw-direct",
                        "wide-smem", "pw-smem"])
def gemm_mode(request, monkeypatch):
    """The four GEMM kernels (CTA pairs on 256x256 tiles; one CTA per 128x256 tile; one CTA per
    256x256 tile; CTA pairs on 512x256 tiles), each with the TMA-store epilogue and with the
    per-thread store epilogue; the two kernels whose accumulator fills tensor memory also with
    their third epilogue (whole lines written by the warps after staging in shared memory)."""
    mode, _, store = request.param.partition("-")
    monkeypatch.setenv("F8B200_GEMM_MODE", mode)
    monkeypatch.setenv("F8B200_GEMM_STORE", store or "tma")
    return request.param


def gemm(a8, b8, sa, sb, out_dtype=torch.bfloat16, bias=None):
    m, k = a8.shape
    n = b8.shape[0]
    out = torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda")
    N.gemm_fp8(a8, a8.stride(0), b8, b8.stride(0), sa, sb, bias, out, n, m, n, k, False)
    torch.cuda.synchronize()
    assert N.read_device_error() == 0
    return out


def check_gemm(out, ref):
    out, ref = out.double(), ref.double()
    sqnr = 20 * torch.log10(ref.norm() / (ref - out).norm()).item()
    max_rel = ((ref - out).abs().max() / ref.abs().max()).item()
    assert sqnr >= GEMM_SQNR_DB, sqnr
    assert max_rel <= GEMM_MAX_REL, max_rel


@pytest.mark.parametrize("mnk", [(128, 256, 128), (256, 512, 1024), (200, 264, 144), (1, 8, 16), (130, 40, 4096),
                                 (640, 1024, 2064), (300, 520, 272), (130, 20, 64), (257, 72, 48)])
@pytest.mark.parametrize("a_kind", [O.E4M3, O.E5M2])
def test_gemm_against_oracle(mnk, a_kind, gemm_mode):
    m, n, k = mnk
    g = torch.Generator().manual_seed(m * 7 + n * 3 + k)
    a = torch.randn(m, k, generator=g).to(TF8[a_kind]).cuda()
    b = torch.randn(n, k, generator=g).to(torch.float8_e4m3fn).cuda()
    sa, sb = torch.tensor(3.0, device="cuda"), torch.tensor(0.25, device="cuda")
    out = gemm(a, b, sa, sb)
    ref = O.mm_float8_emulated(host_bits(a), a_kind, 3.0, host_bits(b).T, O.E4M3, 0.25, O.FP32)
    check_gemm(out.float().cpu(), torch.from_numpy(ref))


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_gemm_output_types_and_bias(out_dtype, gemm_mode):
    a = torch.randn(256, 512, device="cuda").to(torch.float8_e4m3fn)
    b = torch.randn(384, 512, device="cuda").to(torch.float8_e4m3fn)
    bias = torch.randn(384, device="cuda").to(out_dtype)
    one = torch.tensor(1.0, device="cuda")
    out = gemm(a, b, one, one, out_dtype, bias)
    ref = a.float() @ b.float().t() + bias.float()
    check_gemm(out.float(), ref)
    if out_dtype == torch.float32:
        # products of fp8 values are exact in fp32: only the summation order differs
        assert (out - ref).abs().max().item() < 1e-3


def test_gemm_full_size_linearity(gemm_mode):
    """At a full LLaMa-2-70B shape the oracle is too slow; check size-independent properties:
    agreement with an fp32 GEMM of the dequantised operands on sampled rows, and
    out(2a, b) == 2 out(a, b) exactly (powers of two commute with every rounding)."""
    m, n, k = 16384, 8192, 8192
    a = torch.randn(m, k, device="cuda").mul_(0.5).to(torch.float8_e4m3fn)
    b = torch.randn(n, k, device="cuda").mul_(0.5).to(torch.float8_e4m3fn)
    one = torch.tensor(1.0, device="cuda")
    out = gemm(a, b, one, one)
    rows = torch.tensor([0, 127, 128, 5000, 16383], device="cuda")
    ref = a[rows].float() @ b.float().t()
    check_gemm(out[rows].float(), ref)
    half = torch.tensor(0.5, device="cuda")
    out2 = gemm(a, b, half, one)  # dividing by scale 0.5 doubles the result
    assert torch.equal(out2.float(), out.float() * 2)


@pytest.mark.parametrize("mnk", [(4096, 8192, 512), (8192, 4096 + 48, 1024 + 16), (2048, 2048, 128)])
def test_gemm_dynamic_schedule_matches_fixed_stride(mnk, gemm_mode, monkeypatch):
    """With a workspace the persistent kernels claim tiles from a counter; without one every
    CTA walks a fixed stride.  Each tile is accumulated the same way in both, so the outputs
    are bit-identical, call after call (the counter is reset by every call)."""
    m, n, k = mnk
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = torch.randn(m, k, device="cuda", generator=g).to(torch.float8_e4m3fn)
    b = torch.randn(n, k, device="cuda", generator=g).to(torch.float8_e4m3fn)
    sa, sb = torch.tensor(2.0, device="cuda"), torch.tensor(0.5, device="cuda")
    monkeypatch.setenv("F8B200_GEMM_WS", "0")
    fixed = gemm(a, b, sa, sb)
    monkeypatch.setenv("F8B200_GEMM_WS", "1")
    for _ in range(3):
        assert torch.equal(gemm(a, b, sa, sb).view(torch.int16), fixed.view(torch.int16))
    rows = torch.tensor([0, 255, 256, m - 1], device="cuda")
    check_gemm(fixed[rows].float(), a[rows].float() @ b.float().t())


@pytest.mark.parametrize("mnk", [(2048, 1024, 384), (4096 + 40, 2048 + 24, 1024 + 16), (1024, 512, 128 * 3),
                                 (8192, 4096, 128 * 6), (8192, 8192, 128 * 8), (4096, 4096, 128 * 9 + 16), (512, 256, 128)])
def test_gemm_split_drain_matches_whole_drain(mnk, monkeypatch):
    """The 512x256 pair kernel starts the next tile on the accumulator half its epilogue has already
    drained; with F8B200_GEMM_SPLIT_DRAIN=0 it waits for the whole accumulator.  Every output element
    is accumulated in the same order either way, so the outputs are bit-identical, and equal to the
    256x256 pair kernel's."""
    m, n, k = mnk
    g = torch.Generator(device="cuda").manual_seed(m + 3 * n + k)
    a = torch.randn(m, k, device="cuda", generator=g).to(torch.float8_e4m3fn)
    b = torch.randn(n, k, device="cuda", generator=g).to(torch.float8_e4m3fn)
    sa, sb = torch.tensor(2.0, device="cuda"), torch.tensor(0.5, device="cuda")
    monkeypatch.setenv("F8B200_GEMM_MODE", "2cta")
    want = gemm(a, b, sa, sb)
    monkeypatch.setenv("F8B200_GEMM_MODE", "pw")
    for split in ("0", "head", "1", "1"):  # none / start of the next tile only / both ends (the default)
        monkeypatch.setenv("F8B200_GEMM_SPLIT_DRAIN", split)
        assert torch.equal(gemm(a, b, sa, sb).view(torch.int16), want.view(torch.int16)), split
    rows = torch.tensor(sorted({min(r, m - 1) for r in (0, 127, 128, 255, 256, 511, 512, m - 1)}), device="cuda")
    check_gemm(want[rows].float(), a[rows].float() @ b.float().t())


@pytest.mark.parametrize("store", ["", "direct"])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("mnk_dests_rows", [((2048, 1024, 256), 2, 256), ((4096, 2048 + 24, 1024 + 16), 4, 128),
                                            ((1536, 512, 128), 3, 512), ((1024, 768, 384), 1, 1024)])
def test_gemm_scatter_rows_matches_plain_gemm(mnk_dests_rows, out_dtype, store, monkeypatch):
    """`f8b200_gemm_fp8_scatter_rows` sends output row block i to destination i % n at block row i // n.
    Put back in order, the destinations hold the bits of the plain GEMM, with the warp-written whole-line
    stores (the default) as with per-thread stores."""
    (m, n, k), dests, rpb = mnk_dests_rows
    g = torch.Generator(device="cuda").manual_seed(m + 5 * n + k + dests)
    a = torch.randn(m, k, device="cuda", generator=g).to(torch.float8_e4m3fn)
    b = torch.randn(n, k, device="cuda", generator=g).to(torch.float8_e5m2)
    sa, sb = torch.tensor(2.0, device="cuda"), torch.tensor(0.25, device="cuda")
    want = gemm(a, b, sa, sb, out_dtype=out_dtype)
    blocks = m // rpb
    assert blocks % dests == 0
    outs = [torch.full((blocks // dests * rpb, n), float("nan"), dtype=out_dtype, device="cuda") for _ in range(dests)]
    monkeypatch.setenv("F8B200_GEMM_SCATTER_STORE", store)
    for _ in range(2):
        N.gemm_fp8_scatter_rows(a, k, b, k, sa, sb, out_dtype, [o.data_ptr() for o in outs], rpb, n, m, n, k)
    got = torch.empty_like(want)
    for blk in range(blocks):
        src = outs[blk % dests][(blk // dests) * rpb:(blk // dests + 1) * rpb]
        got[blk * rpb:(blk + 1) * rpb] = src
    as_int = torch.int16 if out_dtype == torch.bfloat16 else torch.int32
    assert torch.equal(got.view(as_int), want.view(as_int))


@pytest.mark.parametrize("layouts", [(False, True), (True, False), (True, True)])
@pytest.mark.parametrize("mnk", [(512, 768, 256), (4096, 2048 + 16, 1024 + 48), (8192, 4096, 16384 + 128)])
@pytest.mark.parametrize("mode", ["2cta", "wide", "pw"])
def test_gemm_mn_major_operands(mnk, layouts, mode, monkeypatch):
    """An operand may be handed over as the transpose of the usual storage ([K, rows], rows
    contiguous): the result has to be bit-identical to the K-major call on the same values."""
    monkeypatch.setenv("F8B200_GEMM_MODE", mode)
    m, n, k = mnk
    a_mn, b_mn = layouts
    g = torch.Generator(device="cuda").manual_seed(m * 3 + n + k)
    a = torch.randn(m, k, device="cuda", generator=g).to(torch.float8_e5m2)
    b = torch.randn(n, k, device="cuda", generator=g).to(torch.float8_e4m3fn)
    sa, sb = torch.tensor(2.0, device="cuda"), torch.tensor(0.5, device="cuda")
    want = gemm(a, b, sa, sb)
    a_arg = a.view(torch.uint8).t().contiguous().view(torch.float8_e5m2) if a_mn else a      # [k, m]
    b_arg = b.view(torch.uint8).t().contiguous().view(torch.float8_e4m3fn) if b_mn else b    # [k, n]
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    N.gemm_fp8(a_arg, a_arg.stride(0), b_arg, b_arg.stride(0), sa, sb, None, out, n, m, n, k, False,
               a_mn_major=a_mn, b_mn_major=b_mn)
    torch.cuda.synchronize()
    assert N.read_device_error() == 0
    rows = torch.tensor([0, 127, 128, 255, 256, m - 1], device="cuda")
    check_gemm(out[rows].float(), a[rows].float() @ b.float().t() / (2.0 * 0.5))
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("mnk", [(256, 384, 100), (300, 72, 1000 + 8), (1024, 512, 16384 + 40)])
def test_gemm_inner_dimension_need_not_be_a_multiple_of_16(mnk, gemm_mode):
    """K is free as long as the row pitch is a multiple of 16 bytes: TMA zero-fills beyond K."""
    m, n, k = mnk
    pitch = -(-k // 16) * 16
    g = torch.Generator(device="cuda").manual_seed(k)
    a_buf = torch.randn(m, pitch, device="cuda", generator=g).to(torch.float8_e4m3fn)  # junk beyond K
    b_buf = torch.randn(n, pitch, device="cuda", generator=g).to(torch.float8_e4m3fn)
    a, b = a_buf[:, :k], b_buf[:, :k]
    one = torch.tensor(1.0, device="cuda")
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    N.gemm_fp8(a, pitch, b, pitch, one, one, None, out, n, m, n, k, False)
    torch.cuda.synchronize()
    assert N.read_device_error() == 0
    ref = a.float() @ b.float().t()
    check_gemm(out, ref)
    assert (out - ref).abs().max().item() <= 1e-3 * max(1.0, ref.abs().max().item())


def test_cast_full_size_properties():
    """Full-size activation (16384 x 8192 bf16): the oracle is too slow here, so check
    size-independent properties: amax equals max|x|; the transposed copy is the transpose;
    every decoded value is within half an fp8 step of x*scale; casting the dequantised
    tensor again with the same scale returns the same bytes (idempotence)."""
    torch.manual_seed(5)
    x = torch.randn(16384, 8192, device="cuda", dtype=torch.bfloat16)
    x[123, 4567] = 37.5
    rows, cols = x.shape
    out = torch.empty(rows, cols, dtype=torch.uint8, device="cuda")
    out_t = torch.empty(cols, rows, dtype=torch.uint8, device="cuda")
    amax, sc = torch.zeros((), device="cuda"), torch.zeros((), device="cuda")
    N.amax(x, amax)
    N.cast(x, rows, cols, cols, 1, amax, sc, False, N.E4M3, out, cols, out_t, rows, None, True)
    torch.cuda.synchronize()
    assert amax.item() == 37.5
    assert sc.item() == float(O.amax_to_scale(np.float32(37.5), O.E4M3, O.BF16, O.BF16))
    assert torch.equal(out_t, out.t())
    deq = out.view(torch.float8_e4m3fn).float()
    prod = (x * sc.to(torch.bfloat16)).float()  # the reference's bf16 product
    err = (deq - prod).abs()
    step = torch.maximum(prod.abs() * 2.0 ** -4, torch.tensor(2.0 ** -10, device="cuda"))  # half ulp of e4m3
    assert bool((err <= step).all())
    again = torch.empty_like(out)
    one = torch.ones((), device="cuda")
    N.cast(deq, rows, cols, cols, 0, one, None, True, N.E4M3, again, cols, None, 0, None, False)
    assert torch.equal(again, out)


@pytest.mark.parametrize("hist_len", [1, 4, 16, 17, 40])
def test_delayed_sync_history_lengths(hist_len):
    rng = np.random.default_rng(hist_len)
    rows = 77
    amax = (rng.random(rows) * 5).astype(np.float32)
    hist = (rng.random((rows, hist_len)) * 5).astype(np.float32)
    hist[3, 0] = np.nan
    amax[9] = np.nan
    kinds = [O.E4M3] * 50 + [O.E5M2] * 27
    ref_scale, ref_hist = O.sync_amax_and_scale(amax, hist, kinds, O.FP32, True)
    a, h = torch.from_numpy(amax).cuda(), torch.from_numpy(hist).cuda()
    s = torch.zeros(rows, device="cuda")
    N.delayed_sync(a, h, 50, N.FP32, s, h)  # in place
    got_s, got_h = s.cpu().numpy(), h.cpu().numpy()
    assert np.all((got_s == ref_scale) | (np.isnan(got_s) & np.isnan(ref_scale)))
    assert np.all((got_h == ref_hist) | (np.isnan(got_h) & np.isnan(ref_hist)))
