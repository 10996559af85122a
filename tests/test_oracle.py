"""The oracle against the reference's recorded outputs and against torch's own fp8
conversion.  CPU only."""
import os

import numpy as np
import pytest
import torch

from oracle import f8_oracle as O

TORCH_F8 = {O.E4M3: torch.float8_e4m3fn, O.E5M2: torch.float8_e5m2}


def nan_class_equal(a, b):
    """fp8 bytes equal, NaN encodings compared by class (the sign of a NaN depends on the
    host's vector ISA and is not part of the contract)."""
    an, bn = (a & 0x7F) == 0x7F, (b & 0x7F) == 0x7F
    return bool(np.all((a == b) | (an & bn)))


def test_casts_match_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "casts.npz"))
    for i in range(int(g["n"])):
        dname, fname = [str(s) for s in g[f"c{i}_meta"]]
        x = g[f"c{i}_x"]
        bits, scale, _ = O.cast_dynamic(x, dname, fname)
        assert np.float32(scale) == g[f"c{i}_dyn_scale"], (i, dname, fname)
        assert np.array_equal(bits, g[f"c{i}_dyn_bits"]), (i, dname, fname)
        dbits, amax = O.cast_delayed(x, dname, g[f"c{i}_del_scale"][0], fname)
        assert np.array_equal(dbits, g[f"c{i}_del_bits"]), (i, dname, fname)
        assert amax == g[f"c{i}_del_amax"][0]


def test_every_bf16_pattern(golden_dir):
    g = np.load(os.path.join(golden_dir, "exhaustive_bf16.npz"))
    pat = np.arange(65536, dtype=np.uint16)
    for fname in (O.E4M3, O.E5M2):
        for si, s in enumerate(g["scales"]):
            got0 = O.cast_to_fp8(pat, O.BF16, s, fname, O.BF16)
            got1 = O.cast_to_fp8(pat, O.BF16, s, fname, O.FP32)
            assert nan_class_equal(got0, g[f"{fname}_{si}_dim0"]), (fname, s)
            assert nan_class_equal(got1, g[f"{fname}_{si}_dim1"]), (fname, s)


def test_scale_of_every_amax_pattern(golden_dir):
    g = np.load(os.path.join(golden_dir, "exhaustive_bf16.npz"))
    pat = np.arange(32768, dtype=np.uint16)
    for dname in (O.BF16, O.FP16):
        for fname in (O.E4M3, O.E5M2):
            got = O.amax_to_scale(O.to_f32(pat, dname), fname, dname, dname)
            ref = g[f"scale_{dname}_{fname}"].view(np.float32)
            same = (got.view(np.uint32) == ref.view(np.uint32)) | (np.isnan(got) & np.isnan(ref))
            assert same.all(), (dname, fname, int((~same).sum()))


def test_fp8_codec_against_torch():
    b = np.arange(256, dtype=np.uint8)
    for fname, tdt in TORCH_F8.items():
        ref = torch.from_numpy(b.copy()).view(tdt).float().numpy()
        got = O.fp8_decode(b, fname)
        assert np.all((ref == got) | (np.isnan(ref) & np.isnan(got)))
        finite = np.isfinite(got)
        assert np.array_equal(O.fp8_encode_rne(got[finite], fname), b[finite])
    g = torch.Generator().manual_seed(3)
    x = torch.randn(100000, generator=g) * torch.exp(4 * torch.randn(100000, generator=g))
    for fname, tdt in TORCH_F8.items():
        f = torch.finfo(tdt).max
        ref = x.clamp(-f, f).to(tdt).view(torch.uint8).numpy()
        assert np.array_equal(O.fp8_encode_rne(np.clip(x.numpy(), -f, f), fname), ref)


def test_sync_matches_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "sync.npz"))
    for dname in (O.BF16, O.FP16, O.FP32):
        amax, hist = g[f"{dname}_amax"], g[f"{dname}_hist"]
        L = amax.shape[1]
        kinds = [O.E4M3] * (2 * L) + [O.E5M2] * L
        scales, hist_after = O.sync_amax_and_scale(amax.reshape(-1), hist.reshape(3 * L, -1), kinds, dname)
        assert np.array_equal(scales.reshape(3, L), g[f"{dname}_scales"]), dname
        # the reference leaves the module histories untouched
        assert np.array_equal(hist_after.reshape(hist.shape), g[f"{dname}_hist_after"])
        assert np.array_equal(g[f"{dname}_hist_after"], hist)


def test_linear_matches_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "linear_small.npz"))
    for dname in (O.BF16, O.FP32):
        r = O.float8_linear_fwd_bwd(g[f"{dname}_x0"], g[f"{dname}_w"], g[f"{dname}_go0"], dname)
        for key in ("y", "dx", "dw"):
            ref = O.to_f32(g[f"{dname}_dyn_{key}"], dname)
            got = r[key]
            # same fp8 operands, fp32 accumulation in a different order
            assert O.sqnr_db(ref, got) > 60.0, (dname, key, O.sqnr_db(ref, got))


def test_delayed_iterations_match_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "linear_small.npz"))
    dname = O.BF16
    names = ("input", "weight", "grad_output")
    kinds = {"input": O.E4M3, "weight": O.E4M3, "grad_output": O.E5M2}
    hist = {n: np.zeros(16, dtype=np.float32) for n in names}
    scale = {n: np.float32(1.0) for n in names}
    amax = {}
    for it in range(3):
        tensors = {"input": g[f"{dname}_x{it}"], "weight": g[f"{dname}_w"], "grad_output": g[f"{dname}_go{it}"]}
        if it == 0:  # first-iteration initialisation from the data
            for n in names:
                a = O.tensor_to_amax(tensors[n], dname)
                amax[n], hist[n], scale[n] = O.init_amax_history(a, hist[n], kinds[n], dname)
        else:  # sync before the forward
            for n in names:
                s, _ = O.sync_amax_and_scale(np.array([amax[n]]), hist[n][None], [kinds[n]], dname)
                scale[n] = s[0]
        for n in names:
            _, amax[n] = O.cast_delayed(tensors[n], dname, scale[n], kinds[n])
            assert amax[n] == g[f"{dname}_del{it}_amax_{n}"][0], (it, n)
            assert scale[n] == g[f"{dname}_del{it}_scale_{n}"][0], (it, n)
            assert np.array_equal(hist[n], g[f"{dname}_del{it}_hist_{n}"]), (it, n)


def test_config1_digests(golden_dir):
    from golden_inputs import config1_inputs, sha256

    g = np.load(os.path.join(golden_dir, "config1.npz"))
    x, w, go = config1_inputs()
    bx = x.view(torch.int16).numpy().view(np.uint16)
    if sha256(bx) != str(g["sha_x"]):
        pytest.skip("torch's CPU generator produced different inputs than when the fixture was made")
    bits, scale, _ = O.cast_dynamic(bx, O.BF16, O.E4M3)
    assert scale == g["scale_x"]
    assert sha256(bits) == str(g["sha_x8"])
    bg = go.view(torch.int16).numpy().view(np.uint16)
    bits, scale, _ = O.cast_dynamic(bg, O.BF16, O.E5M2)
    assert scale == g["scale_g"]
    assert sha256(bits) == str(g["sha_g8"])
