"""The C restatement against the numpy oracle and the reference's recorded outputs."""
import os

import numpy as np

from oracle import f8_oracle as O
from oracle import f8_oracle_c as C


def nan_class_equal(a, b):
    an, bn = (a & 0x7F) == 0x7F, (b & 0x7F) == 0x7F
    return bool(np.all((a == b) | (an & bn)))


def test_casts_match_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "casts.npz"))
    for i in range(int(g["n"])):
        dname, fname = [str(s) for s in g[f"c{i}_meta"]]
        bits, scale, _ = C.cast_dynamic(g[f"c{i}_x"], dname, fname)
        assert scale == g[f"c{i}_dyn_scale"] and np.array_equal(bits, g[f"c{i}_dyn_bits"]), (i, dname, fname)
        dbits = C.cast_to_fp8(g[f"c{i}_x"], dname, g[f"c{i}_del_scale"][0], fname, "fp32")
        assert np.array_equal(dbits, g[f"c{i}_del_bits"]), (i, dname, fname)
        assert C.tensor_to_amax(g[f"c{i}_x"], dname) == g[f"c{i}_del_amax"][0]


def test_every_bf16_pattern(golden_dir):
    g = np.load(os.path.join(golden_dir, "exhaustive_bf16.npz"))
    pat = np.arange(65536, dtype=np.uint16)
    for fname in (O.E4M3, O.E5M2):
        for si, s in enumerate(g["scales"]):
            assert nan_class_equal(C.cast_to_fp8(pat, "bf16", s, fname, "bf16"), g[f"{fname}_{si}_dim0"])
            assert nan_class_equal(C.cast_to_fp8(pat, "bf16", s, fname, "fp32"), g[f"{fname}_{si}_dim1"])


def test_against_numpy_oracle_fp32_and_fp16():
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(200000) * np.exp(4 * rng.standard_normal(200000))).astype(np.float32)
    xh = x.astype(np.float16).view(np.uint16)
    for fname in (O.E4M3, O.E5M2):
        for s in (1.0, 3.7, 1e-4):
            assert np.array_equal(C.cast_to_fp8(x, "fp32", s, fname, "fp32"), O.cast_to_fp8(x, O.FP32, s, fname, O.FP32))
            assert np.array_equal(C.cast_to_fp8(xh, "fp16", s, fname, "fp16"), O.cast_to_fp8(xh, O.FP16, s, fname, O.FP16))
        b = np.arange(256, dtype=np.uint8)
        d, r = C.dequant_f32(b, fname, 2.0), O.fp8_decode(b, fname) / np.float32(2.0)
        assert np.all((d == r) | (np.isnan(d) & np.isnan(r)))
    for a in (0.0, 1e-13, 0.3, 448.0, 7e4):
        for dt in (O.BF16, O.FP16, O.FP32):
            av = O.round_f32_to(np.float32(a), dt)
            assert C.amax_to_scale(av, O.E4M3, dt, dt) == O.amax_to_scale(av, O.E4M3, dt, dt)


def test_linear_matches_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "linear_small.npz"))
    for dname in ("bf16", "fp32"):
        r = C.float8_linear_fwd_bwd(g[f"{dname}_x0"], g[f"{dname}_w"], g[f"{dname}_go0"], dname)
        for key in ("y", "dx", "dw"):
            ref = O.to_f32(g[f"{dname}_dyn_{key}"], dname)
            assert O.sqnr_db(ref, O.to_f32(r[key], dname)) > 60.0, (dname, key)
