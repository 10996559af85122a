"""Generates the golden fixtures in this directory by running the REFERENCE library
(pytorch-labs/float8_experimental, imported from a checkout) on CPU with emulate=True.

    python tests/golden/make_golden.py /path/to/float8_experimental/checkout

The fixtures pin the oracle (`oracle/f8_oracle.py`) and, through it and directly, the
CUDA kernels.  They are small `.npz` files; bf16/fp16 tensors are stored as uint16 bit
patterns, fp8 tensors as uint8.  Inputs are stored with the outputs, so the tests never
depend on a random-number generator reproducing them.  The one exception is the
4096x4096-layer / 2048-token case, whose inputs (16-32 MB each) are regenerated from fixed
torch seeds; its fixture stores SHA-256 digests of inputs and outputs plus a few
sampled output rows.
"""
from __future__ import annotations

import hashlib
import os
import sys

import numpy as np
import torch

if len(sys.argv) < 2:
    raise SystemExit("usage: make_golden.py /path/to/float8_experimental/checkout")
REF = sys.argv[1]
sys.path.insert(0, REF)
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

import float8_experimental  # noqa: E402
from float8_experimental.config import CastConfig, Float8LinearConfig, ScalingType  # noqa: E402
from float8_experimental.float8_linear import Float8Linear  # noqa: E402
from float8_experimental.float8_linear_utils import sync_float8_amax_and_scale_history  # noqa: E402
from float8_experimental.float8_scaling_utils import (  # noqa: E402
    hp_tensor_to_float8_delayed,
    hp_tensor_to_float8_dynamic,
)
from float8_experimental.float8_tensor import LinearMMConfig  # noqa: E402
from float8_experimental.float8_utils import amax_to_scale, to_fp8_saturated  # noqa: E402

from golden_inputs import config1_inputs, sha256  # noqa: E402

DT = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}
F8 = {"e4m3fn": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}


def bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().contiguous()
    if t.dtype == torch.float32:
        return t.numpy().copy()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        return t.view(torch.uint8).numpy().copy()
    return t.numpy().copy()


def gen_casts():
    """Dynamic and delayed casts on small, odd-shaped tensors of every dtype."""
    g = torch.Generator().manual_seed(1234)
    out = {}
    shapes = [(1, 4), (16, 4), (37, 5), (130, 132), (64, 96), (3, 7, 24)]
    cfg = LinearMMConfig()
    idx = 0
    for dname, dt in DT.items():
        for shape in shapes:
            for fname, f8 in F8.items():
                x = (torch.randn(shape, generator=g) * torch.exp(torch.randn(shape, generator=g))).to(dt)
                if idx % 3 == 0:
                    x.view(-1)[0] = 300.0  # outlier dominating the amax
                if idx % 5 == 0:
                    x.view(-1)[-1] = 0.0
                dyn = hp_tensor_to_float8_dynamic(x, f8, cfg)
                amax_buf = torch.tensor([0.0])
                stored_scale = torch.tensor([float(3.0 + idx)])
                dly = hp_tensor_to_float8_delayed(x, stored_scale, f8, amax_buf, cfg)
                key = f"c{idx}"
                out[key + "_x"] = bits(x)
                out[key + "_meta"] = np.array([dname, fname])
                out[key + "_dyn_bits"] = bits(dyn._data)
                out[key + "_dyn_scale"] = dyn._scale.numpy().copy()
                out[key + "_del_scale"] = stored_scale.numpy().copy()
                out[key + "_del_bits"] = bits(dly._data)
                out[key + "_del_amax"] = amax_buf.numpy().copy()
                idx += 1
    out["n"] = np.array(idx)
    np.savez_compressed(os.path.join(HERE, "casts.npz"), **out)


def gen_exhaustive():
    """Every bf16 bit pattern through both product-rounding routes, several scales."""
    pat = np.arange(65536, dtype=np.uint16)
    x = torch.from_numpy(pat.view(np.int16).copy()).view(torch.bfloat16)
    scales = [1.0, 0.37, 135.0, 1e-3, 19114.0, 3e38]
    out = {"scales": np.array(scales, dtype=np.float32)}
    for fname, f8 in F8.items():
        for si, s in enumerate(scales):
            out[f"{fname}_{si}_dim0"] = bits(to_fp8_saturated(x * torch.tensor(s), f8))
            out[f"{fname}_{si}_dim1"] = bits(to_fp8_saturated(x * torch.tensor([s]), f8))
    # scales for every non-negative bf16 / fp16 amax pattern
    nonneg = np.arange(32768, dtype=np.uint16)
    for dname in ("bf16", "fp16"):
        a = torch.from_numpy(nonneg.view(np.int16).copy()).view(DT[dname])
        for fname, f8 in F8.items():
            out[f"scale_{dname}_{fname}"] = amax_to_scale(a, f8, DT[dname]).numpy().view(np.uint32).copy()
    np.savez_compressed(os.path.join(HERE, "exhaustive_bf16.npz"), **out)


def run_linear(x, w, go, config, iters=1, sync=False, extra_inputs=None):
    lin = torch.nn.Linear(w.shape[1], w.shape[0], bias=False, dtype=w.dtype)
    with torch.no_grad():
        lin.weight.copy_(w)
    m = Float8Linear.from_float(lin, config)
    rec = []
    for it in range(iters):
        xi = (x if it == 0 else extra_inputs[it - 1][0]).clone().requires_grad_(True)
        goi = go if it == 0 else extra_inputs[it - 1][1]
        m.weight.grad = None
        if sync and it > 0:
            sync_float8_amax_and_scale_history(m)
        y = m(xi)
        y.backward(goi)
        item = dict(y=bits(y), dx=bits(xi.grad), dw=bits(m.weight.grad))
        if m.has_any_delayed_scaling:
            for name in ("input", "weight", "grad_output"):
                item[f"amax_{name}"] = getattr(m, f"fp8_amax_{name}").numpy().copy()
                item[f"hist_{name}"] = getattr(m, f"fp8_amax_history_{name}").numpy().copy()
                item[f"scale_{name}"] = getattr(m, f"fp8_scale_{name}").numpy().copy()
        rec.append(item)
    if sync:
        sync_float8_amax_and_scale_history(m)
        final = {}
        for name in ("input", "weight", "grad_output"):
            final[f"amax_{name}"] = getattr(m, f"fp8_amax_{name}").numpy().copy()
            final[f"hist_{name}"] = getattr(m, f"fp8_amax_history_{name}").numpy().copy()
            final[f"scale_{name}"] = getattr(m, f"fp8_scale_{name}").numpy().copy()
        rec.append(final)
    return rec


def gen_linear_small():
    """Float8Linear fwd+bwd (emulate=True) on a small layer: dynamic, and three
    iterations of delayed scaling with a sync between them."""
    g = torch.Generator().manual_seed(77)
    M, K, N = 96, 128, 80
    out = {}
    for dname in ("bf16", "fp32"):
        dt = DT[dname]
        mk = lambda *s, sc=1.0: (torch.randn(*s, generator=g) * sc).to(dt)  # noqa: E731
        xs = [mk(M, K), mk(M, K, sc=3.0), mk(M, K, sc=0.5)]
        gos = [mk(M, N, sc=1e-3), mk(M, N, sc=5e-3), mk(M, N, sc=2e-4)]
        w = mk(N, K, sc=0.02)
        out[f"{dname}_w"] = bits(w)
        for i in range(3):
            out[f"{dname}_x{i}"] = bits(xs[i])
            out[f"{dname}_go{i}"] = bits(gos[i])
        dyn = run_linear(xs[0], w, gos[0], Float8LinearConfig(emulate=True))[0]
        for k, v in dyn.items():
            out[f"{dname}_dyn_{k}"] = v
        dcfg = Float8LinearConfig(
            emulate=True,
            cast_config_input=CastConfig(scaling_type=ScalingType.DELAYED),
            cast_config_weight=CastConfig(scaling_type=ScalingType.DELAYED),
            cast_config_grad_output=CastConfig(scaling_type=ScalingType.DELAYED),
        )
        rec = run_linear(xs[0], w, gos[0], dcfg, iters=3, sync=True, extra_inputs=[(xs[1], gos[1]), (xs[2], gos[2])])
        for it, item in enumerate(rec):
            for k, v in item.items():
                out[f"{dname}_del{it}_{k}"] = v
    np.savez_compressed(os.path.join(HERE, "linear_small.npz"), **out)


def gen_sync():
    """sync_float8_amax_and_scale_history over 5 layers with seeded histories."""
    g = torch.Generator().manual_seed(5)
    L, H = 5, 16
    dcfg = Float8LinearConfig(
        emulate=True,
        cast_config_input=CastConfig(scaling_type=ScalingType.DELAYED),
        cast_config_weight=CastConfig(scaling_type=ScalingType.DELAYED),
        cast_config_grad_output=CastConfig(scaling_type=ScalingType.DELAYED),
    )
    out = {}
    for dname in ("bf16", "fp16", "fp32"):
        model = torch.nn.Sequential(*[torch.nn.Linear(8, 8, bias=False) for _ in range(L)])
        from float8_experimental.float8_linear_utils import convert_to_float8_training

        convert_to_float8_training(model, config=dcfg)
        amax = torch.rand(3, L, generator=g) * torch.tensor([10.0, 0.1, 1e-3]).unsqueeze(1)
        if dname == "fp16":
            amax[2, 0] = 1e-7  # scale would exceed the fp16 range without the clamp
        hist = torch.rand(3, L, H, generator=g) * torch.tensor([10.0, 0.1, 1e-3]).view(3, 1, 1)
        for i, layer in enumerate(model):
            layer.last_seen_input_dtype = DT[dname]
            for k, name in enumerate(("input", "weight", "grad_output")):
                getattr(layer, f"fp8_amax_{name}").fill_(amax[k, i])
                getattr(layer, f"fp8_amax_history_{name}").copy_(hist[k, i])
        sync_float8_amax_and_scale_history(model)
        scales = torch.stack([
            torch.cat([getattr(layer, f"fp8_scale_{name}") for layer in model])
            for name in ("input", "weight", "grad_output")
        ])
        hist_after = torch.stack([
            torch.stack([getattr(layer, f"fp8_amax_history_{name}") for layer in model])
            for name in ("input", "weight", "grad_output")
        ])
        out[f"{dname}_amax"] = amax.numpy().copy()
        out[f"{dname}_hist"] = hist.numpy().copy()
        out[f"{dname}_scales"] = scales.numpy().copy()
        out[f"{dname}_hist_after"] = hist_after.numpy().copy()
    np.savez_compressed(os.path.join(HERE, "sync.npz"), **out)


def gen_config1():
    """Float8Linear(4096, 4096), M = 2048 tokens with outliers, dynamic scaling, emulate."""
    x, w, go = config1_inputs()
    rec = run_linear(x, w, go, Float8LinearConfig(emulate=True))[0]
    cfg = LinearMMConfig()
    x8 = hp_tensor_to_float8_dynamic(x, torch.float8_e4m3fn, cfg)
    w8 = hp_tensor_to_float8_dynamic(w, torch.float8_e4m3fn, cfg)
    g8 = hp_tensor_to_float8_dynamic(go, torch.float8_e5m2, cfg)
    rows = np.array([0, 1, 777, 2047])
    out = dict(
        sha_x=np.array(sha256(bits(x))), sha_w=np.array(sha256(bits(w))), sha_go=np.array(sha256(bits(go))),
        sha_x8=np.array(sha256(bits(x8._data))), sha_w8=np.array(sha256(bits(w8._data))),
        sha_g8=np.array(sha256(bits(g8._data))),
        scale_x=x8._scale.numpy().copy(), scale_w=w8._scale.numpy().copy(), scale_g=g8._scale.numpy().copy(),
        rows=rows,
        y_rows=rec["y"][rows], dx_rows=rec["dx"][rows], dw_rows=rec["dw"][rows],
        sha_y=np.array(sha256(rec["y"])),
    )
    np.savez_compressed(os.path.join(HERE, "config1.npz"), **out)


if __name__ == "__main__":
    torch.manual_seed(0)
    gen_casts()
    gen_exhaustive()
    gen_linear_small()
    gen_sync()
    gen_config1()
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))
