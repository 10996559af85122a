"""Benchmark of the Float8Linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (the headline single-GPU configuration): the four LLaMa-2-70B linear shapes, M = 16384 tokens,
dynamic scaling of input / weight / grad_output, bf16 in and out.  One "step" is one
forward + backward of each of the four `Float8Linear` layers through the public module
API (3 amax reductions, 3 casts, 3 fp8 GEMMs per layer).  FLOPs per layer = 3*2*M*K*N.
Inputs are synthetic (seeded normal draws of the configured scales).

Prints ONE JSON line on rank 0 (see `main`).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M_TOKENS = 16384
SHAPES = [("wqkv", 8192, 10240), ("wo", 8192, 8192), ("w13", 8192, 57344), ("w2", 28672, 8192)]
METRIC = "Float8Linear fwd+bwd TFLOP/s (LLaMa-2-70B shapes); amax+cast HBM GB/s"
NOMINAL_FP8_TFLOPS = 4500.0
NOMINAL_HBM_GBS = 8000.0
# casts also write a transposed fp8 copy only when asked to (the GEMMs read either memory order)
TRANSPOSED_COPIES = os.environ.get("F8B200_CAST_TRANSPOSED", "0") == "1"
# dram__bytes_write of the cast kernel on a 16384x8192 bf16 tensor without the transposed copy
# (profiles/cast_tile8_kernel_16384x8192_bf16.md; 134 MB are written, 78 MB have left L2 at kernel end)
CAST_WRITE_TRAFFIC_1COPY = 78.2e6
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def layer_flops(k: int, n: int, m: int = M_TOKENS) -> float:
    return 3.0 * 2.0 * m * k * n


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {k: float(d[k]) for k in FALLBACK_PEAKS if k in d} | {"source": "measured"}
    return dict(FALLBACK_PEAKS) | {"source": "fallback"}


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, smax, power = [], [], []
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [c.strip() for c in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for nm, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # samples under load: the upper half by power draw
        cut = statistics.median(power)
        loaded = [s for s, p in zip(sm, power) if p >= cut] or sm
        return {"sm_mhz": statistics.median(loaded), "sm_max_mhz": max(smax), "power_w_max": max(power),
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------
# CPU arm: the oracle's restatement of the reference's emulate path
# ---------------------------------------------------------------------------
def cpu_sample_step(sample):
    # C/OpenMP restatement of the casts + numpy BLAS for the three fp32 GEMMs
    from oracle import f8_oracle_c as C

    return C.float8_linear_fwd_bwd(sample["x"], sample["w"], sample["go"], "bf16")


def make_cpu_sample(rows: int = 2048):
    """`rows` tokens of the `wo` layer (K = N = 8192)."""
    import numpy as np

    from oracle import f8_oracle as O

    rng = np.random.default_rng(7)
    k, n = SHAPES[1][1], SHAPES[1][2]
    f = lambda a: O.f32_to_bf16_bits(a.astype(np.float32))  # noqa: E731
    return {"x": f(rng.standard_normal((rows, k))), "w": f(rng.standard_normal((n, k)) * 0.02),
            "go": f(rng.standard_normal((rows, n)) * 1e-3), "rows": rows, "k": k, "n": n,
            "flops": layer_flops(k, n, rows),
            "desc": f"wo layer (K=N=8192) fwd+bwd on {rows} of {M_TOKENS} token rows; port of the emulate=True path "
                    "(casts in C with OpenMP, fp32 GEMMs through numpy BLAS, all host cores)"}


def time_cpu(sample, steps: int, warmup: int):
    for _ in range(warmup):
        cpu_sample_step(sample)
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter()
        cpu_sample_step(sample)
        ts.append(time.perf_counter() - t0)
    return ts


def run_reference_arm(args, rank: int, world: int):
    if rank != 0:
        return
    steps, warmup = max(1, min(args.steps, 10)), max(1, min(args.warmup, 2))
    sample = make_cpu_sample()
    ts = time_cpu(sample, steps, warmup)
    tflops = sample["flops"] / statistics.median(ts) / 1e12
    cores = os.cpu_count() or 1
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": statistics.median(ts) * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp8", "data": "synthetic",
        "config": {"workload": "LLaMa-2-70B linear shapes, M=16384, dynamic scaling (CPU arm: bounded sample)",
                   "sample": sample["desc"]},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample["desc"]},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def measure_delayed(torch, f8, _native, dev, x):
    """Config 3: one batched sync over 320 linears (960 rows, history 16) and the one-pass
    delayed cast (amax + cast + transposed copy) of a [16384, 8192] bf16 activation."""
    from float8_experimental_b200.float8_linear_utils import get_float8_layers

    d = f8.CastConfig(scaling_type=f8.ScalingType.DELAYED)
    cfg = f8.Float8LinearConfig(cast_config_input=d, cast_config_weight=d, cast_config_grad_output=d)
    model = torch.nn.Sequential(*[torch.nn.Linear(16, 16, bias=False, device=dev) for _ in range(320)])
    f8.convert_to_float8_training(model, config=cfg)
    layers = get_float8_layers(model)
    g = torch.Generator(device=dev).manual_seed(3)
    for m in layers:
        m.last_seen_input_dtype = torch.bfloat16
        for name, sigma in (("input", 1.0), ("weight", 0.02), ("grad_output", 1e-3)):
            getattr(m, f"fp8_amax_history_{name}").copy_(torch.randn(16, device=dev, generator=g).abs() * 4 * sigma)
            getattr(m, f"fp8_amax_{name}").copy_(torch.randn(1, device=dev, generator=g).abs() * 4 * sigma)
    for _ in range(3):
        f8.sync_float8_amax_and_scale_history(model, layers)
    torch.cuda.synchronize()
    _native.reset_counters()
    _native.enable_kernel_events(True)
    t0 = time.perf_counter()
    for _ in range(20):
        f8.sync_float8_amax_and_scale_history(model, layers)
    torch.cuda.synchronize()
    wall_us = (time.perf_counter() - t0) / 20 * 1e6
    ev = _native.kernel_event_totals().get("sync", (0.0, 1))
    _native.enable_kernel_events(False)
    # one-pass delayed cast
    from float8_experimental_b200.float8_scaling_utils import hp_tensor_to_float8_delayed

    scale, amax = torch.ones(1, device=dev), torch.zeros(1, device=dev)
    for _ in range(3):
        hp_tensor_to_float8_delayed(x, scale, torch.float8_e4m3fn, amax)
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for _ in range(20):
        hp_tensor_to_float8_delayed(x, scale, torch.float8_e4m3fn, amax)
    s1.record()
    torch.cuda.synchronize()
    cast_ms = s0.elapsed_time(s1) / 20
    return {"sync_rows": 960, "sync_kernel_us": ev[0] / max(ev[1], 1) * 1e3, "sync_launches_per_call": 1,
            "sync_wall_us_per_call": wall_us, "step": measure_delayed_step(torch, f8, dev),
            "delayed_cast_ms_16384x8192": cast_ms,
            "delayed_cast_gbs": (4.0 if TRANSPOSED_COPIES else 3.0) * x.numel() / (cast_ms * 1e-3) / 1e9,
            "delayed_cast_bytes": ("4 B per element: 2 read + 1 fp8 + 1 transposed fp8, amax from the same read"
                                   if TRANSPOSED_COPIES else "3 B per element: 2 read + 1 fp8, amax from the same read")}


def measure_delayed_step(torch, f8, dev, steps: int = 10):
    """The step of the timed region with delayed scaling for all three tensors (the reference's
    third configuration): the same four linears, fwd+bwd, plus one
    sync_float8_amax_and_scale_history over them per step.  Casts are one launch each (the amax
    comes from the cast's own read), so the dynamic step's twelve amax launches disappear."""
    from float8_experimental_b200.float8_linear import Float8Linear

    d = f8.CastConfig(scaling_type=f8.ScalingType.DELAYED)
    cfg = f8.Float8LinearConfig(cast_config_input=d, cast_config_weight=d, cast_config_grad_output=d)
    gen = torch.Generator(device=dev).manual_seed(77)
    layers, xs, gos = [], [], []
    for _, k, n in SHAPES:
        lin = torch.nn.Linear(k, n, bias=False, device=dev, dtype=torch.bfloat16)
        with torch.no_grad():
            lin.weight.normal_(0.0, 0.02, generator=gen)
        layers.append(Float8Linear.from_float(lin, cfg))
        xs.append(torch.randn(M_TOKENS, k, device=dev, dtype=torch.bfloat16, generator=gen).requires_grad_(True))
        gos.append(torch.randn(M_TOKENS, n, device=dev, dtype=torch.bfloat16, generator=gen).mul_(1e-3))
    model = torch.nn.ModuleList(layers)

    def step():
        for layer, x, go in zip(layers, xs, gos):
            x.grad = None
            layer.weight.grad = None
            layer(x).backward(go)
        f8.sync_float8_amax_and_scale_history(model, layers)

    for _ in range(3):
        step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    flops = sum(layer_flops(k, n) for _, k, n in SHAPES)
    return {"ms_per_step": ms, "tflops": flops / (ms * 1e-3) / 1e12, "steps": steps,
            "workload": "the four linears with delayed scaling x3, fwd+bwd, one sync per step"}


def measure_fused_norm(torch, dev, x):
    """RMSNorm fused into the dynamic cast (two launches, 5 B per element: x read twice, fp8
    written once) against the unfused sequence on the same [16384, 8192] bf16 activation: RMSNorm
    in eager mode, then this library's amax and cast kernels."""
    from float8_experimental_b200.float8_scaling_utils import hp_tensor_to_float8_dynamic
    from float8_experimental_b200.float8_tensor import LinearMMConfig
    from float8_experimental_b200.fused_norm import rms_norm_to_float8_dynamic

    w = torch.ones(x.shape[-1], device=dev, dtype=x.dtype)
    cfg = LinearMMConfig()

    def unfused():
        xf = x.float()
        y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)).type_as(x) * w
        return hp_tensor_to_float8_dynamic(y, torch.float8_e4m3fn, cfg)

    def timed(fn):
        for _ in range(3):
            fn()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(20):
            fn()
        s1.record()
        torch.cuda.synchronize()
        return s0.elapsed_time(s1) / 20

    fused_ms = timed(lambda: rms_norm_to_float8_dynamic(x, w, 1e-6))
    unfused_ms = timed(unfused)
    # SwiGLU gate of the LLaMa-2-70B FFN: a, b = halves of the fused w1|w3 output [16384, 57344]
    from float8_experimental_b200.fused_norm import swiglu_to_float8_dynamic

    h = torch.randn(x.shape[0], 57344, device=dev, dtype=x.dtype)
    a, b = h[:, :28672], h[:, 28672:]
    glu_ms = timed(lambda: swiglu_to_float8_dynamic(a, b))
    glu_recompute_ms = timed(lambda: swiglu_to_float8_dynamic(a, b, recompute=True))
    glu_unfused_ms = timed(lambda: hp_tensor_to_float8_dynamic(torch.nn.functional.silu(a) * b, torch.float8_e4m3fn, cfg))
    # backward of the two producers (CUDA kernels) against eager autograd of the same formulas
    from float8_experimental_b200._ops import ops

    rstd, _ = ops.rmsnorm_amax(x, w, 1e-6)
    gy = torch.randn_like(x)
    norm_bwd_ms = timed(lambda: ops.rmsnorm_bwd(x, gy, w, rstd))

    def eager_norm_bwd():
        xr = x.detach().requires_grad_(True)
        wr = w.detach().requires_grad_(True)
        xf = xr.float()
        ((xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)).type_as(xr) * wr).backward(gy)

    norm_bwd_eager_ms = timed(eager_norm_bwd)
    gg = torch.randn(a.shape, device=dev, dtype=x.dtype)
    glu_bwd_ms = timed(lambda: ops.swiglu_bwd(a, b, gg))

    def eager_glu_bwd():
        ar, br = a.detach().requires_grad_(True), b.detach().requires_grad_(True)
        (torch.nn.functional.silu(ar) * br).backward(gg)

    glu_bwd_eager_ms = timed(eager_glu_bwd)
    backward = {"rmsnorm_bwd_ms": norm_bwd_ms, "rmsnorm_bwd_gbs": 6.0 * x.numel() / (norm_bwd_ms * 1e-3) / 1e9,
                "rmsnorm_eager_fwd_bwd_ms": norm_bwd_eager_ms,
                "swiglu_bwd_ms": glu_bwd_ms, "swiglu_bwd_gbs": 10.0 * a.numel() / (glu_bwd_ms * 1e-3) / 1e9,
                "swiglu_eager_fwd_bwd_ms": glu_bwd_eager_ms}
    return {"shape": list(x.shape), "backward": backward,
            "fused_ms": fused_ms, "fused_gbs": 5.0 * x.numel() / (fused_ms * 1e-3) / 1e9,
            "fused_bytes": "5 B per element: 2 read (1/rms + amax pass) + 2 read + 1 fp8 written (cast pass)",
            "unfused_eager_norm_then_cast_ms": unfused_ms,
            "swiglu": {"shape": list(a.shape), "fused_ms": glu_ms, "fused_gbs": 9.0 * a.numel() / (glu_ms * 1e-3) / 1e9,
                       "fused_bytes": "9 B per element: a and b read, gate output written (4 + 2); read back and cast "
                                      "(2 + 1)",
                       "fused_recompute_ms": glu_recompute_ms,
                       "unfused_eager_silu_mul_then_cast_ms": glu_unfused_ms}}


def measure_ffn_fragment(torch, f8, dev):
    """RMSNorm -> w1|w3 -> SwiGLU -> w2 with a residual, forward + backward, at the LLaMa-2-70B FFN
    size (16384 tokens, 8192 -> 2 x 28672 -> 8192; the fragment of the reference's benchmark model):
    the two producers fused into the casts of the float8 linears that follow them, against the
    same float8 linears fed by eager RMSNorm and silu * mul."""
    from float8_experimental_b200.float8_linear import Float8Linear
    from float8_experimental_b200.fused_norm import rms_norm_to_float8_dynamic, swiglu_to_float8_dynamic

    dim, hidden = 8192, 28672
    gen = torch.Generator(device=dev).manual_seed(5)
    mk = lambda i, o: Float8Linear.from_float(  # noqa: E731
        torch.nn.Linear(i, o, bias=False, device=dev, dtype=torch.bfloat16), f8.Float8LinearConfig())
    w13, w2 = mk(dim, 2 * hidden), mk(hidden, dim)
    nw = torch.ones(dim, device=dev, dtype=torch.bfloat16, requires_grad=True)
    x = torch.randn(M_TOKENS, dim, device=dev, dtype=torch.bfloat16, generator=gen).requires_grad_(True)
    go = torch.randn(M_TOKENS, dim, device=dev, dtype=torch.bfloat16, generator=gen).mul_(1e-3)

    def fused():
        h = w13(rms_norm_to_float8_dynamic(x, nw, 1e-6, linear_mm_config=w13.linear_mm_config))
        y = x + w2(swiglu_to_float8_dynamic(h[:, :hidden], h[:, hidden:], linear_mm_config=w2.linear_mm_config))
        y.backward(go)

    def unfused():
        xf = x.float()
        n = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)).type_as(x) * nw
        h = w13(n)
        y = x + w2(torch.nn.functional.silu(h[:, :hidden]) * h[:, hidden:])
        y.backward(go)

    out = {"shape": {"tokens": M_TOKENS, "dim": dim, "hidden": hidden}}
    for name, fn in (("fused_ms", fused), ("unfused_ms", unfused)):
        for _ in range(2):
            x.grad = nw.grad = w13.weight.grad = w2.weight.grad = None
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(5):
            x.grad = nw.grad = w13.weight.grad = w2.weight.grad = None
            fn()
        e1.record()
        torch.cuda.synchronize()
        out[name] = e0.elapsed_time(e1) / 5
    return out


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def run_gpu_arm(args, rank: int, local_rank: int, world: int):
    import torch
    import torch.distributed as dist

    import float8_experimental_b200 as f8
    from float8_experimental_b200 import _native
    from float8_experimental_b200.float8_linear import Float8Linear

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    _native.load()
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    gen = torch.Generator(device=dev).manual_seed(1234 + rank)  # activations differ per rank
    wgen = torch.Generator(device=dev).manual_seed(99)           # weights are the same everywhere
    # N > 1: FSDP2 over the ranks.  Every weight is sharded on dim 0, cast to e4m3 shard by
    # shard and all-gathered as 1 byte per element before forward and again before backward;
    # gradients are reduce-scattered in bf16; after the step ONE all-reduce refreshes all
    # weight scales (precompute_float8_dynamic_scale_for_fsdp).  Tokens per GPU stay fixed.
    fsdp = world > 1
    cfg = f8.Float8LinearConfig(enable_fsdp_float8_all_gather=fsdp)
    layers, xs, gos, host = [], [], [], []
    shapes = [s for s in SHAPES if args.layers is None or s[0] in args.layers.split(",")]
    for name, k, n in shapes:
        lin = torch.nn.Linear(k, n, bias=False, device=dev, dtype=torch.bfloat16)
        with torch.no_grad():
            lin.weight.normal_(0.0, 0.02, generator=wgen)
        layers.append(Float8Linear.from_float(lin, cfg))
        xs.append(torch.randn(M_TOKENS, k, device=dev, dtype=torch.bfloat16, generator=gen).requires_grad_(True))
        gos.append(torch.randn(M_TOKENS, n, device=dev, dtype=torch.bfloat16, generator=gen).mul_(1e-3))

    class _Layers(torch.nn.Module):
        """The four independent linears under one module; with --fsdp-root 1 it becomes the FSDP2
        root, so that the layers share one communication context and the next layer's all-gather
        is prefetched."""

        def __init__(self, mods):
            super().__init__()
            self.mods = torch.nn.ModuleList(mods)

        def forward(self, inputs):
            return [m(x) for m, x in zip(self.mods, inputs)]

    holder = _Layers(layers)
    if fsdp:
        from torch.distributed.fsdp import fully_shard

        for layer in layers:
            fully_shard(layer)
        if args.fsdp_root:
            fully_shard(holder)
        f8.precompute_float8_dynamic_scale_for_fsdp(holder)

    def step():
        for layer, x in zip(layers, xs):
            x.grad = None
            layer.weight.grad = None
        if fsdp and args.fsdp_root:
            torch.autograd.backward(holder(xs), gos)
            f8.precompute_float8_dynamic_scale_for_fsdp(holder)
        elif fsdp:
            for layer, x, go in zip(layers, xs, gos):
                layer(x).backward(go)
            f8.precompute_float8_dynamic_scale_for_fsdp(holder)
        else:
            for layer, x, go in zip(layers, xs, gos):
                layer(x).backward(go)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing -------------------------------------------
    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    _native.reset_counters()
    _native.enable_kernel_events(True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    _native.enable_kernel_events(False)
    clocks = sampler.stop() if rank == 0 else None
    ms_total = e0.elapsed_time(e1)
    launches = _native.launch_count()
    kernel_ms = _native.kernel_event_totals()  # {"gemm": (ms, calls), "cast": ..., "amax": ...}
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = t.item()
    ms_per_step = ms_total / args.steps
    flops_per_step = sum(layer_flops(k, n) for _, k, n in shapes)
    value = world * flops_per_step / (ms_per_step * 1e-3) / 1e12
    if args.kernel_only:
        if rank == 0:
            print(json.dumps({"kernel_only": True, "layers": [s[0] for s in shapes], "value": value,
                              "unit": "TFLOP/s", "ms_per_step": ms_per_step, "kernel_ms": kernel_ms}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- end to end: pinned host inputs, H2D per step, D2H of a result ------
    for x, go in zip(xs, gos):
        host.append((torch.empty(x.shape, dtype=x.dtype, pin_memory=True).copy_(x.detach()),
                     torch.empty(go.shape, dtype=go.dtype, pin_memory=True).copy_(go)))
    result_host = torch.empty(len(shapes), 8, dtype=torch.bfloat16, pin_memory=True)
    copy_stream = torch.cuda.Stream(device=dev)
    h2d_bytes = sum(hx.numel() * 2 + hg.numel() * 2 for hx, hg in host)
    d2h_bytes = result_host.numel() * 2

    def e2e_step():
        main = torch.cuda.current_stream()
        ready = []
        copy_stream.wait_stream(main)  # previous step's readers are done with the buffers
        with torch.cuda.stream(copy_stream):
            for (hx, hg), x, go in zip(host, xs, gos):
                x.detach().copy_(hx, non_blocking=True)
                go.copy_(hg, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(copy_stream)
                ready.append(ev)
        if fsdp:
            for ev in ready:
                main.wait_event(ev)
            step()
        for i, (layer, x, go) in enumerate(zip(layers, xs, gos)):
            if not fsdp:
                main.wait_event(ready[i])
                x.grad = None
                layer.weight.grad = None
                layer(x).backward(go)
            g = layer.weight.grad
            g = g.to_local() if hasattr(g, "to_local") else g  # FSDP2 hands out DTensor gradients
            result_host[i].copy_(g[0, :8], non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller reads the result

    e2e_steps = max(1, min(args.steps, 5))
    e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = t.item()
    e2e_value = world * flops_per_step / e2e_s / 1e12

    # ---- delayed-scaling side measurements (the delayed-scaling configuration: 320 linears, history 16), outside the timed region ----
    # Side measurements never cost the headline line: a failure is recorded in their place.
    def side(fn, *a):
        try:
            return fn(*a)
        except Exception as exc:  # noqa: BLE001
            torch.cuda.synchronize()
            return {"error": f"{type(exc).__name__}: {exc}"[:300]}

    delayed = None
    if rank == 0 and world == 1:
        delayed = side(measure_delayed, torch, f8, _native, dev, xs[0].detach())
    fused_norm = None
    if rank == 0 and world == 1 and shapes[0][1] == 8192:
        fused_norm = side(measure_fused_norm, torch, dev, xs[0].detach())
        if args.layers is None and "error" not in fused_norm:
            fused_norm["ffn_fragment"] = side(measure_ffn_fragment, torch, f8, dev)

    # ---- library kernel to beat, outside every timed region -----------------
    cublaslt = None
    if rank == 0:
        try:
            k, n = SHAPES[1][1], SHAPES[1][2]
            a = torch.randn(M_TOKENS, k, device=dev).to(torch.float8_e4m3fn)
            b = torch.randn(n, k, device=dev).to(torch.float8_e4m3fn)
            one = torch.tensor(1.0, device=dev)
            f = lambda: torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16, use_fast_accum=True)  # noqa: E731
            for _ in range(3):
                f()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            for _ in range(10):
                f()
            s1.record()
            torch.cuda.synchronize()
            cublaslt = 2.0 * M_TOKENS * k * n / (s0.elapsed_time(s1) / 10 * 1e-3) / 1e12
            del a, b
        except Exception as e:  # pragma: no cover
            cublaslt = f"unavailable: {e}"

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = load_peaks()
    gemm_ms, gemm_calls = kernel_ms.get("gemm", (0.0, 0))
    cast_ms, cast_calls = kernel_ms.get("cast", (0.0, 0))
    amax_ms, amax_calls = kernel_ms.get("amax", (0.0, 0))
    gemm_flops = args.steps * flops_per_step
    gemm_tflops = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
    fp8_peak = 2.0 * peaks["bf16_tflops_sustained"]
    # dynamic amax+cast of n bf16 elements: 2n (amax read) + 2n (cast read) + n (fp8) bytes, + n when the
    # transposed copy is emitted too (F8B200_CAST_TRANSPOSED=1; off by default: the GEMMs read
    # operands in either memory order).  Under FSDP2 each rank casts 1/world of every weight and
    # the weight amaxes come from one multi-tensor launch.
    per_elem = 6.0 if TRANSPOSED_COPIES else 5.0
    act_elems = sum(M_TOKENS * k + M_TOKENS * n for _, k, n in shapes)
    w_elems = sum(n * k for _, k, n in shapes)
    cast_bytes = args.steps * (per_elem * act_elems + (5.0 * w_elems / world if fsdp else per_elem * w_elems))
    if fsdp and args.fsdp_root:
        # non-root FSDP2 modules reshard after forward: the shard is cast again for the backward all-gather
        cast_bytes += args.steps * 3.0 * w_elems / world
    cast_gbs = cast_bytes / ((cast_ms + amax_ms) * 1e-3) / 1e9 if (cast_ms + amax_ms) > 0 else None

    # bounded CPU sample (rank 0, N = 1 only)
    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        sample = make_cpu_sample()
        ts = time_cpu(sample, 6, 1)
        cpu_baseline = {"value": sample["flops"] / min(ts) / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count() or 1,
                        "kind": "port", "sample": sample["desc"]}

    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8", "data": "synthetic",
        "config": {
            "workload": "LLaMa-2-70B linear shapes (wqkv, wo, w13, w2), M=16384 tokens per GPU, Float8Linear fwd+bwd, "
                        "dynamic scaling, bf16 in/out",
            "shapes_KN": {name: [k, n] for name, k, n in shapes},
            "l2": "inputs larger than L2 (smallest tensor cast per layer is 134 MB; L2 is 126 MB)",
            "parallelism": (f"fsdp2 x{world}: " + (
                "one root, fp8 weight all-gather (1 B/elem) before forward and again before backward, "
                if args.fsdp_root else
                "each layer its own FSDP2 root (a root keeps its gathered weight for backward): one fp8 weight "
                "all-gather (1 B/elem) per layer and step, ") + "bf16 grad reduce-scatter, one amax all-reduce per step")
            if fsdp else "single GPU",
        },
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                "ms_per_step": e2e_s * 1e3},
        "gpu_launches": launches,
        "roofline": {
            "kernel": ("gemm_fp8_pair_kernel (K < 16384; tcgen05.mma.cta_group::2) + " +
                       ("gemm_fp8_mc_kernel (K >= 16384; 2x1 clusters of 256x256 tiles, B multicast)"
                        if _native._mc_cluster(16384, 8192, 16384) is not None else
                        "gemm_fp8_wide_kernel (K >= 16384; cta_group::1, 256x256 per CTA)") + ", kind::f8f6f4"),
            "bound": "tensor", "achieved": gemm_tflops,
            "peak": fp8_peak, "unit": "TFLOP/s", "frac": (gemm_tflops / fp8_peak) if gemm_tflops else None,
            "peak_source": f"2 x bf16_tflops_sustained of {peaks['source']} MEASURED_PEAKS (fp8 issues at twice the bf16 rate)",
            "frac_of_nominal_4500": (gemm_tflops / NOMINAL_FP8_TFLOPS) if gemm_tflops else None,
            "launches": gemm_calls,
            # dram__bytes_read + dram__bytes_write per launch, mean of the three GEMMs of the wo layer (fwd and dgrad
            # 16384x8192x8192 on the pair kernel, wgrad 8192x8192x16384 on the multicast kernel; 0.881 GB read on the wide kernel), from the ncu captures
            # summarised in profiles/gemm_fp8_pair_kernel_wo_16384x8192x8192.md and
            # profiles/gemm_fp8_wide_kernel_wo_w2_w13.md
            "traffic": (0.346e9 + 0.249e9 + 0.425e9 + 0.249e9 + 0.820e9 + 0.120e9) / 3,
            "traffic_algorithmic": (2 * (201.3e6 + 268.4e6) + (268.4e6 + 134.2e6)) / 3,
        },
        "roofline_cast": {
            "kernel": "amax_flat_kernel + cast_tile8_kernel (dynamic amax+cast with transposed copy)", "bound": "hbm",
            "achieved": cast_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": (cast_gbs / peaks["hbm_gbs"]) if cast_gbs else None,
            "frac_of_nominal_8000": (cast_gbs / NOMINAL_HBM_GBS) if cast_gbs else None,
            "algorithmic_bytes": ("6 bytes per bf16 element (2 amax read + 2 cast read + 1 fp8 + 1 transposed fp8)"
                                  if TRANSPOSED_COPIES else
                                  "5 bytes per bf16 element (2 amax read + 2 cast read + 1 fp8; no transposed copy)"),
            "launches": cast_calls + amax_calls,
            # one 16384x8192 bf16 tensor, amax + cast launches, from profiles/cast_tile8_kernel_16384x8192_bf16.md
            "traffic": 268.4e6 + 268.5e6 + (211.9e6 if TRANSPOSED_COPIES else CAST_WRITE_TRAFFIC_1COPY),
            "traffic_algorithmic": (6 if TRANSPOSED_COPIES else 5) * 134.2e6,
        },
        "time_share_ms_per_step": {"gemm": gemm_ms / args.steps, "cast": cast_ms / args.steps,
                                   "amax": amax_ms / args.steps},
        "cublaslt_fp8_tflops_wo_fwd": cublaslt,
        "delayed_scaling": delayed,
        "fused_rmsnorm_cast": fused_norm,
        "cpu_baseline": cpu_baseline,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_gemm_sweep(args):
    """Sustained per-shape comparison of GEMM variants in ONE process (box-to-box variation is
    larger than the differences between variants): every GEMM of the step runs for ~0.6 s with
    each variant in turn.  Variants: 2cta, 1cta, wide (kernels of libf8b200.so), mc21 / mc22 / mc41
    (the single-GPU multicast library: wide tiles in 2x1 / 2x2 clusters, two CTA pairs), auto (the default choice), cublaslt (torch._scaled_mm);
    suffix -static = fixed tile stride, -direct = per-thread store epilogue."""
    import torch

    from float8_experimental_b200 import _native as N

    dev = torch.device("cuda", 0)
    variants = args.gemm_sweep.split(",")
    shapes = [s for s in SHAPES if args.layers is None or s[0] in args.layers.split(",")]
    one = torch.tensor(1.0, device=dev)
    rows, totals = [], {v: 0.0 for v in variants}

    def sustained(fn, seconds=0.6):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record(); torch.cuda.synchronize()
        iters = max(3, int(seconds * 1e3 / e0.elapsed_time(e1)))
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    for name, k_in, n_out in shapes:
        for tag, m, n, k, a_dt in ((".fwd", M_TOKENS, n_out, k_in, torch.float8_e4m3fn),
                                   (".dgrad", M_TOKENS, k_in, n_out, torch.float8_e5m2),
                                   (".wgrad", n_out, k_in, M_TOKENS, torch.float8_e5m2)):
            a = torch.randn(m, k, device=dev).to(a_dt)
            b = torch.randn(n, k, device=dev).to(torch.float8_e4m3fn)
            out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
            row = {"gemm": name + tag, "m": m, "n": n, "k": k}
            for v in variants:
                if v == "cublaslt":
                    fn = lambda: torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)  # noqa: E731
                else:
                    base = v.split("-")[0]
                    os.environ["F8B200_GEMM_MC"] = base[2:] if base.startswith("mc") else "0"
                    os.environ["F8B200_GEMM_MODE"] = "" if base in ("auto", "mc21", "mc22", "mc41") else base
                    os.environ["F8B200_GEMM_STORE"] = "direct" if v.endswith("-direct") else "tma"
                    os.environ["F8B200_GEMM_WS"] = "0" if v.endswith("-static") else "1"
                    if base == "auto":
                        os.environ.pop("F8B200_GEMM_MC", None)
                    fn = lambda: N.gemm_fp8(a, k, b, k, one, one, None, out, n, m, n, k, False)  # noqa: E731
                ms = sustained(fn)
                totals[v] += ms
                row[v] = {"ms": round(ms, 4), "tflops": round(2.0 * m * n * k / ms / 1e9, 1)}
            rows.append(row)
            print(json.dumps(row), flush=True)
            del a, b, out
    print(json.dumps({"gemm_sweep_totals_ms": {v: round(t, 3) for v, t in totals.items()},
                      "device_error": N.read_device_error()}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--layers", default=None, help="comma list out of wqkv,wo,w13,w2 (default: all four)")
    ap.add_argument("--fsdp-root", type=int, default=1,
                    help="N > 1: 1 = the four layers are children of one FSDP2 root (they reshard after forward, so "
                         "every weight is cast and all-gathered before forward and again before backward, and the "
                         "next layer's all-gather is prefetched under the current layer's GEMMs); 0 = each layer is "
                         "its own root (a root keeps its gathered weight: one all-gather per layer and step, nothing "
                         "overlaps).  Measured at N=8: 41.0 against 41.2 ms/step.")
    ap.add_argument("--gemm-sweep", default=None,
                    help="comma list of GEMM variants to compare per shape in one process (see run_gemm_sweep); "
                         "prints one JSON line per GEMM and the totals, then exits")
    ap.add_argument("--kernel-only", action="store_true",
                    help="device-timed part only, short JSON; for profiler captures of a small case")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gemm_sweep:
        run_gemm_sweep(args)
        return
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    if args.warmup < 3 and not args.kernel_only:
        args.warmup = 3
    run_gpu_arm(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
