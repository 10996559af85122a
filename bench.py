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
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# f8b200_gemm_kernel_choice codes
GEMM_KERNEL_NAMES = {0: "gemm_fp8_kernel (one CTA per 128x256 tile)", 1: "gemm_fp8_pair_kernel (CTA pair per 256x256 tile)",
                     2: "gemm_fp8_wide_kernel (one CTA per 256x256 tile)",
                     3: "gemm_fp8_pairwide_kernel (CTA pair per 512x256 tile, cta_group::2, 256x256 accumulator per CTA)"}
GEMM_KERNEL_SHORT = {0: "1cta", 1: "2cta", 2: "wide", 3: "pw"}
# (dram__bytes_read.sum, dram__bytes_write.sum) per launch from ncu captures of single launches at full size
# (one capture per product and kernel, --clock-control none, bf16 output, K-major operands)
GEMM_DRAM_TRAFFIC = {
    "2cta": {"wo.fwd": (0.34e9, 0.25e9), "wo.wgrad": (0.89e9, 0.12e9), "w13.fwd": (2.10e9, 1.86e9),
             "w13.dgrad": (10.46e9, 0.27e9), "w13.wgrad": (4.76e9, 0.93e9), "w2.fwd": (4.00e9, 0.26e9),
             "w2.dgrad": (1.12e9, 0.92e9)},
    "wide": {"wo.fwd": (0.43e9, 0.24e9), "wo.wgrad": (0.88e9, 0.12e9), "w13.fwd": (2.45e9, 1.86e9),
             "w13.dgrad": (6.54e9, 0.26e9), "w13.wgrad": (5.46e9, 0.93e9), "w2.fwd": (2.93e9, 0.26e9),
             "w2.dgrad": (1.34e9, 0.91e9)},
    "pw": {"wqkv.fwd": (0.61e9, 0.32e9), "wqkv.dgrad": (0.81e9, 0.26e9), "wqkv.wgrad": (1.05e9, 0.16e9),
           "wo.fwd": (0.46e9, 0.25e9), "wo.dgrad": (0.45e9, 0.25e9), "wo.wgrad": (0.82e9, 0.13e9),
           "w13.fwd": (2.56e9, 1.90e9), "w13.dgrad": (8.31e9, 0.27e9), "w13.wgrad": (6.38e9, 0.96e9),
           "w2.fwd": (3.69e9, 0.27e9), "w2.dgrad": (1.35e9, 0.94e9), "w2.wgrad": (2.87e9, 0.48e9)},
}
# amax launch read + cast launch read + cast launch write on one 16384 x 8192 bf16 tensor
CAST_DRAM_TRAFFIC = {"plain": (268.4e6, 268.5e6, 78.2e6), "transposed": (268.4e6, 268.5e6, 211.9e6)}


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
# CPU arm: the reference's own emulate=True path (oracle/_ref, the unmodified package) when it is
# there, else the restatement of that path in oracle/ ("port"), on a bounded sample of the workload
# ---------------------------------------------------------------------------
CPU_SAMPLE_ROWS = 2048


def use_all_host_threads() -> int:
    """Launchers (torch.distributed.run) export OMP_NUM_THREADS=1 for their ranks.  The CPU arm runs
    on ONE rank and is meant to use every host core, so the thread-count variables are set before
    numpy / torch / the OpenMP runtime are loaded.  Returns the count asked for."""
    cores = os.cpu_count() or 1
    for var in ("OMP_NUM_THREADS", "MKL_NUM_THREADS", "OPENBLAS_NUM_THREADS"):
        os.environ[var] = str(cores)
    return cores


def reference_package():
    """The unmodified reference package placed under oracle/_ref by oracle/make_ref.py, or None."""
    from oracle import make_ref

    path = make_ref.ref_path()
    if path is None:
        return None
    if path not in sys.path:
        sys.path.insert(0, path)
    try:
        import float8_experimental  # noqa: F401
        from float8_experimental.float8_linear import Float8Linear  # noqa: F401
    except Exception:  # noqa: BLE001
        return None
    return sys.modules["float8_experimental"]


def _cpu_tensors(rows, k, n, seed=7):
    import torch

    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16)
    go = (torch.randn(rows, n, generator=g) * 1e-3).to(torch.bfloat16)
    return x, w, go


def _reference_cpu_step_fn(rows, k, n):
    """fwd+bwd of the reference's Float8Linear(emulate=True), dynamic scaling, on CPU tensors."""
    import torch
    from float8_experimental.config import Float8LinearConfig
    from float8_experimental.float8_linear import Float8Linear

    x, w, go = _cpu_tensors(rows, k, n)
    lin = torch.nn.Linear(k, n, bias=False, dtype=torch.bfloat16)
    with torch.no_grad():
        lin.weight.copy_(w)
    mod = Float8Linear.from_float(lin, Float8LinearConfig(emulate=True))
    x.requires_grad_(True)

    def step():
        x.grad = None
        mod.weight.grad = None
        mod(x).backward(go)

    return step


def _port_cpu_step_fn(rows, k, n):
    """The same step through the restatement: casts in C with OpenMP, fp32 GEMMs through numpy's BLAS."""
    import numpy as np

    from oracle import f8_oracle_c as C

    x, w, go = _cpu_tensors(rows, k, n)
    bits = lambda t: t.view(__import__("torch").int16).numpy().view(np.uint16)  # noqa: E731
    xb, wb, gb = bits(x), bits(w), bits(go)
    return lambda: C.float8_linear_fwd_bwd(xb, wb, gb, "bf16")


def _time_host(step, steps, warmup):
    for _ in range(warmup):
        step()
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter()
        step()
        ts.append(time.perf_counter() - t0)
    return ts


def time_cpu_arm(steps: int, warmup: int, extras: bool = True):
    """Times the CPU arm: `steps` passes (after `warmup`) over the bounded sample, median.  The
    sample is forward + backward of the `wo` layer (K = N = 8192) on 2048 of the 16384 token rows.
    With `extras`: the reference's own CPU-runnable configuration in full (one Float8Linear 4096 ->
    4096, 2048 tokens) and the other implementation of the arm as a cross-check."""
    import torch

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    k, n = SHAPES[1][1], SHAPES[1][2]
    ref = reference_package()
    kind = "reference" if ref is not None else "port"
    step = _reference_cpu_step_fn(CPU_SAMPLE_ROWS, k, n) if ref is not None else _port_cpu_step_fn(CPU_SAMPLE_ROWS, k, n)
    ts = _time_host(step, steps, warmup)
    flops = layer_flops(k, n, CPU_SAMPLE_ROWS)
    med = statistics.median(ts)
    what = ("the reference's Float8Linear (unmodified package, emulate=True, dynamic scaling) on CPU tensors"
            if ref is not None else
            "restatement of the emulate=True path (casts in C with OpenMP, fp32 GEMMs through numpy BLAS)")
    out = {"value": flops / med / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind,
           "sample": f"wo layer (K=N=8192) fwd+bwd on {CPU_SAMPLE_ROWS} of {M_TOKENS} token rows; {what}; "
                     f"median of {steps} after {warmup} warm-up",
           "ms_per_step": med * 1e3, "statistic": "median"}
    if extras:
        try:
            c1 = _reference_cpu_step_fn(2048, 4096, 4096) if ref is not None else _port_cpu_step_fn(2048, 4096, 4096)
            t1 = statistics.median(_time_host(c1, 3, 1))
            out["config1"] = {"what": "Float8Linear(4096, 4096), 2048 tokens, fwd+bwd, whole configuration", "ms": t1 * 1e3,
                              "tflops": layer_flops(4096, 4096, 2048) / t1 / 1e12}
            if ref is not None:
                tp = statistics.median(_time_host(_port_cpu_step_fn(CPU_SAMPLE_ROWS, k, n), 3, 1))
                out["port_cross_check_tflops"] = flops / tp / 1e12
        except Exception as exc:  # noqa: BLE001
            out["extras_error"] = f"{type(exc).__name__}: {exc}"[:200]
    return out


def run_reference_arm(args, rank: int, world: int):
    """`--impl reference`: the CPU arm alone, on rank 0 (the other ranks of a multi-rank launch exit
    without work), honouring --steps / --warmup, with every host thread."""
    if rank != 0:
        return
    cpu = time_cpu_arm(max(1, args.steps), max(0, args.warmup))
    line = {
        "impl": "reference", "metric": METRIC, "value": cpu["value"], "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": max(1, args.steps), "warmup": max(0, args.warmup), "ms_per_step": cpu["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8", "data": "synthetic",
        "config": {"workload": "LLaMa-2-70B linear shapes (wqkv, wo, w13, w2), M=16384 tokens per GPU, Float8Linear "
                               "fwd+bwd, dynamic scaling, bf16 in/out (CPU arm: bounded sample per step)",
                   "sample": cpu["sample"]},
        "cpu_baseline": cpu,
        "e2e": {"value": cpu["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def run_gpu_arm(args, rank: int, local_rank: int, world: int):
    import torch
    import torch.distributed as dist

    import float8_experimental_b200 as f8
    from float8_experimental_b200 import _native
    from float8_experimental_b200.benchmarks import multi_gpu, single_gpu
    from float8_experimental_b200.float8_linear import Float8Linear

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    _native.load()
    parity_n = None
    if world > 1:
        # a short collective timeout: a rank that fails a parity check ends the run with an error within
        # minutes instead of leaving the others waiting for it
        import datetime

        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=240))
        # the sharded paths are checked on the real NCCL / CUDA route before anything is timed
        parity_n = multi_gpu.run_parity(dev, rank, world)
        if any(v != "ok" for v in parity_n.values()):
            if rank == 0:
                print(json.dumps({"metric": METRIC, "n_gpus": world, "parity_n": parity_n,
                                  "error": "multi-GPU parity check failed; nothing was timed"}), flush=True)
            dist.destroy_process_group()
            sys.exit(3)

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
            # --fsdp-reshard 0 (default): the gathered fp8 weight (1 byte per element, 0.94 GB for the four
            # layers) stays for the backward pass instead of being cast and all-gathered a second time
            fully_shard(layer, reshard_after_forward=bool(args.fsdp_reshard))
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
    _native.check_device_error()  # a bounded wait that gave up inside a GEMM voids the run
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

    x_ready, go_ready = [None] * len(layers), [None] * len(layers)
    if fsdp:
        # each layer's forward waits for its own input only (a pre-forward hook on the GPU stream),
        # the backward for the gradients: the copies of later layers overlap the earlier layers' work
        def _make_hook(i):
            def hook(mod, inputs):
                if x_ready[i] is not None:
                    torch.cuda.current_stream().wait_event(x_ready[i])
            return hook

        hook_handles = [layer.register_forward_pre_hook(_make_hook(i)) for i, layer in enumerate(layers)]

    # Without FSDP the layers are independent: each layer's input and gradient are copied together and the
    # layers run in descending order of work, so that what is left to compute after the last copy has
    # landed (the step is bound by the host link) is the smallest layer.  Under the FSDP2 root the forward of
    # all layers precedes the backward: inputs are copied first, gradients after them.
    order = sorted(range(len(layers)), key=lambda i: -layer_flops(shapes[i][1], shapes[i][2]))

    def e2e_step():
        main = torch.cuda.current_stream()
        copy_stream.wait_stream(main)  # previous step's readers are done with the buffers
        with torch.cuda.stream(copy_stream):
            def copy_x(i):
                xs[i].detach().copy_(host[i][0], non_blocking=True)
                x_ready[i] = torch.cuda.Event()
                x_ready[i].record(copy_stream)

            def copy_go(i):
                gos[i].copy_(host[i][1], non_blocking=True)
                go_ready[i] = torch.cuda.Event()
                go_ready[i].record(copy_stream)

            if fsdp and args.fsdp_root:
                for i in range(len(layers)):
                    copy_x(i)
                for i in reversed(range(len(layers))):  # backward runs from the last layer to the first
                    copy_go(i)
            else:
                for i in order:
                    copy_x(i)
                    copy_go(i)
        for layer, x in zip(layers, xs):
            x.grad = None
            layer.weight.grad = None
        if fsdp and args.fsdp_root:
            outs = holder(xs)
            for ev in go_ready:
                main.wait_event(ev)
            torch.autograd.backward(outs, gos)
            f8.precompute_float8_dynamic_scale_for_fsdp(holder)
        else:
            for i in order:
                if not fsdp:
                    main.wait_event(x_ready[i])
                y = layers[i](xs[i])
                main.wait_event(go_ready[i])
                y.backward(gos[i])
            if fsdp:
                f8.precompute_float8_dynamic_scale_for_fsdp(holder)
        for i, layer in enumerate(layers):
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
    _native.check_device_error()
    if fsdp:
        for h in hook_handles:
            h.remove()
        x_ready = [None] * len(layers)

    # ---- side measurements, outside every timed region ----------------------
    # They never cost the headline line: a failure is recorded in their place.
    def side(fn, *a, **kw):
        try:
            return fn(*a, **kw)
        except Exception as exc:  # noqa: BLE001
            torch.cuda.synchronize()
            return {"error": f"{type(exc).__name__}: {exc}"[:300]}

    delayed = fused_norm = gemm_vs_cublaslt = fp8_peak_measured = reference_gpu = llama3_one_gpu = None
    comm_split = tp_sp_ffn = llama3_fsdp = cast_all_gather = None
    full = args.layers is None and not args.quick
    if world == 1 and rank == 0:
        # the delayed-scaling configuration (320 linears, history 16) and the fused producers
        delayed = side(single_gpu.measure_delayed, torch, f8, _native, dev, xs[0].detach())
        if shapes[0][1] == 8192:
            fused_norm = side(single_gpu.measure_fused_norm, torch, dev, xs[0].detach())
            if full and "error" not in fused_norm:
                fused_norm["ffn_fragment"] = side(single_gpu.measure_ffn_fragment, torch, f8, dev)
    if world > 1 and args.layers is None:
        # where the N > 1 step spends its device time (all ranks run the steps, rank 0 profiles)
        if rank == 0:
            comm_split = side(multi_gpu.profile_step_split, step, dev)
        else:
            for _ in range(3):
                step()
            torch.cuda.synchronize()
    # the headline tensors are not needed any more
    del layers, holder, xs, gos, host
    torch.cuda.empty_cache()
    if rank == 0 and full:
        # the library kernels to beat and the reference's own GPU operator sequence
        fp8_peak_measured = side(single_gpu.measure_fp8_peak, torch, dev)
        if world == 1:
            gemm_vs_cublaslt = side(single_gpu.measure_gemm_vs_cublaslt)
            ref_linear = None
            try:
                if reference_package() is not None:
                    from float8_experimental.config import Float8LinearConfig as RefConfig
                    from float8_experimental.float8_linear import Float8Linear as RefLinear

                    ref_linear = lambda lin: RefLinear.from_float(lin, RefConfig())  # noqa: E731
            except Exception:  # noqa: BLE001
                ref_linear = None
            reference_gpu = side(single_gpu.measure_reference_gpu_path, torch, dev, 5, ref_linear)
            if ref_linear is not None and "error" in reference_gpu:
                first_error = reference_gpu["error"]
                reference_gpu = side(single_gpu.measure_reference_gpu_path, torch, dev, 5, None)
                reference_gpu["reference_module_error"] = first_error
            ref_convert = None
            if ref_linear is not None:
                from float8_experimental.float8_linear_utils import convert_to_float8_training as ref_convert
            llama3_one_gpu = side(single_gpu.measure_llama3_8b_linears, torch, dev, 3, 32, 8192, ref_convert)
    if world > 1 and full:
        # the tensor / sequence parallel and the Llama-3-8B FSDP2 configurations (all ranks take part)
        tp_sp_ffn = side(multi_gpu.measure_tp_sp_ffn, dev, rank, world)
        cast_all_gather = side(multi_gpu.measure_cast_all_gather, dev, rank, world)
        llama3_fsdp = side(multi_gpu.measure_fsdp2_llama3_8b_linears, dev, rank, world)
        _native.check_device_error()

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
    fp8_peak = 2.0 * peaks["bf16_tflops_sustained"]  # proxy: MEASURED_PEAKS holds no fp8 figure
    fp8_lib = fp8_peak_measured if isinstance(fp8_peak_measured, float) else None
    # dynamic amax+cast of n bf16 elements: 2n (amax read) + 2n (cast read) + n (fp8) bytes, + n when the
    # transposed copy is emitted too (F8B200_CAST_TRANSPOSED=1; off by default: the GEMMs read
    # operands in either memory order).  Under FSDP2 each rank casts 1/world of every weight and
    # the weight amaxes come from one multi-tensor launch.
    per_elem = 6.0 if TRANSPOSED_COPIES else 5.0
    act_elems = sum(M_TOKENS * k + M_TOKENS * n for _, k, n in shapes)
    w_elems = sum(n * k for _, k, n in shapes)
    cast_bytes = args.steps * (per_elem * act_elems + (5.0 * w_elems / world if fsdp else per_elem * w_elems))
    if fsdp and args.fsdp_root and args.fsdp_reshard:
        # resharding after forward: the shard is cast again for the backward all-gather
        cast_bytes += args.steps * 3.0 * w_elems / world
    cast_gbs = cast_bytes / ((cast_ms + amax_ms) * 1e-3) / 1e9 if (cast_ms + amax_ms) > 0 else None

    # which GEMM kernel the library chose for the products of the step, and its DRAM traffic
    products = single_gpu.gemm_products(shapes)
    chosen = [_native.gemm_kernel_choice(m, n, k) for _, m, n, k, _ in products]
    gemm_kernel_desc = ", ".join(f"{GEMM_KERNEL_NAMES[c]} x{chosen.count(c)}" for c in sorted(set(chosen))) + \
        "; tcgen05.mma kind::f8f6f4, TMA loads and stores, fp32 accumulators in tensor memory"
    known = [GEMM_DRAM_TRAFFIC.get(GEMM_KERNEL_SHORT[c], {}).get(name) for c, (name, *_r) in zip(chosen, products)]
    traffic = sum(r + w for r, w in known) / len(known) if known and all(t is not None for t in known) else None
    traffic_algo = sum(m * k + n * k + 2.0 * m * n for _, m, n, k, _ in products) / len(products)
    traffic_src = ("mean over the GEMM launches of one step of ncu dram__bytes_read.sum + dram__bytes_write.sum per "
                   "launch, one capture per product, for the kernel each product ran on" if traffic is not None else
                   "no capture for this kernel choice")

    # bounded CPU sample (rank 0, N = 1 only): the reference's emulate=True path on the host cores
    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        try:
            cpu_baseline = time_cpu_arm(4, 1, extras=full)
        except Exception as exc:  # noqa: BLE001
            cpu_baseline = {"error": f"{type(exc).__name__}: {exc}"[:300]}

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
                "one root, " if args.fsdp_root else "each layer its own FSDP2 root, ") + (
                "fp8 weight all-gather (1 B/elem) before forward and again before backward, "
                if (args.fsdp_root and args.fsdp_reshard) else
                "one fp8 weight all-gather (1 B/elem) per layer and step (the gathered fp8 weight is kept for backward), ")
                + "bf16 grad reduce-scatter, one amax all-reduce per step")
            if fsdp else "single GPU",
        },
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                "ms_per_step": e2e_s * 1e3},
        "gpu_launches": launches,
        "roofline": {
            "kernel": gemm_kernel_desc,
            "bound": "tensor", "achieved": gemm_tflops,
            "peak": fp8_peak, "unit": "TFLOP/s", "frac": (gemm_tflops / fp8_peak) if gemm_tflops else None,
            "peak_source": f"PROXY: 2 x bf16_tflops_sustained of {peaks['source']} MEASURED_PEAKS (no fp8 figure is "
                           "recorded there; tcgen05 issues fp8 at twice the bf16 rate)",
            "peak_fp8_measured": fp8_lib,
            "peak_fp8_measured_how": "torch._scaled_mm (cuBLASLt) 8192^3 e4m3 x e4m3 -> bf16, back to back for 2 s, this "
                                     "run, outside the timed region",
            "frac_of_peak_fp8_measured": (gemm_tflops / fp8_lib) if (gemm_tflops and fp8_lib) else None,
            "frac_of_nominal_4500": (gemm_tflops / NOMINAL_FP8_TFLOPS) if gemm_tflops else None,
            "launches": gemm_calls,
            "traffic": traffic, "traffic_algorithmic": traffic_algo, "traffic_source": traffic_src,
        },
        "roofline_cast": {
            "kernel": "amax_flat_kernel + cast_tile8_kernel (dynamic amax + cast" +
                      (", with the transposed copy)" if TRANSPOSED_COPIES else ", no transposed copy)"), "bound": "hbm",
            "achieved": cast_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": (cast_gbs / peaks["hbm_gbs"]) if cast_gbs else None,
            "frac_of_nominal_8000": (cast_gbs / NOMINAL_HBM_GBS) if cast_gbs else None,
            "algorithmic_bytes": ("6 bytes per bf16 element (2 amax read + 2 cast read + 1 fp8 + 1 transposed fp8)"
                                  if TRANSPOSED_COPIES else
                                  "5 bytes per bf16 element (2 amax read + 2 cast read + 1 fp8; no transposed copy)"),
            "launches": cast_calls + amax_calls,
            "traffic": sum(CAST_DRAM_TRAFFIC["transposed" if TRANSPOSED_COPIES else "plain"]),
            "traffic_algorithmic": (6 if TRANSPOSED_COPIES else 5) * 134.2e6,
            "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of the amax and the cast launch on one "
                              "16384 x 8192 bf16 tensor",
        },
        "time_share_ms_per_step": {"gemm": gemm_ms / args.steps, "cast": cast_ms / args.steps,
                                   "amax": amax_ms / args.steps},
        "gemm_vs_cublaslt": gemm_vs_cublaslt,
        "reference_gpu_path": reference_gpu,
        "vs_reference_gpu_path": (reference_gpu["ms_per_step"] / ms_per_step
                                  if isinstance(reference_gpu, dict) and "ms_per_step" in reference_gpu else None),
        "llama3_8b_linears": llama3_one_gpu,
        "delayed_scaling": delayed,
        "fused_rmsnorm_cast": fused_norm,
        "cpu_baseline": cpu_baseline,
    }
    if world > 1:
        line["parity_n"] = parity_n
        line["step_split_ms"] = comm_split
        line["tp_sp_ffn"] = tp_sp_ffn
        line["cast_all_gather"] = cast_all_gather
        line["fsdp2_llama3_8b_linears"] = llama3_fsdp
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_gemm_sweep(args):
    """`--gemm-sweep v1,v2,...`: sustained per-shape comparison of GEMM variants in one process
    (`benchmarks.single_gpu.gemm_sweep`); one JSON line per GEMM, then the totals."""
    from float8_experimental_b200 import _native as N
    from float8_experimental_b200.benchmarks import single_gpu

    shapes = [s for s in SHAPES if args.layers is None or s[0] in args.layers.split(",")]
    _, totals = single_gpu.gemm_sweep(args.gemm_sweep.split(","), shapes, emit=lambda row: print(json.dumps(row), flush=True))
    print(json.dumps({"gemm_sweep_totals_ms": totals, "device_error": N.read_device_error()}), flush=True)


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
                         "overlaps)")
    ap.add_argument("--fsdp-reshard", type=int, default=0,
                    help="N > 1: 1 = layers free their gathered fp8 weight after forward and gather it again before "
                         "backward (FSDP2's default for non-root modules); 0 = they keep it until backward")
    ap.add_argument("--quick", action="store_true",
                    help="headline numbers only: skip the side measurements that need extra seconds (GEMM comparison "
                         "with cuBLASLt, the reference's GPU path, the multi-GPU side configurations)")
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
        if rank == 0:
            use_all_host_threads()  # before numpy / torch load their thread pools
            run_reference_arm(args, rank, world)
        return
    if args.warmup < 3 and not args.kernel_only:
        args.warmup = 3
    run_gpu_arm(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
