"""Side measurements of the single-GPU benchmark (everything here runs OUTSIDE the headline timed
region of `bench.py` and only on CUDA): the delayed-scaling configuration, the fused producers,
the FFN fragment, the per-shape GEMM comparison with cuBLASLt, the sustained fp8 rate of the
library GEMM, and the reference's GPU operator sequence for the same layers.

Counterparts in the reference: benchmarks/bench_linear_float8.py (per-shape fwd+bwd timing, TFLOP
convention :73-77), benchmarks/bench_matmul.py (GEMM against the library), benchmarks/
profile_linear_float8.py (the norm -> linear fragments)."""
from __future__ import annotations

import os
import statistics
import time

M_TOKENS = 16384
SHAPES = [("wqkv", 8192, 10240), ("wo", 8192, 8192), ("w13", 8192, 57344), ("w2", 28672, 8192)]
TRANSPOSED_COPIES = os.environ.get("F8B200_CAST_TRANSPOSED", "0") == "1"


def layer_flops(k: int, n: int, m: int = M_TOKENS) -> float:
    return 3.0 * 2.0 * m * k * n


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
    glu_approx_ms = timed(lambda: swiglu_to_float8_dynamic(a, b, approx_gate=True))
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
    glu_bwd_approx_ms = timed(lambda: ops.swiglu_bwd(a, b, gg, True))

    def eager_glu_bwd():
        ar, br = a.detach().requires_grad_(True), b.detach().requires_grad_(True)
        (torch.nn.functional.silu(ar) * br).backward(gg)

    glu_bwd_eager_ms = timed(eager_glu_bwd)
    backward = {"rmsnorm_bwd_ms": norm_bwd_ms, "rmsnorm_bwd_gbs": 6.0 * x.numel() / (norm_bwd_ms * 1e-3) / 1e9,
                "rmsnorm_eager_fwd_bwd_ms": norm_bwd_eager_ms,
                "swiglu_bwd_ms": glu_bwd_ms, "swiglu_bwd_gbs": 10.0 * a.numel() / (glu_bwd_ms * 1e-3) / 1e9,
                "swiglu_bwd_approx_gate_ms": glu_bwd_approx_ms,
                "swiglu_eager_fwd_bwd_ms": glu_bwd_eager_ms}
    return {"shape": list(x.shape), "backward": backward,
            "fused_ms": fused_ms, "fused_gbs": 5.0 * x.numel() / (fused_ms * 1e-3) / 1e9,
            "fused_bytes": "5 B per element: 2 read (1/rms + amax pass) + 2 read + 1 fp8 written (cast pass)",
            "unfused_eager_norm_then_cast_ms": unfused_ms,
            "swiglu": {"shape": list(a.shape), "fused_ms": glu_ms, "fused_gbs": 9.0 * a.numel() / (glu_ms * 1e-3) / 1e9,
                       "fused_bytes": "9 B per element: a and b read, gate output written (4 + 2); read back and cast "
                                      "(2 + 1)",
                       "fused_recompute_ms": glu_recompute_ms,
                       "fused_approx_gate_ms": glu_approx_ms,
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




_NVML_HANDLES = {}


def _sm_clock_mhz(torch):
    """Current SM clock of torch's current device read through NVML (a query; nothing is set), or None."""
    dev = torch.cuda.current_device()
    if dev not in _NVML_HANDLES:
        try:
            import pynvml

            pynvml.nvmlInit()
            uuid = "GPU-" + str(torch.cuda.get_device_properties(dev).uuid)
            _NVML_HANDLES[dev] = (pynvml, pynvml.nvmlDeviceGetHandleByUUID(uuid))
        except Exception:  # noqa: BLE001
            _NVML_HANDLES[dev] = None
    entry = _NVML_HANDLES[dev]
    if entry is None:
        return None
    try:
        return float(entry[0].nvmlDeviceGetClockInfo(entry[1], entry[0].NVML_CLOCK_SM))
    except Exception:  # noqa: BLE001
        return None


def _sustained_ms(torch, fn, seconds: float = 0.6, clock_samples=None) -> float:
    """Mean time of `fn` repeated back to back for about `seconds` (power-capped parts settle at
    their sustained clock within a fraction of a second), CUDA events on the current stream.
    With `clock_samples` (a list) the SM clock is read every 20 ms while the queued work runs."""
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    iters = max(3, int(seconds * 1e3 / max(e0.elapsed_time(e1), 1e-3)))
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    if clock_samples is not None:
        while not e1.query():
            mhz = _sm_clock_mhz(torch)
            if mhz is None:
                break
            clock_samples.append(mhz)
            time.sleep(0.02)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def gemm_products(shapes=None):
    """The GEMMs of one step: (name, m, n, k, fp8 format of A) for forward, dgrad and wgrad of each layer."""
    import torch

    out = []
    for name, k_in, n_out in (shapes or SHAPES):
        out.append((name + ".fwd", M_TOKENS, n_out, k_in, torch.float8_e4m3fn))
        out.append((name + ".dgrad", M_TOKENS, k_in, n_out, torch.float8_e5m2))
        out.append((name + ".wgrad", n_out, k_in, M_TOKENS, torch.float8_e5m2))
    return out


def gemm_sweep(variants, shapes=None, seconds: float = 0.6, emit=None):
    """Sustained per-shape comparison of GEMM variants in ONE process (box-to-box variation is
    larger than the differences between variants): every GEMM of the step runs for `seconds` with
    each variant in turn.  Variants: 2cta, pw, 1cta, wide (kernels of libf8b200.so), mc21 / mc22 /
    mc41 (the single-GPU multicast library), auto (the default choice), cublaslt (torch._scaled_mm);
    suffix -static = fixed tile stride, -direct = per-thread store epilogue, -tma / -smem = TMA-store epilogue /
    warp-written whole lines after staging in shared memory (default: TMA stores).  Returns (rows,
    totals_ms); `emit(row)` is called per GEMM.  Every entry also carries the median SM clock read while
    it ran ("sm_mhz"), so that time x clock (cycles) can be compared where the power limit moves the clock."""
    import torch

    from .. import _native as N

    dev = torch.device("cuda", torch.cuda.current_device())
    one = torch.tensor(1.0, device=dev)
    rows, totals = [], {v: 0.0 for v in variants}
    saved = {k: os.environ.get(k) for k in ("F8B200_GEMM_MC", "F8B200_GEMM_MODE", "F8B200_GEMM_STORE", "F8B200_GEMM_WS")}
    try:
        for name, m, n, k, a_dt in gemm_products(shapes):
            a = torch.randn(m, k, device=dev).to(a_dt)
            b = torch.randn(n, k, device=dev).to(torch.float8_e4m3fn)
            out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
            row = {"gemm": name, "m": m, "n": n, "k": k}
            for v in variants:
                if v == "cublaslt":
                    fn = lambda: torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)  # noqa: E731
                else:
                    base = v.split("-")[0]
                    os.environ["F8B200_GEMM_MC"] = base[2:] if base.startswith("mc") else "0"
                    os.environ["F8B200_GEMM_MODE"] = "" if base in ("auto", "mc21", "mc22", "mc41") else base
                    os.environ["F8B200_GEMM_STORE"] = ("direct" if v.endswith("-direct") else
                                                       "tma" if v.endswith("-tma") else "smem" if v.endswith("-smem") else "")
                    os.environ["F8B200_GEMM_WS"] = "0" if v.endswith("-static") else "1"
                    if base == "auto":
                        os.environ.pop("F8B200_GEMM_MC", None)
                    fn = lambda: N.gemm_fp8(a, k, b, k, one, one, None, out, n, m, n, k, False)  # noqa: E731
                clocks = []
                ms = _sustained_ms(torch, fn, seconds, clocks)
                totals[v] += ms
                row[v] = {"ms": round(ms, 4), "tflops": round(2.0 * m * n * k / ms / 1e9, 1)}
                if clocks:
                    row[v]["sm_mhz"] = statistics.median(clocks)
            rows.append(row)
            if emit is not None:
                emit(row)
            del a, b, out
    finally:
        for k_, v_ in saved.items():
            if v_ is None:
                os.environ.pop(k_, None)
            else:
                os.environ[k_] = v_
    return rows, {v: round(t, 3) for v, t in totals.items()}


def measure_gemm_vs_cublaslt(seconds: float = 0.35):
    """The twelve GEMMs of the step, this library's default kernel choice against cuBLASLt
    (`torch._scaled_mm`, the kernel the reference calls: float8_python_api.py:43-63), sustained,
    same process, same operands."""
    rows, totals = gemm_sweep(["auto", "cublaslt"], seconds=seconds)
    clocked = all("sm_mhz" in r[v] for r in rows for v in ("auto", "cublaslt"))

    def mcycles(v):  # sum over the GEMMs of time x median SM clock while it ran, in millions of SM cycles
        return round(sum(r[v]["ms"] * r[v]["sm_mhz"] for r in rows) / 1e3, 2) if clocked else None

    def mean_mhz(v):  # time-weighted
        return round(sum(r[v]["ms"] * r[v]["sm_mhz"] for r in rows) / sum(r[v]["ms"] for r in rows), 1) if clocked else None

    return {"ours_ms": totals["auto"], "cublaslt_ms": totals["cublaslt"],
            "ours_sm_mhz": mean_mhz("auto"), "cublaslt_sm_mhz": mean_mhz("cublaslt"),
            "ours_mcycles": mcycles("auto"), "cublaslt_mcycles": mcycles("cublaslt"),
            "per_shape_tflops": {r["gemm"]: [r["auto"]["tflops"], r["cublaslt"]["tflops"]] for r in rows},
            "how": f"each GEMM back to back for {seconds} s per variant, CUDA events, bf16 output, K-major operands"}


def measure_fp8_peak(torch, dev, seconds: float = 2.0):
    """Sustained rate of the library fp8 GEMM (cuBLASLt through torch._scaled_mm) on 8192^3, back
    to back for `seconds`: the measured fp8 counterpart of the bf16 figure in MEASURED_PEAKS.json."""
    n = 8192
    a = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
    b = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
    one = torch.tensor(1.0, device=dev)
    ms = _sustained_ms(torch, lambda: torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16),
                       seconds)
    return 2.0 * n ** 3 / ms / 1e9


def _eager_reference_linear_step(torch, x, w, go):
    """The operator sequence the reference's Float8Linear launches on a GPU for one forward +
    backward with dynamic scaling (eager mode), written with plain torch ops:
    amax = max(abs(x)) (float8_utils.py:104); scale = fp8_max / clamp(amax, EPS) (:47-56);
    x * scale, clamp, .to(fp8) (float8_tensor.py:158, float8_utils.py:136-137); the layout
    fix-ups of preprocess_addmm (float8_ops.py:150-153); scale reciprocals and torch._scaled_mm
    (float8_python_api.py:39-63), three times."""
    e4, e5 = torch.float8_e4m3fn, torch.float8_e5m2

    def cast(t, dt):
        fmax = torch.finfo(dt).max
        amax = torch.max(torch.abs(t))
        scale = (fmax / torch.clamp(amax, min=1e-12)).to(torch.float32)
        return (t * scale).clamp(min=-fmax, max=fmax).to(dt), scale

    def mm(a8, sa, b8, sb):  # a row-major, b column-major, inverse scales
        if not a8.is_contiguous():
            a8 = a8.contiguous()
        if b8.stride(0) != 1:
            b8 = b8.t().contiguous().t()
        return torch._scaled_mm(a8, b8, scale_a=sa.reciprocal(), scale_b=sb.reciprocal(), out_dtype=torch.bfloat16)

    x8, sx = cast(x, e4)
    w8, sw = cast(w, e4)
    y = mm(x8, sx, w8.t(), sw)
    g8, sg = cast(go, e5)
    dx = mm(g8, sg, w8, sw)                # grad_output @ W: W [N, K] must become column-major
    dw = mm(g8.t(), sg, x8, sx).t()        # grad_output^T @ x, then transposed back (float8_linear.py:95)
    return y, dx, dw


def measure_reference_gpu_path(torch, dev, steps: int = 5, reference_linear=None):
    """Forward + backward of the four layers through the REFERENCE's GPU path on this GPU: eager
    amax / scale / cast ops, transposed copies, cuBLASLt GEMMs.  `reference_linear(lin)`, when
    given, wraps an nn.Linear in the reference's own Float8Linear (the unmodified module); without
    it the same operator sequence is issued from `_eager_reference_linear_step`."""
    gen = torch.Generator(device=dev).manual_seed(77)
    flops = sum(layer_flops(k, n) for _, k, n in SHAPES)
    per_layer, total = {}, 0.0
    for name, k, n in SHAPES:
        lin = torch.nn.Linear(k, n, bias=False, device=dev, dtype=torch.bfloat16)
        with torch.no_grad():
            lin.weight.normal_(0.0, 0.02, generator=gen)
        x = torch.randn(M_TOKENS, k, device=dev, dtype=torch.bfloat16, generator=gen).requires_grad_(True)
        go = torch.randn(M_TOKENS, n, device=dev, dtype=torch.bfloat16, generator=gen).mul_(1e-3)
        if reference_linear is not None:
            mod = reference_linear(lin)

            def step():
                x.grad = None
                mod.weight.grad = None
                mod(x).backward(go)
        else:
            w = lin.weight.detach()

            def step():
                with torch.no_grad():
                    _eager_reference_linear_step(torch, x.detach(), w, go)

        for _ in range(2):
            step()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        per_layer[name] = e0.elapsed_time(e1) / steps
        total += per_layer[name]
        del lin, x, go
        torch.cuda.empty_cache()
    return {"ms_per_step": total, "tflops": flops / (total * 1e-3) / 1e12, "per_layer_ms": per_layer, "steps": steps,
            "kind": "reference module (Float8Linear of the reference, emulate=False)" if reference_linear is not None
                    else "eager operator sequence of the reference, restated with torch ops",
            "what": "eager abs/max, scale, mul, clamp, .to(fp8), transposed copies, torch._scaled_mm x3 per layer"}


def measure_llama3_8b_linears(torch, dev, steps: int = 3, n_blocks: int = 32, seq: int = 8192, reference_convert=None):
    """The 224 float8 linears of a Llama-3-8B-shaped decoder (32 blocks x 7 linears, seq 8192, batch 1)
    on one GPU, forward + backward: many small layers per step, where the host work per layer counts as
    much as the kernels.  `reference_convert(model)`, when given, converts a second copy of the model with
    the reference's own `convert_to_float8_training` for the same measurement."""
    import float8_experimental_b200 as f8

    from .models import Llama3Block

    per_block = 4096 * 4096 * 2 + 4096 * 1024 * 2 + 3 * 4096 * 14336
    flops = 6.0 * seq * per_block * n_blocks
    g = torch.Generator(device=dev).manual_seed(200)
    x = torch.randn(1, seq, 4096, device=dev, dtype=torch.bfloat16, generator=g).requires_grad_(True)
    go = torch.randn(1, seq, 4096, device=dev, dtype=torch.bfloat16, generator=g) * 1e-3
    out = {"blocks": n_blocks, "linears": 7 * n_blocks, "tokens": seq, "flops_per_step": flops}

    def build():
        torch.manual_seed(11)
        blocks = []
        for _ in range(n_blocks):
            blk = Llama3Block().to(device=dev, dtype=torch.bfloat16)
            for p in blk.parameters():
                torch.nn.init.normal_(p, 0.0, 0.02)
            blocks.append(blk)
        return torch.nn.Sequential(*blocks)

    def timed(model):
        def step():
            x.grad = None
            for p in model.parameters():
                p.grad = None
            model(x).backward(go)

        for _ in range(2):
            step()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        host_ms = (time.perf_counter() - t0) / steps * 1e3  # time to ENQUEUE a step: above the device time = host-bound
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        return {"ms_per_step": ms, "tflops": flops / ms / 1e9, "host_enqueue_ms_per_step": host_ms}

    def timed_graph(model):
        """The same step captured once into a CUDA graph and replayed: no host work per layer."""
        def step():
            model(x).backward(go)

        def clear():
            x.grad = None
            for p in model.parameters():
                p.grad = None

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                clear()
                step()
        torch.cuda.current_stream().wait_stream(side)
        clear()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        for _ in range(2):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        del graph
        clear()
        return {"ms_per_step": ms, "tflops": flops / ms / 1e9}

    model = build()
    f8.convert_to_float8_training(model, config=f8.Float8LinearConfig())
    out["ours"] = timed(model)
    try:
        out["ours_cuda_graph"] = timed_graph(model)
    except Exception as exc:  # noqa: BLE001
        torch.cuda.synchronize()
        out["ours_cuda_graph"] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    os.environ["F8B200_LINEAR_SINGLE_NODE"] = "0"
    try:
        out["ours_general_route"] = timed(model)
    finally:
        os.environ.pop("F8B200_LINEAR_SINGLE_NODE", None)
    del model
    torch.cuda.empty_cache()
    if reference_convert is not None:
        try:
            ref = build()
            reference_convert(ref)
            out["reference_module"] = timed(ref)
            del ref
        except Exception as exc:  # noqa: BLE001
            torch.cuda.synchronize()
            out["reference_module"] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        torch.cuda.empty_cache()
    return out
