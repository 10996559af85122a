"""Multi-GPU parts of the benchmark (one process per GPU, NCCL): parity checks of the sharded paths
that run BEFORE anything is timed, and the side measurements of the FSDP2 and tensor / sequence
parallel configurations.  CUDA only; every function is called on all ranks.

Reference counterparts: test/test_fsdp2/test_fsdp2_common.py:17-54 (FSDP2 == unsharded model, loss
for loss), test/test_fsdp2/test_fsdp2.py:348-375 (1 byte per weight element in the all-gather),
test/test_dtensor.py:189-231 (TP and SP == unsharded), float8_linear_utils.py:261-271 (one all-reduce
per sync), benchmarks/bench_multi_gpu.py (FSDP timing)."""
from __future__ import annotations

import copy

import torch
import torch.distributed as dist
import torch.nn as nn


# ---------------------------------------------------------------------------
# small models
# ---------------------------------------------------------------------------
class _MLP(nn.Module):
    def __init__(self, dim=256, hidden=512, n=3):
        super().__init__()
        self.layers = nn.ModuleList(
            [nn.Sequential(nn.Linear(dim, hidden, bias=False), nn.ReLU(), nn.Linear(hidden, dim, bias=False))
             for _ in range(n)]
        )

    def forward(self, x):
        for blk in self.layers:
            x = x + blk(x)
        return x


class FeedForward(nn.Module):
    """SwiGLU feed-forward block: w2(silu(w1(x)) * w3(x))."""

    def __init__(self, dim, hidden):
        super().__init__()
        self.w1 = nn.Linear(dim, hidden, bias=False)
        self.w2 = nn.Linear(hidden, dim, bias=False)
        self.w3 = nn.Linear(dim, hidden, bias=False)

    def forward(self, x):
        return self.w2(nn.functional.silu(self.w1(x)) * self.w3(x))


class _Holder(nn.Module):
    def __init__(self, ffn):
        super().__init__()
        self.ffn = ffn

    def forward(self, x):
        return self.ffn(x)


def _all_gather_cat(t, world, dim):
    outs = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(outs, t.contiguous())
    return torch.cat(outs, dim=dim)


# ---------------------------------------------------------------------------
# parity
# ---------------------------------------------------------------------------
def parity_fsdp2(dev, rank, world):
    """FSDP2 with fp8 weight all-gather + precomputed scales against the unsharded float8 model
    with hand-averaged gradients: equal losses over 3 Adam steps; the block all-gathers carry uint8
    payloads of 1 byte per weight element."""
    from torch.distributed.fsdp import fully_shard

    import float8_experimental_b200 as f8

    torch.manual_seed(42)
    base = _MLP().to(dev)
    ref_model = copy.deepcopy(base)
    f8.convert_to_float8_training(ref_model, config=f8.Float8LinearConfig())
    fsdp_model = copy.deepcopy(base)
    f8.convert_to_float8_training(fsdp_model, config=f8.Float8LinearConfig(enable_fsdp_float8_all_gather=True))
    for blk in fsdp_model.layers:
        fully_shard(blk)
    fully_shard(fsdp_model)
    gathered = []
    real_ag = dist.all_gather_into_tensor

    def counting_ag(out, inp, *a, **k):
        gathered.append((inp.dtype, inp.numel() * inp.element_size()))
        return real_ag(out, inp, *a, **k)

    dist.all_gather_into_tensor = counting_ag
    ref_opt = torch.optim.Adam(ref_model.parameters(), lr=1e-2)
    fsdp_opt = torch.optim.Adam(fsdp_model.parameters(), lr=1e-2)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    try:
        for step in range(3):
            x = torch.randn(64, 256, device=dev, generator=g)
            losses = []
            for model, opt in ((ref_model, ref_opt), (fsdp_model, fsdp_opt)):
                opt.zero_grad()
                loss = model(x).pow(2).sum()
                loss.backward()
                if model is ref_model:
                    for p in model.parameters():
                        dist.all_reduce(p.grad)
                        p.grad.div_(world)
                opt.step()
                if model is fsdp_model:
                    f8.precompute_float8_dynamic_scale_for_fsdp(model)
                losses.append(loss.detach())
            # Two ranks add two numbers: reduce-scatter and all-reduce give the same sums and the losses agree to
            # rounding of the loss itself.  From four ranks on the two collectives add in different orders, the
            # fp32 gradients differ in their last bits, and after an Adam step a few weights fall on the other
            # side of an fp8 rounding boundary: the losses then agree to ~1e-4, not to the last bit.
            rtol = 1e-5 if world <= 2 else 1e-3
            torch.testing.assert_close(losses[0], losses[1], rtol=rtol, atol=0,
                                       msg=f"fsdp2 step {step}: {[float(v) for v in losses]}")
    finally:
        dist.all_gather_into_tensor = real_ag
    per_block = (512 * 256 + 256 * 512) // world
    block_gathers = [x for x in gathered if x[1] == per_block]
    assert len(block_gathers) >= 3 * 3, gathered
    assert all(dt == torch.uint8 for dt, _ in block_gathers), block_gathers
    return "ok"


def parity_tensor_parallel(dev, rank, world, sequence_parallel, cast_all_gather=False, fused_reduce_scatter=False):
    """TP (or SP) float8 FFN == the unsharded float8 FFN: outputs, input gradients and a weight
    gradient.  With `cast_all_gather` the sequence-parallel input goes through the cast whose
    stores are the all-gather (peer memory) instead of cast + NCCL all-gather; with
    `fused_reduce_scatter` the row-parallel GEMM scatters its partial product into the owners'
    buffers (peer memory) instead of GEMM + NCCL reduce-scatter."""
    from torch.distributed._tensor import DTensor, Replicate, Shard
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor.parallel import parallelize_module

    import float8_experimental_b200 as f8
    from float8_experimental_b200.float8_tensor_parallel import (
        Float8ColwiseParallel,
        Float8RowwiseParallel,
        PrepareFloat8ModuleInput,
    )

    mesh = init_device_mesh("cuda", (world,))
    torch.manual_seed(5)
    dim, hidden, batch, seq = 256, 512 * world, 2, 64 * world
    ref = _Holder(FeedForward(dim, hidden)).to(dev)
    f8.convert_to_float8_training(ref, config=f8.Float8LinearConfig())
    tp = copy.deepcopy(ref)
    if sequence_parallel:
        pool = None
        if cast_all_gather:
            from float8_experimental_b200.fp8_all_gather import CastAllGatherPool

            pool = CastAllGatherPool(mesh.get_group(0), max_numel_per_rank=batch * (seq // world) * dim, depth=2)
        rs = None
        if fused_reduce_scatter:
            from float8_experimental_b200.fused_reduce_scatter import GemmReduceScatter

            rs = GemmReduceScatter(mesh.get_group(0), max_out_numel_per_rank=batch * (seq // world) * dim,
                                   dtype=torch.float32)
        plan = {
            "ffn": PrepareFloat8ModuleInput(input_layouts=Shard(1), desired_input_layouts=Replicate(),
                                            cast_all_gather=pool),
            "ffn.w1": Float8ColwiseParallel(),
            "ffn.w2": Float8RowwiseParallel(output_layouts=Shard(1), fused_reduce_scatter=rs),
            "ffn.w3": Float8ColwiseParallel(),
        }
    else:
        plan = {"ffn.w1": Float8ColwiseParallel(), "ffn.w2": Float8RowwiseParallel(), "ffn.w3": Float8ColwiseParallel()}
    tp = parallelize_module(tp, mesh, plan)
    g = torch.Generator(device=dev).manual_seed(9)  # the same global input on every rank
    x_full = torch.randn(batch, seq, dim, device=dev, generator=g)
    x_ref = x_full.clone().requires_grad_(True)
    y_ref = ref(x_ref)
    y_ref.sum().backward()
    for _ in range(2):  # twice: the second pass reuses pooled gather buffers
        if sequence_parallel:
            x_loc = x_full.chunk(world, dim=1)[rank].clone().requires_grad_(True)
            y = tp(x_loc)
            y_loc = y.to_local() if isinstance(y, DTensor) else y
            y_full = _all_gather_cat(y_loc.detach(), world, 1)
            y_loc.sum().backward()
            gx = _all_gather_cat(x_loc.grad, world, 1)
        else:
            x_loc = x_full.clone().requires_grad_(True)
            y = tp(x_loc)
            y_full = y.full_tensor() if isinstance(y, DTensor) else y
            y_full.sum().backward()
            gx = x_loc.grad
        tol = dict(rtol=2e-3, atol=1e-4)
        torch.testing.assert_close(y_full.detach(), y_ref.detach(), **tol)
        torch.testing.assert_close(gx, x_ref.grad, **tol)
        w1g = tp.ffn.w1.weight.grad
        w1g = w1g.full_tensor() if isinstance(w1g, DTensor) else w1g
        torch.testing.assert_close(w1g, ref.ffn.w1.weight.grad, **tol)
        for p in tp.parameters():
            p.grad = None
    return "ok"


def parity_delayed_sync(dev, rank, world):
    """One all-reduce (MAX) over the [3 * n_layers] amax slab per sync; amaxes become the maximum
    over the ranks and the scales follow from them."""
    import float8_experimental_b200 as f8
    from float8_experimental_b200 import _native as N
    from float8_experimental_b200._ops import ops

    d = f8.CastConfig(scaling_type=f8.ScalingType.DELAYED)
    cfg = f8.Float8LinearConfig(cast_config_input=d, cast_config_weight=d, cast_config_grad_output=d)
    model = nn.Sequential(nn.Linear(16, 16, bias=False), nn.Linear(16, 16, bias=False)).to(dev)
    f8.convert_to_float8_training(model, config=cfg)
    for i, layer in enumerate(model):
        layer.last_seen_input_dtype = torch.float32
        layer.fp8_amax_input.fill_(1.0 + rank + i)
        layer.fp8_amax_weight.fill_(0.5 * (world - rank))
        layer.fp8_amax_grad_output.fill_(1e-3 * (1 + rank))
    calls = []
    real = dist.all_reduce

    def counting(t, *a, **k):
        calls.append(t.numel())
        return real(t, *a, **k)

    dist.all_reduce = counting
    try:
        f8.sync_float8_amax_and_scale_history(model)
    finally:
        dist.all_reduce = real
    assert calls == [6], calls
    for i, layer in enumerate(model):
        assert layer.fp8_amax_input.item() == float(world + i)
        assert layer.fp8_amax_weight.item() == 0.5 * world
        want = ops.amax_to_scale(torch.tensor([float(world + i)], device=dev), N.E4M3, N.FP32, N.FP32)
        assert layer.fp8_scale_input.item() == want.item()
    return "ok"


def parity_cast_all_gather(dev, rank, world):
    """The cast whose stores are the all-gather gives the bytes and the scale of cast-then-NCCL
    all-gather, call after call."""
    from float8_experimental_b200.float8_scaling_utils import hp_tensor_to_float8_dynamic
    from float8_experimental_b200.float8_tensor import LinearMMConfig
    from float8_experimental_b200.fp8_all_gather import CastAllGather

    gather = CastAllGather(max_numel_per_rank=2048 * 1024)
    cfg = LinearMMConfig()
    for it, (rows, cols) in enumerate([(2048, 1024), (1000, 520), (2048, 1024)]):
        g = torch.Generator(device=dev).manual_seed(100 * it + rank)
        x = torch.randn(rows, cols, device=dev, generator=g).mul_(1.0 + rank).to(torch.bfloat16)
        got = gather(x)
        ref_local = hp_tensor_to_float8_dynamic(x, torch.float8_e4m3fn, cfg, reduce_amax=True)
        ref = torch.empty(world * rows, cols, dtype=torch.uint8, device=dev)
        dist.all_gather_into_tensor(ref, ref_local._data.view(torch.uint8).contiguous())
        assert got._scale.item() == ref_local._scale.item()
        assert torch.equal(got._data.view(torch.uint8), ref)
    return "ok"


def run_parity(dev, rank, world):
    """All checks, each reported as "ok" or the failure text.  A failure on any rank is a failure
    of the run: the results are combined over the ranks."""
    results = {}
    cases = [
        ("fsdp2", lambda: parity_fsdp2(dev, rank, world)),
        ("tp", lambda: parity_tensor_parallel(dev, rank, world, False)),
        ("sp", lambda: parity_tensor_parallel(dev, rank, world, True)),
        ("delayed_sync", lambda: parity_delayed_sync(dev, rank, world)),
        ("cast_all_gather", lambda: parity_cast_all_gather(dev, rank, world)),
        ("sp_cast_all_gather", lambda: parity_tensor_parallel(dev, rank, world, True, cast_all_gather=True)),
        ("sp_fused_reduce_scatter", lambda: parity_tensor_parallel(dev, rank, world, True, fused_reduce_scatter=True)),
    ]
    for name, fn in cases:
        try:
            results[name] = fn()
        except Exception as exc:  # noqa: BLE001
            results[name] = f"FAILED: {type(exc).__name__}: {exc}"[:300]
        # agree on the outcome before the next case: a rank that failed must not leave the others
        # waiting inside a collective of the following case; every rank learns what failed where
        outcomes = [None] * world
        dist.all_gather_object(outcomes, results[name])
        bad = [f"rank {r}: {o}" for r, o in enumerate(outcomes) if o != "ok"]
        if bad:
            results[name] = "; ".join(bad)[:600]
            break
    torch.cuda.synchronize()
    return results


# ---------------------------------------------------------------------------
# side measurements
# ---------------------------------------------------------------------------
def _timed_steps(step, steps, dev):
    for _ in range(3):
        step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    dist.barrier()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms.item()


def measure_tp_sp_ffn(dev, rank, world, steps: int = 5):
    """Tensor / sequence parallel LLaMa-2-70B feed-forward block (8192 -> 2 x 28672 -> 8192), 2 x 8192
    tokens sequence-sharded over the ranks: PrepareFloat8ModuleInput + Float8ColwiseParallel x 2 +
    Float8RowwiseParallel, forward + backward.  Three routes: NCCL collectives issued by DTensor
    (cast + fp8 all-gather of the input, GEMM + bf16 reduce-scatter of the output: what the
    reference does); the input gathered by the cast whose stores are the all-gather (peer memory);
    and, on top of that, the row-parallel GEMM whose epilogue scatters its partial product into the
    owners' buffers."""
    from torch.distributed._tensor import Replicate, Shard
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor.parallel import parallelize_module

    import float8_experimental_b200 as f8
    from float8_experimental_b200.float8_tensor_parallel import (
        Float8ColwiseParallel,
        Float8RowwiseParallel,
        PrepareFloat8ModuleInput,
    )
    from float8_experimental_b200.fp8_all_gather import CastAllGatherPool

    dim, hidden, batch, seq = 8192, 28672, 2, 8192
    mesh = init_device_mesh("cuda", (world,))
    out = {"shape": {"dim": dim, "hidden": hidden, "tokens": batch * seq, "tp": world},
           "flops_per_step": 3 * 6.0 * batch * seq * dim * hidden}
    g = torch.Generator(device=dev).manual_seed(5 + rank)
    x = torch.randn(batch, seq // world, dim, dtype=torch.bfloat16, device=dev, generator=g).requires_grad_(True)
    go = torch.randn(batch, seq // world, dim, dtype=torch.bfloat16, device=dev, generator=g) * 1e-3
    from float8_experimental_b200.fused_reduce_scatter import GemmReduceScatter

    for route in ("nccl_collectives", "cast_all_gather", "cast_all_gather_and_fused_reduce_scatter"):
        torch.manual_seed(5)
        model = _Holder(FeedForward(dim, hidden)).to(device=dev, dtype=torch.bfloat16)
        f8.convert_to_float8_training(model, config=f8.Float8LinearConfig())
        pool = rs = None
        if route != "nccl_collectives":
            pool = CastAllGatherPool(mesh.get_group(0), max_numel_per_rank=batch * (seq // world) * dim, depth=2)
        if route == "cast_all_gather_and_fused_reduce_scatter":
            rs = GemmReduceScatter(mesh.get_group(0), max_out_numel_per_rank=batch * (seq // world) * dim)
        plan = {
            "ffn": PrepareFloat8ModuleInput(input_layouts=Shard(1), desired_input_layouts=Replicate(),
                                            cast_all_gather=pool),
            "ffn.w1": Float8ColwiseParallel(),
            "ffn.w2": Float8RowwiseParallel(output_layouts=Shard(1), fused_reduce_scatter=rs),
            "ffn.w3": Float8ColwiseParallel(),
        }
        model = parallelize_module(model, mesh, plan)

        def step():
            x.grad = None
            for p in model.parameters():
                p.grad = None
            y = model(x)
            y = y.to_local() if hasattr(y, "to_local") else y
            y.backward(go)

        try:
            ms = _timed_steps(step, steps, dev)
            out[route] = {"ms_per_step": ms, "tflops": out["flops_per_step"] / ms / 1e9}
        except Exception as exc:  # noqa: BLE001
            torch.cuda.synchronize()
            out[route] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        del model, pool, rs
        torch.cuda.empty_cache()
    return out


from .models import Llama3Block as _Llama3Block  # noqa: E402


def measure_fsdp2_llama3_8b_linears(dev, rank, world, steps: int = 3, n_blocks: int = 32, seq: int = 8192):
    """The 224 float8 linears of a Llama-3-8B-shaped decoder (32 blocks x 7 linears) under FSDP2, one
    `fully_shard` per block: fp8 weight all-gather per block before forward and before backward, bf16
    gradient reduce-scatter, one amax all-reduce for all 224 weights per step
    (precompute_float8_dynamic_scale_for_fsdp).  seq 8192 x batch 1 per GPU, forward + backward."""
    from torch.distributed.fsdp import fully_shard

    import float8_experimental_b200 as f8

    torch.manual_seed(11)
    blocks = nn.ModuleList()
    for _ in range(n_blocks):
        blk = _Llama3Block().to(device=dev, dtype=torch.bfloat16)
        for p in blk.parameters():
            nn.init.normal_(p, 0.0, 0.02)
        f8.convert_to_float8_training(blk, config=f8.Float8LinearConfig(enable_fsdp_float8_all_gather=True))
        fully_shard(blk)
        blocks.append(blk)
    model = nn.Sequential(*blocks)
    fully_shard(model)
    f8.precompute_float8_dynamic_scale_for_fsdp(model)
    g = torch.Generator(device=dev).manual_seed(200 + rank)
    x = torch.randn(1, seq, 4096, device=dev, dtype=torch.bfloat16, generator=g).requires_grad_(True)
    go = torch.randn(1, seq, 4096, device=dev, dtype=torch.bfloat16, generator=g) * 1e-3
    weights = sum(p.numel() for p in model.parameters()) * world  # parameters are sharded DTensors
    per_block = 4096 * 4096 * 2 + 4096 * 1024 * 2 + 3 * 4096 * 14336

    flops = 6.0 * seq * per_block * n_blocks
    out = {"blocks": n_blocks, "linears": 7 * n_blocks, "tokens_per_gpu": seq,
           "fp8_weight_bytes_gathered_per_pass": per_block * n_blocks, "local_weight_elements": weights // world}
    # the reference's schedule (each shard cast when its all-gather is issued, twice per step), and all
    # shards cast once per step by one multi-tensor launch right after the scales are known
    for name, cast_now in (("cast_per_all_gather", False), ("cast_all_shards_at_once", True)):
        def step():
            x.grad = None
            for p in model.parameters():
                p.grad = None
            model(x).backward(go)
            f8.precompute_float8_dynamic_scale_for_fsdp(model, cast_now=cast_now)

        ms = _timed_steps(step, steps, dev)
        out[name] = {"ms_per_step": ms, "tflops_all_gpus": world * flops / ms / 1e9}
    return out


def measure_cast_all_gather(dev, rank, world, rows: int = 8192, cols: int = 8192):
    """The fused cast + all-gather over peer memory against cast + NCCL all-gather on one
    [rows, cols] bf16 shard per rank."""
    from float8_experimental_b200.float8_scaling_utils import hp_tensor_to_float8_dynamic
    from float8_experimental_b200.float8_tensor import LinearMMConfig
    from float8_experimental_b200.fp8_all_gather import CastAllGather

    gather = CastAllGather(max_numel_per_rank=rows * cols)
    cfg = LinearMMConfig()
    x = torch.randn(rows, cols, device=dev).to(torch.bfloat16)
    ref = torch.empty(world * rows, cols, dtype=torch.uint8, device=dev)

    def unfused():
        r = hp_tensor_to_float8_dynamic(x, torch.float8_e4m3fn, cfg, reduce_amax=True)
        dist.all_gather_into_tensor(ref, r._data.view(torch.uint8))

    return {"shard": [rows, cols], "fused_ms": _timed_steps(lambda: gather(x), 10, dev),
            "cast_then_nccl_all_gather_ms": _timed_steps(unfused, 10, dev)}


def profile_step_split(step, dev, steps: int = 2):
    """Per-step CUDA time by kind of kernel over `steps` profiled steps (torch.profiler kernel
    sums; taken outside every timed region): this library's GEMM / cast / amax kernels, NCCL
    all-gather, reduce-scatter and all-reduce, and everything else (FSDP2's copy-in / copy-out and
    gradient plumbing).  Kernels of different streams overlap, so the parts add up to more than the
    step time; what matters is their size against the step."""
    from torch.profiler import ProfilerActivity, profile

    step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(steps):
            step()
        torch.cuda.synchronize()
    kinds = {"gemm": 0.0, "cast": 0.0, "amax": 0.0, "nccl_all_gather": 0.0, "nccl_reduce_scatter": 0.0,
             "nccl_all_reduce": 0.0, "memcpy_memset": 0.0, "other_kernels": 0.0}
    for ev in prof.key_averages():
        name = ev.key
        us = float(getattr(ev, "device_time_total", 0.0) or getattr(ev, "cuda_time_total", 0.0) or 0.0)
        if us <= 0.0:
            continue
        low = name.lower()
        if "gemm_fp8" in low:
            kinds["gemm"] += us
        elif "cast_" in low and "kernel" in low:
            kinds["cast"] += us
        elif "amax" in low:
            kinds["amax"] += us
        elif "nccl" in low and "allgather" in low:
            kinds["nccl_all_gather"] += us
        elif "nccl" in low and "reducescatter" in low:
            kinds["nccl_reduce_scatter"] += us
        elif "nccl" in low and "allreduce" in low:
            kinds["nccl_all_reduce"] += us
        elif "memcpy" in low or "memset" in low:
            kinds["memcpy_memset"] += us
        else:
            kinds["other_kernels"] += us
    out = {k: round(v / steps / 1e3, 3) for k, v in kinds.items()} | {"unit": "ms of device time per step", "steps": steps}
    try:
        out["timeline"] = _timeline_of(prof, steps)
    except Exception as exc:  # noqa: BLE001
        out["timeline"] = {"error": f"{type(exc).__name__}: {exc}"[:200]}
    return out


def _timeline_of(prof, steps):
    """Where the step's wall time goes on the stream that runs the GEMMs, from the profiler's kernel
    timeline: time that stream is busy, time it idles while an NCCL kernel runs on another stream (the
    exposed communication), and time it idles with nothing running anywhere (host-side gaps)."""
    import json
    import tempfile

    with tempfile.NamedTemporaryFile(suffix=".json") as f:
        prof.export_chrome_trace(f.name)
        trace = json.load(open(f.name))
    kernels = [e for e in trace.get("traceEvents", []) if e.get("cat") in ("kernel", "gpu_memcpy", "gpu_memset")
               and "dur" in e and "ts" in e]
    if not kernels:
        return {"error": "no kernel events in the trace"}
    stream_of = lambda e: e.get("args", {}).get("stream")  # noqa: E731
    gemm_streams = {}
    for e in kernels:
        if "gemm_fp8" in e["name"]:
            gemm_streams[stream_of(e)] = gemm_streams.get(stream_of(e), 0.0) + e["dur"]
    if not gemm_streams:
        return {"error": "no GEMM kernels in the trace"}
    main = max(gemm_streams, key=gemm_streams.get)
    t0 = min(e["ts"] for e in kernels)
    t1 = max(e["ts"] + e["dur"] for e in kernels)

    def merged(events):
        spans = sorted((e["ts"], e["ts"] + e["dur"]) for e in events)
        out_spans = []
        for a, b in spans:
            if out_spans and a <= out_spans[-1][1]:
                out_spans[-1][1] = max(out_spans[-1][1], b)
            else:
                out_spans.append([a, b])
        return out_spans

    def overlap(spans_a, spans_b):
        i = j = 0
        tot = 0.0
        while i < len(spans_a) and j < len(spans_b):
            lo, hi = max(spans_a[i][0], spans_b[j][0]), min(spans_a[i][1], spans_b[j][1])
            if hi > lo:
                tot += hi - lo
            if spans_a[i][1] < spans_b[j][1]:
                i += 1
            else:
                j += 1
        return tot

    busy = merged([e for e in kernels if stream_of(e) == main])
    idle, prev = [], t0
    for a, b in busy:
        if a > prev:
            idle.append([prev, a])
        prev = max(prev, b)
    if t1 > prev:
        idle.append([prev, t1])
    nccl = merged([e for e in kernels if "nccl" in e["name"].lower() and stream_of(e) != main])
    others = merged([e for e in kernels if stream_of(e) != main])
    busy_ms = sum(b - a for a, b in busy) / 1e3 / steps
    idle_ms = sum(b - a for a, b in idle) / 1e3 / steps
    idle_nccl = overlap(idle, nccl) / 1e3 / steps
    idle_other = overlap(idle, others) / 1e3 / steps
    gaps = sorted(((b - a) / 1e3 for a, b in idle), reverse=True)[:6]
    return {"span_ms_per_step": round((t1 - t0) / 1e3 / steps, 3), "gemm_stream_busy_ms": round(busy_ms, 3),
            "gemm_stream_idle_ms": round(idle_ms, 3), "idle_while_nccl_runs_ms": round(idle_nccl, 3),
            "idle_while_any_other_stream_runs_ms": round(idle_other, 3),
            "idle_with_nothing_running_ms": round(idle_ms - idle_other, 3),
            "largest_idle_gaps_ms": [round(g, 3) for g in gaps]}
