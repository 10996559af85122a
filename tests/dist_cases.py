"""Bodies of the multi-rank CPU tests (gloo, world_size 2).  Each function runs on every
rank inside a process spawned by `tests/test_distributed_cpu.py`; the `f8b200::*` ops
are served on CPU by the oracle-backed stand-ins of `tests/oracle_backend.py`."""
from __future__ import annotations

import copy
import os

import torch
import torch.distributed as dist
import torch.nn as nn


DEVICE = "cpu"  # "cuda" when F8_DIST_DEVICE=cuda: NCCL ranks, one GPU each, real kernels


def _init(rank: int, world: int, port: int):
    global DEVICE
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    if os.environ.get("F8_DIST_DEVICE") == "cuda":
        DEVICE = "cuda"
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        torch.set_default_device("cuda")
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        import oracle_backend

        oracle_backend.install()


def _delayed_config(f8, **kw):
    d = f8.CastConfig(scaling_type=f8.ScalingType.DELAYED)
    return f8.Float8LinearConfig(cast_config_input=d, cast_config_weight=d, cast_config_grad_output=d, **kw)


# ---------------------------------------------------------------------------
def case_sync_all_reduce(rank, world, port):
    """sync_float8_amax_and_scale_history takes the MAX of every amax over the ranks with
    one all-reduce, then derives the scales from it."""
    _init(rank, world, port)
    import float8_experimental_b200 as f8
    from oracle import f8_oracle as O

    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(8, 8, bias=False), nn.Linear(8, 8, bias=False))
    f8.convert_to_float8_training(model, config=_delayed_config(f8))
    for i, layer in enumerate(model):
        layer.last_seen_input_dtype = torch.float32
        layer.fp8_amax_input.fill_(1.0 + rank + i)          # max over ranks: world + i
        layer.fp8_amax_weight.fill_(0.5 * (world - rank))   # max over ranks: 0.5 * world
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
    assert calls == [6], calls  # one collective over the [3 * n_layers] slab
    for i, layer in enumerate(model):
        assert layer.fp8_amax_input.item() == float(world + i)
        assert layer.fp8_amax_weight.item() == 0.5 * world
        exp = O.amax_to_scale(float(world + i), O.E4M3, O.FP32, O.FP32)
        assert layer.fp8_scale_input.item() == float(exp)
        exp = O.amax_to_scale(1e-3 * world, O.E5M2, O.FP32, O.FP32)
        assert layer.fp8_scale_grad_output.item() == float(exp)
    dist.destroy_process_group()


# ---------------------------------------------------------------------------
class _MLP(nn.Module):
    def __init__(self, dim=32, hidden=64, n=3):
        super().__init__()
        self.layers = nn.ModuleList(
            [nn.Sequential(nn.Linear(dim, hidden, bias=False), nn.ReLU(), nn.Linear(hidden, dim, bias=False))
             for _ in range(n)]
        )

    def forward(self, x):
        for blk in self.layers:
            x = x + blk(x)
        return x


def case_fsdp2_fp8_all_gather(rank, world, port, precompute, cast_now=False):
    """FSDP2 with fp8 weight all-gather reproduces, loss for loss, an unsharded float8
    model whose gradients are averaged by hand (the reference's parity criterion,
    test/test_fsdp2/test_fsdp2_common.py:17-54); the all-gather carries 1 byte per
    weight element (test/test_fsdp2/test_fsdp2.py:324-405)."""
    _init(rank, world, port)
    from torch.distributed.fsdp import fully_shard

    import float8_experimental_b200 as f8
    from float8_experimental_b200.fsdp_utils import WeightWithDynamicFloat8CastTensor

    torch.manual_seed(42)
    base = _MLP()
    ref_model = copy.deepcopy(base)
    f8.convert_to_float8_training(ref_model, config=f8.Float8LinearConfig())
    fsdp_model = copy.deepcopy(base)
    f8.convert_to_float8_training(fsdp_model, config=f8.Float8LinearConfig(enable_fsdp_float8_all_gather=True))
    assert isinstance(fsdp_model.layers[0][0].weight, WeightWithDynamicFloat8CastTensor)
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
    torch.manual_seed(100 + rank)
    try:
        for step in range(3):
            x = torch.randn(16, 32)
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
                if model is fsdp_model and precompute:
                    f8.precompute_float8_dynamic_scale_for_fsdp(model, cast_now=cast_now)
                losses.append(loss.detach())
            if DEVICE == "cpu":
                assert torch.equal(losses[0], losses[1]), (step, losses)
            else:
                torch.testing.assert_close(losses[0], losses[1], rtol=1e-5, atol=0)
    finally:
        dist.all_gather_into_tensor = real_ag
    # every block all-gather moved bytes: (64*32 + 32*64) / world per rank, 1 byte each
    per_block = (64 * 32 + 32 * 64) // world
    block_gathers = [g for g in gathered if g[1] == per_block]
    assert len(block_gathers) >= 3 * 3, gathered
    assert all(dt == torch.uint8 for dt, _ in block_gathers)
    if precompute:
        w = fsdp_model.layers[0][0].weight._local_tensor
        assert w._precomputed_scale is not None and w._precomputed_scale.dim() == 0
        assert (w._precomputed_fp8 is not None) == bool(cast_now)
        if cast_now:  # the cached bytes are the bytes a cast at all-gather time would produce
            from float8_experimental_b200.float8_tensor import GemmInputRole, hp_tensor_and_scale_to_float8

            again = hp_tensor_and_scale_to_float8(w._tensor, w._precomputed_scale, torch.float8_e4m3fn,
                                                  w._linear_mm_config, GemmInputRole.WEIGHT)
            assert torch.equal(again._data.view(torch.uint8), w._precomputed_fp8.view(torch.uint8))
    dist.destroy_process_group()


def case_fsdp2_delayed(rank, world, port):
    """Delayed weight scaling under FSDP2: the wrapper updates the layer's own buffers and
    precompute refuses to run."""
    _init(rank, world, port)
    from torch.distributed.fsdp import fully_shard

    import float8_experimental_b200 as f8

    torch.manual_seed(1)
    model = _MLP(n=2)
    cfg = f8.Float8LinearConfig(
        enable_fsdp_float8_all_gather=True,
        cast_config_weight=f8.CastConfig(scaling_type=f8.ScalingType.DELAYED),
    )
    f8.convert_to_float8_training(model, config=cfg)
    for blk in model.layers:
        fully_shard(blk)
    fully_shard(model)
    lin = model.layers[0][0]
    before = lin.fp8_amax_weight.clone()
    torch.manual_seed(7 + rank)
    for _ in range(2):
        f8.sync_float8_amax_and_scale_history(model)
        model(torch.randn(16, 32)).sum().backward()
    assert not torch.equal(lin.fp8_amax_weight, before)
    full_w = lin.weight.full_tensor()
    assert lin.fp8_amax_history_weight[0].item() == full_w.abs().max().item()
    try:
        f8.precompute_float8_dynamic_scale_for_fsdp(model)
    except NotImplementedError:
        pass
    else:
        raise AssertionError("precompute must reject delayed weight scaling")
    dist.destroy_process_group()


# ---------------------------------------------------------------------------
class _FFN(nn.Module):
    def __init__(self, dim=16, hidden=32):
        super().__init__()
        self.w1 = nn.Linear(dim, hidden, bias=False)
        self.w2 = nn.Linear(hidden, dim, bias=False)
        self.w3 = nn.Linear(dim, hidden, bias=False)

    def forward(self, x):
        return self.w2(nn.functional.silu(self.w1(x)) * self.w3(x))


class _Toy(nn.Module):
    def __init__(self, dim=16, hidden=32):
        super().__init__()
        self.ffn = _FFN(dim, hidden)

    def forward(self, x):
        return self.ffn(x)


class _StubReduceScatter:
    """Stands in for `GemmReduceScatter` where there is no peer memory (CPU ranks): the local
    product through the ordinary op, an all-reduce, and this rank's slice.  What the test then
    covers is the host side of the fused route: the autograd function, its backward (fp8 all-gather
    of the gradient, the two float8 products) and the parallel style's wiring."""

    def __call__(self, x8, w8_t, shard_dim):
        from float8_experimental_b200.float8_python_api import addmm_float8_unwrapped

        lead = tuple(x8.shape[:-1])
        y = addmm_float8_unwrapped(x8._data.reshape(-1, x8.shape[-1]), x8._scale, w8_t._data, w8_t._scale,
                                   output_dtype=x8._orig_dtype)
        dist.all_reduce(y)
        y = y.reshape(*lead, y.shape[-1])
        return y.chunk(dist.get_world_size(), dim=shard_dim)[dist.get_rank()].contiguous()


def case_tensor_parallel(rank, world, port, sequence_parallel, fused_reduce_scatter=False):
    """TP (and SP) float8 FFN == the unsharded float8 FFN
    (the reference's criterion, test/test_dtensor.py:189-231)."""
    _init(rank, world, port)
    from torch.distributed._tensor import DTensor, Replicate, Shard
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor.parallel import parallelize_module

    import float8_experimental_b200 as f8
    from float8_experimental_b200.float8_tensor import Float8Tensor
    from float8_experimental_b200.float8_tensor_parallel import (
        Float8ColwiseParallel,
        Float8RowwiseParallel,
        PrepareFloat8ModuleInput,
    )

    mesh = init_device_mesh(DEVICE, (world,))
    torch.manual_seed(5)
    ref = _Toy()
    f8.convert_to_float8_training(ref, config=f8.Float8LinearConfig())
    tp = copy.deepcopy(ref)

    gathered_dtypes = []
    if sequence_parallel:
        plan = {
            "ffn": PrepareFloat8ModuleInput(input_layouts=Shard(1), desired_input_layouts=Replicate()),
            "ffn.w1": Float8ColwiseParallel(),
            "ffn.w2": Float8RowwiseParallel(output_layouts=Shard(1),
                                            fused_reduce_scatter=_StubReduceScatter() if fused_reduce_scatter else None),
            "ffn.w3": Float8ColwiseParallel(),
        }
    else:
        plan = {
            "ffn.w1": Float8ColwiseParallel(),
            "ffn.w2": Float8RowwiseParallel(),
            "ffn.w3": Float8ColwiseParallel(),
        }
    tp = parallelize_module(tp, mesh, plan)

    torch.manual_seed(9)  # same global input on every rank
    x_full = torch.randn(2, 8, 16)
    x_ref = x_full.clone().requires_grad_(True)
    y_ref = ref(x_ref)
    y_ref.sum().backward()

    if sequence_parallel:
        x_loc = x_full.chunk(world, dim=1)[rank].clone().requires_grad_(True)
        # spy on the functional all-gather payload
        import float8_experimental_b200.float8_ops as fo

        inner = fo.FLOAT8_OPS_TABLE[torch.ops._c10d_functional.all_gather_into_tensor.default]

        def spy(op, args, kwargs=None):
            gathered_dtypes.append((type(args[0]), args[0]._data.dtype))
            return inner(op, args, kwargs)

        fo.FLOAT8_OPS_TABLE[torch.ops._c10d_functional.all_gather_into_tensor.default] = spy
        y = tp(x_loc)
        y_full = torch.cat(_all_gather_list(y if not isinstance(y, DTensor) else y.to_local(), world), dim=1)
        y.sum().backward() if not isinstance(y, DTensor) else y.to_local().sum().backward()
        gx = torch.cat(_all_gather_list(x_loc.grad, world), dim=1)
        assert gathered_dtypes and gathered_dtypes[0] == (Float8Tensor, torch.float8_e4m3fn), gathered_dtypes
    else:
        x_loc = x_full.clone().requires_grad_(True)
        y = tp(x_loc)
        y_full = y.full_tensor() if isinstance(y, DTensor) else y
        y_full.sum().backward()
        gx = x_loc.grad
    tol = dict(rtol=1e-5, atol=1e-6) if DEVICE == "cpu" else dict(rtol=2e-3, atol=1e-4)
    torch.testing.assert_close(y_full.detach(), y_ref.detach(), **tol)
    torch.testing.assert_close(gx, x_ref.grad, **tol)
    w1g = tp.ffn.w1.weight.grad
    w1g = w1g.full_tensor() if isinstance(w1g, DTensor) else w1g
    torch.testing.assert_close(w1g, ref.ffn.w1.weight.grad, **tol)
    dist.destroy_process_group()


def case_cast_all_gather_over_peer_memory(rank, world, port):
    """The cast that scatters its result into every rank's gathered buffer (peer stores) gives
    the bytes and the scale of cast-then-NCCL-all-gather; repeated calls reuse the buffers.
    GPU only: symmetric memory needs peer access."""
    _init(rank, world, port)
    from float8_experimental_b200.float8_scaling_utils import hp_tensor_to_float8_dynamic
    from float8_experimental_b200.float8_tensor import LinearMMConfig
    from float8_experimental_b200.fp8_all_gather import CastAllGather

    gather = CastAllGather(max_numel_per_rank=8192 * 8192)
    cfg = LinearMMConfig()
    for it, (rows, cols) in enumerate([(8192, 8192), (1000, 520), (8192, 8192)]):
        g = torch.Generator(device="cuda").manual_seed(100 * it + rank)
        x = torch.randn(rows, cols, device="cuda", generator=g).mul_(1.0 + rank).to(torch.bfloat16)
        got = gather(x)
        # reference route: global-amax cast, then the NCCL all-gather of the bytes
        ref_local = hp_tensor_to_float8_dynamic(x, torch.float8_e4m3fn, cfg, reduce_amax=True)
        ref = torch.empty(world * rows, cols, dtype=torch.uint8, device="cuda")
        dist.all_gather_into_tensor(ref, ref_local._data.view(torch.uint8).contiguous())
        assert got._scale.item() == ref_local._scale.item()
        assert got._data.shape == (world * rows, cols)
        assert torch.equal(got._data.view(torch.uint8), ref)
    dist.barrier()
    dist.destroy_process_group()


def case_fsdp1_composition(rank, world, port, weight_dynamic):
    """Float8Linear under the first-generation FSDP wrapper (flat parameters, `use_orig_params=True`), the
    procedure of the reference's test/test_fsdp.py:68-184: a two-layer model, once in the base dtype and
    once converted to float8 (input and grad_output delayed, weight delayed or dynamic), both wrapped,
    two SGD iterations on per-rank slices of one global batch with `sync_float8_amax_and_scale_history`
    after each float8 backward; the gathered outputs and the full parameters of the two models must agree
    to more than 15 dB."""
    _init(rank, world, port)
    import float8_experimental_b200 as f8
    from float8_experimental_b200.float8_utils import compute_error
    from torch.distributed.fsdp import FullyShardedDataParallel as FSDP

    batch, seq, k, n = 8, 8, 32, 32
    dtype = torch.bfloat16 if DEVICE == "cuda" else torch.float32
    torch.manual_seed(0)
    base = nn.Sequential(nn.Linear(k, n, dtype=dtype), nn.ReLU(), nn.Linear(n, n, dtype=dtype)).to(DEVICE)
    model_f8 = copy.deepcopy(base)
    delayed = f8.CastConfig(scaling_type=f8.ScalingType.DELAYED)
    config = f8.Float8LinearConfig(
        cast_config_input=delayed, cast_config_grad_output=delayed,
        cast_config_weight=f8.CastConfig(scaling_type=f8.ScalingType.DYNAMIC) if weight_dynamic else delayed)
    f8.convert_to_float8_training(model_f8, config=config)
    device_id = torch.device("cuda", rank) if DEVICE == "cuda" else torch.device("cpu")
    base = FSDP(base, use_orig_params=True, device_id=device_id)
    model_f8 = FSDP(model_f8, use_orig_params=True, device_id=device_id)
    opt = torch.optim.SGD(base.parameters(), lr=0.01)
    opt_f8 = torch.optim.SGD(model_f8.parameters(), lr=0.01)
    lo, hi = rank * batch // world, (rank + 1) * batch // world
    xs = [torch.randn(batch, seq, k, device=DEVICE).to(dtype)[lo:hi] for _ in range(2)]
    gs = [torch.randn(batch, seq, n, device=DEVICE).to(dtype)[lo:hi] for _ in range(2)]
    y = y_f8 = None
    for i in range(2):  # the second iteration is the first that casts with scales from the history
        opt.zero_grad()
        y = base(xs[i])
        y.backward(gs[i])
        opt.step()
        opt_f8.zero_grad()
        y_f8 = model_f8(xs[i])
        y_f8.backward(gs[i])
        assert f8.linear_requires_sync(config)
        f8.sync_float8_amax_and_scale_history(model_f8)
        opt_f8.step()
    whole = torch.cat(_all_gather_list(y.detach(), world))
    whole_f8 = torch.cat(_all_gather_list(y_f8.detach(), world))
    assert compute_error(whole, whole_f8).item() > 15.0
    # the reference compares full state dicts; gathering the full parameters compares the same tensors
    with FSDP.summon_full_params(base), FSDP.summon_full_params(model_f8):
        full = dict(base.named_parameters())
        full_f8 = dict(model_f8.named_parameters())
        assert len(full) == 4 and full.keys() == full_f8.keys()
        for name, v in full.items():
            assert compute_error(v.detach().float(), full_f8[name].detach().float()).item() > 15.0, name
    dist.barrier()
    dist.destroy_process_group()


def case_package_parity(rank, world, port, name):
    """The parity checks the benchmark runs before it times anything on several GPUs
    (`float8_experimental_b200.benchmarks.multi_gpu`), one by one.  GPU only."""
    _init(rank, world, port)
    from float8_experimental_b200.benchmarks import multi_gpu

    dev = torch.device("cuda", rank)
    fn = {
        "fsdp2": lambda: multi_gpu.parity_fsdp2(dev, rank, world),
        "tp": lambda: multi_gpu.parity_tensor_parallel(dev, rank, world, False),
        "sp": lambda: multi_gpu.parity_tensor_parallel(dev, rank, world, True),
        "delayed_sync": lambda: multi_gpu.parity_delayed_sync(dev, rank, world),
        "cast_all_gather": lambda: multi_gpu.parity_cast_all_gather(dev, rank, world),
        "sp_cast_all_gather": lambda: multi_gpu.parity_tensor_parallel(dev, rank, world, True, cast_all_gather=True),
        "sp_fused_reduce_scatter": lambda: multi_gpu.parity_tensor_parallel(dev, rank, world, True,
                                                                            fused_reduce_scatter=True),
    }[name]
    assert fn() == "ok"
    torch.cuda.synchronize()
    from float8_experimental_b200 import _native

    assert _native.read_device_error() == 0
    dist.barrier()
    dist.destroy_process_group()


def _all_gather_list(t, world):
    outs = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(outs, t.contiguous())
    return outs
