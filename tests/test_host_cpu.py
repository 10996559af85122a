"""Host-side logic on CPU: the package's Python layer runs unchanged, the `f8b200::*`
ops are served by the oracle-backed stand-ins from `tests/oracle_backend.py`."""
import copy
import io
import os
import subprocess
import sys

import numpy as np
import pytest
import torch
import torch.nn as nn

import oracle_backend
from oracle import f8_oracle as O

oracle_backend.install()

import float8_experimental_b200 as f8  # noqa: E402
from float8_experimental_b200 import float8_linear_utils  # noqa: E402
from float8_experimental_b200.float8_linear import Float8Linear  # noqa: E402
from float8_experimental_b200.float8_ops import FLOAT8_OPS_TABLE  # noqa: E402
from float8_experimental_b200.float8_scaling_utils import (  # noqa: E402
    hp_tensor_to_float8_delayed,
    hp_tensor_to_float8_dynamic,
)
from float8_experimental_b200.float8_tensor import (  # noqa: E402
    Float8Tensor,
    GemmInputRole,
    hp_tensor_and_scale_to_float8,
    LinearMMConfig,
    ScaledMMConfig,
)
from float8_experimental_b200.float8_utils import (  # noqa: E402
    amax_to_scale,
    compute_error,
    e4m3_dtype,
    e5m2_dtype,
    fp8_tensor_statistics,
    tensor_to_amax,
    tensor_to_scale,
    to_fp8_saturated,
)

DT = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}
F8 = {"e4m3fn": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def t_from(arr, dname):
    return oracle_backend.from_np(arr, DT[dname])


def delayed_config(**kw):
    d = f8.CastConfig(scaling_type=f8.ScalingType.DELAYED)
    return f8.Float8LinearConfig(cast_config_input=d, cast_config_weight=d, cast_config_grad_output=d, **kw)


def make_linear(w, config):
    lin = nn.Linear(w.shape[1], w.shape[0], bias=False, dtype=w.dtype)
    with torch.no_grad():
        lin.weight.copy_(w)
    return Float8Linear.from_float(lin, config)


# ---------------------------------------------------------------------------
def test_casts_through_public_functions(golden_dir):
    g = np.load(os.path.join(golden_dir, "casts.npz"))
    cfg = LinearMMConfig()
    for i in range(int(g["n"])):
        dname, fname = [str(s) for s in g[f"c{i}_meta"]]
        x = t_from(g[f"c{i}_x"], dname)
        dyn = hp_tensor_to_float8_dynamic(x, F8[fname], cfg)
        assert isinstance(dyn, Float8Tensor) and dyn._scale.dim() == 0 and dyn._scale.dtype == torch.float32
        assert np.array_equal(oracle_backend.to_np(dyn._data), g[f"c{i}_dyn_bits"])
        assert dyn._scale.item() == g[f"c{i}_dyn_scale"]
        buf = torch.tensor([0.0])
        dly = hp_tensor_to_float8_delayed(x, torch.from_numpy(g[f"c{i}_del_scale"].copy()), F8[fname], buf, cfg)
        assert np.array_equal(oracle_backend.to_np(dly._data), g[f"c{i}_del_bits"])
        assert buf.item() == g[f"c{i}_del_amax"][0]
        # the emitted second layout holds the same values
        if dyn._alt is not None:
            flat = dyn._data.reshape(-1, dyn._data.shape[-1]).view(torch.uint8)
            assert torch.equal(dyn._alt.view(torch.uint8), flat)
            assert dyn._alt.stride(0) == 1


def test_scale_helpers_match_reference_semantics():
    x = torch.randn(64, 32, dtype=torch.bfloat16)
    amax = tensor_to_amax(x)
    assert amax.dtype == torch.bfloat16 and amax.dim() == 0
    assert amax == x.abs().max()
    s = tensor_to_scale(x, e4m3_dtype)
    assert s.dtype == torch.float32
    # scale computed in bf16: representable in bf16
    assert s == s.to(torch.bfloat16).float()
    tiny = torch.tensor([1e-7], dtype=torch.float16)
    assert torch.isfinite(amax_to_scale(tiny.abs().max(), e4m3_dtype, torch.float16))
    assert amax_to_scale(torch.tensor(0.0, dtype=torch.float16), e5m2_dtype, torch.float16) == 65504.0
    y = to_fp8_saturated(torch.tensor([1e6, -1e6, 1.0]), e4m3_dtype)
    assert y.float().tolist() == [448.0, -448.0, 1.0]


def test_linear_dynamic_matches_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "linear_small.npz"))
    for dname in ("bf16", "fp32"):
        m = make_linear(t_from(g[f"{dname}_w"], dname), f8.Float8LinearConfig())
        x = t_from(g[f"{dname}_x0"], dname).requires_grad_(True)
        y = m(x)
        assert y.dtype == DT[dname]
        y.backward(t_from(g[f"{dname}_go0"], dname))
        for got, key in ((y, "y"), (x.grad, "dx"), (m.weight.grad, "dw")):
            ref = t_from(g[f"{dname}_dyn_{key}"], dname).float()
            assert got.shape == ref.shape
            assert compute_error(ref, got.detach().float()) > 55.0, (dname, key)


def test_linear_delayed_three_iterations(golden_dir):
    g = np.load(os.path.join(golden_dir, "linear_small.npz"))
    dname = "bf16"
    m = make_linear(t_from(g[f"{dname}_w"], dname), delayed_config())
    names = ("input", "weight", "grad_output")
    for it in range(3):
        if it > 0:
            f8.sync_float8_amax_and_scale_history(m)
        x = t_from(g[f"{dname}_x{it}"], dname).requires_grad_(True)
        m.weight.grad = None
        y = m(x)
        y.backward(t_from(g[f"{dname}_go{it}"], dname))
        for n in names:
            assert getattr(m, f"fp8_amax_{n}").item() == g[f"{dname}_del{it}_amax_{n}"][0], (it, n)
            assert getattr(m, f"fp8_scale_{n}").item() == g[f"{dname}_del{it}_scale_{n}"][0], (it, n)
            assert np.array_equal(getattr(m, f"fp8_amax_history_{n}").numpy(), g[f"{dname}_del{it}_hist_{n}"])
        ref = t_from(g[f"{dname}_del{it}_y"], dname).float()
        assert compute_error(ref, y.detach().float()) > 55.0
    f8.sync_float8_amax_and_scale_history(m)
    for n in names:
        assert getattr(m, f"fp8_scale_{n}").item() == g[f"{dname}_del3_scale_{n}"][0]
        assert np.array_equal(getattr(m, f"fp8_amax_history_{n}").numpy(), g[f"{dname}_del3_hist_{n}"])


def test_forward_without_sync_raises(golden_dir):
    m = make_linear(torch.randn(16, 32), delayed_config())
    x = torch.randn(4, 32)
    m(x)
    with pytest.raises(AssertionError, match="amaxes and scales not synced"):
        m(x)
    f8.sync_float8_amax_and_scale_history(m)
    m(x)


def test_sync_batched_over_layers(golden_dir):
    g = np.load(os.path.join(golden_dir, "sync.npz"))
    for dname in ("bf16", "fp16", "fp32"):
        amax, hist = g[f"{dname}_amax"], g[f"{dname}_hist"]
        L = amax.shape[1]
        model = nn.Sequential(*[nn.Linear(8, 8, bias=False) for _ in range(L)])
        f8.convert_to_float8_training(model, config=delayed_config())
        for i, layer in enumerate(model):
            layer.last_seen_input_dtype = DT[dname]
            for k, n in enumerate(("input", "weight", "grad_output")):
                getattr(layer, f"fp8_amax_{n}").fill_(float(amax[k, i]))
                getattr(layer, f"fp8_amax_history_{n}").copy_(torch.from_numpy(hist[k, i].copy()))
        f8.sync_float8_amax_and_scale_history(model)
        for i, layer in enumerate(model):
            assert layer.amax_and_scale_synced
            for k, n in enumerate(("input", "weight", "grad_output")):
                assert getattr(layer, f"fp8_scale_{n}").item() == g[f"{dname}_scales"][k, i], (dname, n, i)
                assert np.array_equal(getattr(layer, f"fp8_amax_history_{n}").numpy(), g[f"{dname}_hist_after"][k, i])
        # second call reuses the slabs; buffers are views into them
        slabs = getattr(model[0], "_f8_sync_slabs")
        f8.sync_float8_amax_and_scale_history(model)
        assert getattr(model[0], "_f8_sync_slabs") is slabs
        assert model[1].fp8_scale_weight.data_ptr() == slabs.scale[L + 1 : L + 2].data_ptr()
        # moving the module invalidates the views; the next sync re-packs
        model.to(torch.float32)
        f8.sync_float8_amax_and_scale_history(model)
        assert getattr(model[0], "_f8_sync_slabs") is not slabs
        assert model[2].fp8_scale_input.item() == g[f"{dname}_scales"][0, 2]


def test_sync_write_back_flag():
    model = nn.Sequential(nn.Linear(8, 8, bias=False))
    f8.convert_to_float8_training(model, config=delayed_config())
    model[0].last_seen_input_dtype = torch.float32
    model[0].fp8_amax_input.fill_(3.0)
    model[0].fp8_amax_history_input.copy_(torch.arange(16.0) / 16)
    float8_linear_utils.WRITE_BACK_AMAX_HISTORY = True
    try:
        f8.sync_float8_amax_and_scale_history(model)
    finally:
        float8_linear_utils.WRITE_BACK_AMAX_HISTORY = False
    h = model[0].fp8_amax_history_input
    assert h[0] == 3.0 and torch.equal(h[1:], torch.arange(15.0) / 16)


def test_sync_input_checks():
    model = nn.Sequential(nn.Linear(8, 8), nn.Linear(8, 8))
    f8.convert_to_float8_training(model, config=delayed_config())
    model[0].last_seen_input_dtype = torch.float32
    model[1].last_seen_input_dtype = torch.bfloat16
    with pytest.raises(ValueError, match="same last seen input_dtype"):
        f8.sync_float8_amax_and_scale_history(model)
    f8.sync_float8_amax_and_scale_history(nn.Sequential(nn.ReLU()))  # warns, returns


# ---------------------------------------------------------------------------
def test_module_swap_and_filter():
    lin = nn.Linear(8, 16)
    out = f8.convert_to_float8_training(copy.deepcopy(lin))
    assert isinstance(out, Float8Linear) and out.bias is not None
    assert 'scaling="i:dyn,w:dyn,go:dyn"' in repr(out)

    class Root(nn.Linear):
        def __init__(self):
            super().__init__(4, 4)
            self.child = nn.Linear(4, 4)

    with pytest.raises(AssertionError, match="Does not support a root nn.Linear with children"):
        f8.convert_to_float8_training(Root())

    model = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Sequential(nn.Linear(16, 24), nn.Linear(24, 10)))
    seen = []

    def keep(mod, fqn):
        seen.append(fqn)
        return mod.out_features % 16 != 10 and fqn != "2.0"

    f8.convert_to_float8_training(model, module_filter_fn=keep)
    assert seen == ["0", "2.0", "2.1"]
    assert isinstance(model[0], Float8Linear)
    assert not isinstance(model[2][0], Float8Linear) and not isinstance(model[2][1], Float8Linear)
    assert f8.linear_requires_sync(delayed_config()) and not f8.linear_requires_sync(f8.Float8LinearConfig())
    with pytest.raises(AssertionError):
        f8.DelayedScalingConfig(scale_fn_name="mean")


def test_buffers_stay_fp32_and_state_dict_roundtrip():
    m = make_linear(torch.randn(16, 32), delayed_config())
    m.to(torch.bfloat16)
    assert m.weight.dtype == torch.bfloat16
    for name in m.always_float32_buffers:
        assert getattr(m, name).dtype == torch.float32
    sd = m.state_dict()
    assert set(sd) == {"weight"} | {f"fp8_{k}_{n}" for k in ("amax", "amax_history", "scale")
                                    for n in ("input", "weight", "grad_output")}
    m2 = make_linear(torch.randn(16, 32), delayed_config()).to(torch.bfloat16)
    m2.load_state_dict(sd)
    assert torch.equal(m2.fp8_amax_history_weight, m.fp8_amax_history_weight)


def test_float8_tensor_ops(monkeypatch):
    monkeypatch.setenv("F8B200_CAST_TRANSPOSED", "1")  # casts emit the second layout, which the ops must carry along
    cfg = LinearMMConfig()
    x = torch.randn(16, 32, dtype=torch.bfloat16)
    a = hp_tensor_to_float8_dynamic(x, e4m3_dtype, cfg)
    assert a.dtype == torch.bfloat16 and a._data.dtype == e4m3_dtype
    # split / cat round trip is the identity on the bytes
    parts = torch.split(a, 4, dim=0)
    back = torch.cat(parts, dim=0)
    assert isinstance(back, Float8Tensor) and torch.equal(back._data.view(torch.uint8), a._data.view(torch.uint8))
    # t / transpose / view carry the second layout along
    at = a.t()
    assert at.shape == (32, 16) and at._alt is not None and at._alt.is_contiguous()
    assert a.view(4, 4, 32).reshape(-1, 32)._alt is not None
    assert a[2:5]._alt is None
    # dequantisation
    deq = a.to_original_precision()
    assert deq.dtype == torch.bfloat16 and compute_error(x.float(), deq.float()) > 20
    # copy_ rules
    hp = torch.zeros(16, 32, dtype=torch.bfloat16)
    hp.copy_(a)
    assert torch.equal(hp, deq)
    b = hp_tensor_and_scale_to_float8(x * 0.5, a._scale, e4m3_dtype, cfg)
    a2 = a.detach().clone()
    a2.copy_(b)
    assert torch.equal(a2._data.view(torch.uint8), b._data.view(torch.uint8))
    with pytest.raises(RuntimeError, match="Unsupported semantics for copy_"):
        a2.copy_(x)
    # index_put_
    a3 = a.detach().clone()
    a3[torch.tensor([0, 1])] = b[torch.tensor([2, 3])] if False else Float8Tensor(
        b._data[2:4], b._scale, b._orig_dtype, b._linear_mm_config, b._gemm_input_role)
    assert torch.equal(a3._data[0:2].view(torch.uint8), b._data[2:4].view(torch.uint8))
    # unsupported op
    with pytest.raises(NotImplementedError, match="this is not supported"):
        torch.sin(a)
    # statistics
    z = hp_tensor_and_scale_to_float8(torch.tensor([[0.0, 1e9, 1.0, -1e9]]), torch.tensor(1.0), e4m3_dtype, cfg)
    assert fp8_tensor_statistics(z) == (1, 2)


def test_mm_config_mismatch_message():
    x = torch.randn(16, 16, dtype=torch.bfloat16)
    c1 = LinearMMConfig()
    c2 = LinearMMConfig(ScaledMMConfig(True, False, False, False), c1.grad_input, c1.grad_weight)
    a = hp_tensor_to_float8_dynamic(x, e4m3_dtype, c1)
    b = hp_tensor_to_float8_dynamic(x, e4m3_dtype, c2, gemm_input_role=GemmInputRole.WEIGHT)
    with pytest.raises(AssertionError, match="linear_mm_config.output mismatch"):
        torch.mm(a, b.t())


@pytest.mark.parametrize("single_node", ["1", "0"])
def test_gemms_read_the_cast_outputs_where_they_lie(monkeypatch, single_node):
    """Forward, dgrad and wgrad hand the GEMM views of the three cast results: no transposed
    or contiguous copy of an fp8 tensor is made on the way, on the single-node route as on the
    general one."""
    import float8_experimental_b200.float8_linear as fl
    import float8_experimental_b200.float8_python_api as api
    import float8_experimental_b200.float8_tensor as ft

    monkeypatch.setenv("F8B200_LINEAR_SINGLE_NODE", single_node)

    cast_ptrs, operand_ptrs = set(), []

    class Spy:
        def __init__(self, record):
            self.record = record

        def __getattr__(self, name):
            fn = getattr(torch.ops.f8b200, name)

            def wrapped(*a, **k):
                out = fn(*a, **k)
                self.record(name, a, out)
                return out

            return wrapped

    def on_cast(name, args, out):
        if name in ("cast_from_amax", "cast_dynamic"):
            cast_ptrs.add(out[0].data_ptr())

    def on_mm(name, args, out):
        if name == "scaled_mm":
            operand_ptrs.extend([args[0].data_ptr(), args[1].data_ptr()])

    def on_both(name, args, out):
        on_cast(name, args, out)
        on_mm(name, args, out)

    monkeypatch.setattr(ft, "ops", Spy(on_cast))
    monkeypatch.setattr(api, "ops", Spy(on_mm))
    monkeypatch.setattr(fl, "ops", Spy(on_both))
    m = make_linear(torch.randn(48, 32, dtype=torch.bfloat16), f8.Float8LinearConfig())
    x = torch.randn(2, 8, 32, dtype=torch.bfloat16, requires_grad=True)
    m(x).sum().backward()
    assert len(cast_ptrs) == 3 and len(operand_ptrs) == 6
    assert set(operand_ptrs) == cast_ptrs
    assert x.grad.shape == x.shape and m.weight.grad.shape == (48, 32)


def test_autocast_output_dtype():
    m = make_linear(torch.randn(16, 32), f8.Float8LinearConfig())
    with torch.autocast("cuda", dtype=torch.bfloat16, enabled=False):
        assert m(torch.randn(4, 32)).dtype == torch.float32


def test_weights_only_load_of_float8_tensor():
    a = hp_tensor_to_float8_dynamic(torch.randn(8, 8), e4m3_dtype, LinearMMConfig())
    buf = io.BytesIO()
    torch.save(a, buf)
    buf.seek(0)
    b = torch.load(buf, weights_only=True)
    assert isinstance(b, Float8Tensor) and torch.equal(b._data.view(torch.uint8), a._data.view(torch.uint8))


def test_package_has_no_cpu_path():
    code = (
        "import torch, float8_experimental_b200 as f\n"
        "from float8_experimental_b200.float8_linear import Float8Linear\n"
        "m = Float8Linear.from_float(torch.nn.Linear(16, 16))\n"
        "try:\n"
        "    m(torch.randn(4, 16))\n"
        "except Exception as e:\n"
        "    print('RAISED', type(e).__name__)\n"
        "else:\n"
        "    print('RAN')\n"
    )
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=ROOT)
    assert "RAISED" in out.stdout, out.stdout + out.stderr


def test_gemm_operand_layout_selection():
    """How `scaled_mm` hands an operand to the GEMM: as it lies when K or the rows are contiguous
    and TMA can address it, else as a K-major copy."""
    from float8_experimental_b200._ops import _gemm_operand

    base = torch.zeros(64, 48, dtype=torch.uint8).view(torch.float8_e4m3fn)
    t, ld, mn = _gemm_operand(base)                      # [64, 48], K contiguous
    assert t is base and ld == 48 and mn is False
    t, ld, mn = _gemm_operand(base.t())                  # logical [48, 64] stored [64, 48]: rows contiguous
    assert t.data_ptr() == base.data_ptr() and ld == 48 and mn is True
    odd = torch.zeros(64, 40, dtype=torch.uint8).view(torch.float8_e4m3fn)
    t, ld, mn = _gemm_operand(odd.t())                   # pitch 40 is not a multiple of 16: copied
    assert mn is False and t.is_contiguous() and t.shape == (40, 64) and ld == 64
    sliced = base[:, 1:33]                               # K contiguous but the base address is odd
    t, ld, mn = _gemm_operand(sliced)
    assert mn is False and t.is_contiguous() and ld == 32
    ragged = torch.arange(8 * 40, dtype=torch.uint8).view(8, 40).view(torch.float8_e4m3fn)
    t, ld, mn = _gemm_operand(ragged)                    # K = 40: the copy gets a 48-byte row pitch, K stays 40
    assert mn is False and ld == 48 and t.shape == (8, 40) and t.stride(0) == 48
    assert torch.equal(t.view(torch.uint8), ragged.view(torch.uint8))
    one_row = base[:1]
    t, ld, mn = _gemm_operand(one_row)                   # a single row: any pitch that TMA accepts
    assert mn is False and ld % 16 == 0 and ld >= 48


def test_multicast_gemm_selection_rules(monkeypatch):
    """The single-GPU multicast library is opt-in (F8B200_GEMM_MC=21/22/41), used only when
    present, only in single-GPU jobs, and never when a kernel is forced."""
    from float8_experimental_b200 import _native as N

    monkeypatch.setattr(N, "load_mc", lambda: object())
    monkeypatch.setattr(N, "_single_gpu_job", lambda: True)
    monkeypatch.delenv("F8B200_GEMM_MC", raising=False)
    monkeypatch.delenv("F8B200_GEMM_MODE", raising=False)
    assert N._mc_cluster(8192, 8192, 16384) is None  # not by default
    monkeypatch.setenv("F8B200_GEMM_MC", "21")
    assert N._mc_cluster(8192, 8192, 16384) == (2, 1)
    monkeypatch.setenv("F8B200_GEMM_MODE", "wide")
    assert N._mc_cluster(8192, 8192, 16384) is None
    monkeypatch.delenv("F8B200_GEMM_MODE")
    monkeypatch.setenv("F8B200_GEMM_MC", "22")
    assert N._mc_cluster(16384, 8192, 8192) == (2, 2)
    monkeypatch.setenv("F8B200_GEMM_MC", "0")
    assert N._mc_cluster(8192, 8192, 16384) is None
    monkeypatch.setenv("F8B200_GEMM_MC", "21")
    monkeypatch.setattr(N, "load_mc", lambda: None)  # library not shipped (runs on several GPUs)
    assert N._mc_cluster(8192, 8192, 16384) is None
    # ... and never in a job that may use a second GPU, whatever was shipped or forced
    monkeypatch.setattr(N, "load_mc", lambda: object())
    monkeypatch.setattr(N, "_single_gpu_job", lambda: False)
    assert N._mc_cluster(8192, 8192, 16384) is None


def test_single_gpu_job_rules(monkeypatch):
    """The multicast GEMM is for jobs on one GPU: more than one visible device, a launcher that
    announced several ranks (before any process group exists) or an initialised group of several
    ranks all switch it off."""
    import torch

    from float8_experimental_b200 import _native as N

    for var in ("WORLD_SIZE", "LOCAL_WORLD_SIZE"):
        monkeypatch.delenv(var, raising=False)
    monkeypatch.setattr(torch.cuda, "device_count", lambda: 1)
    assert N._single_gpu_job()
    monkeypatch.setattr(torch.cuda, "device_count", lambda: 2)
    assert not N._single_gpu_job()
    monkeypatch.setattr(torch.cuda, "device_count", lambda: 0)
    assert not N._single_gpu_job()
    monkeypatch.setattr(torch.cuda, "device_count", lambda: 1)
    monkeypatch.setenv("WORLD_SIZE", "2")
    assert not N._single_gpu_job()
    monkeypatch.setenv("WORLD_SIZE", "1")
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "8")
    assert not N._single_gpu_job()
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "1")
    assert N._single_gpu_job()
    monkeypatch.setattr(torch.distributed, "is_initialized", lambda: True)
    monkeypatch.setattr(torch.distributed, "get_world_size", lambda *a, **k: 2)
    assert not N._single_gpu_job()


def test_single_node_route_matches_general_route(monkeypatch):
    """A dynamic-scaling Float8Linear on plain tensors runs as ONE autograd node on raw tensors; with
    F8B200_LINEAR_SINGLE_NODE=0 it takes the general route (Float8Tensor operands, one node per cast
    and per product).  Same kernels, same arguments: outputs and gradients are bit-identical, with and
    without bias, for 2-D and 3-D inputs, and when only one of the two gradients is needed."""
    import copy

    import torch
    import torch.nn as nn

    import float8_experimental_b200 as f8
    from float8_experimental_b200.float8_linear import Float8Linear

    torch.manual_seed(3)
    for bias, shape in ((False, (32, 64)), (True, (2, 16, 64))):
        lin = nn.Linear(64, 48, bias=bias).to(torch.bfloat16)
        x = torch.randn(*shape).to(torch.bfloat16)
        go = (torch.randn(*shape[:-1], 48) * 1e-2).to(torch.bfloat16)
        results = []
        for route in ("1", "0"):
            monkeypatch.setenv("F8B200_LINEAR_SINGLE_NODE", route)
            m = Float8Linear.from_float(copy.deepcopy(lin), f8.Float8LinearConfig())
            assert m._single_node_route(x) == (route == "1")
            xr = x.clone().requires_grad_(True)
            y = m(xr)
            y.backward(go)
            results.append((y.detach(), xr.grad, m.weight.grad, m.bias.grad if bias else None))
        for a, b in zip(*results):
            assert (a is None and b is None) or torch.equal(a, b)
    # frozen weight: only the input gradient is computed
    monkeypatch.setenv("F8B200_LINEAR_SINGLE_NODE", "1")
    m = Float8Linear.from_float(nn.Linear(64, 48, bias=False).to(torch.bfloat16), f8.Float8LinearConfig())
    m.weight.requires_grad_(False)
    xr = torch.randn(16, 64).to(torch.bfloat16).requires_grad_(True)
    m(xr).sum().backward()
    assert xr.grad is not None and m.weight.grad is None
    # delayed scaling, autocast and DTensor inputs keep the general route
    d = f8.CastConfig(scaling_type=f8.ScalingType.DELAYED)
    md = Float8Linear.from_float(nn.Linear(64, 48), f8.Float8LinearConfig(cast_config_input=d))
    assert not md._single_node_route(torch.randn(4, 64))
    with torch.autocast("cpu", dtype=torch.bfloat16):
        assert not m._single_node_route(xr.detach())
    # K that is not a multiple of 16 is refused exactly as on the general route
    odd = Float8Linear.from_float(nn.Linear(72, 48, bias=False).to(torch.bfloat16), f8.Float8LinearConfig())
    with pytest.raises(RuntimeError, match="multiple of 16"):
        odd(torch.randn(16, 72).to(torch.bfloat16))


def test_step_timeline_from_a_profiler_trace(tmp_path):
    """`benchmarks.multi_gpu._timeline_of`: busy / idle time of the stream that runs the GEMMs and the idle
    time spent under NCCL kernels of other streams, from a chrome trace (here a hand-made one)."""
    import json

    from float8_experimental_b200.benchmarks import multi_gpu

    def k(name, ts, dur, stream, cat="kernel"):
        return {"name": name, "cat": cat, "ts": ts, "dur": dur, "args": {"stream": stream}}

    events = [
        k("gemm_fp8_pairwide_kernel", 0, 1000, 7), k("cast_tile8_kernel", 1000, 100, 7),
        # 400 us gap on stream 7: an all-gather runs on stream 20 during 300 us of it
        k("ncclDevKernel_AllGather", 1050, 350, 20),
        k("gemm_fp8_pairwide_kernel", 1500, 2000, 7),
        k("ncclDevKernel_ReduceScatter", 2000, 1800, 21),      # overlaps the GEMM, then 300 us exposed
        k("Memset", 3900, 10, 7, cat="gpu_memset"),
        {"name": "cudaLaunchKernel", "cat": "cuda_runtime", "ts": 0, "dur": 5},
    ]

    class FakeProf:
        def export_chrome_trace(self, path):
            with open(path, "w") as f:
                json.dump({"traceEvents": events}, f)

    t = multi_gpu._timeline_of(FakeProf(), steps=2)
    assert t["span_ms_per_step"] == pytest.approx(3.91 / 2)
    assert t["gemm_stream_busy_ms"] == pytest.approx(3.11 / 2)
    assert t["gemm_stream_idle_ms"] == pytest.approx(0.8 / 2)
    # idle [1100, 1500) under the all-gather until 1400; idle [3500, 3900) under the reduce-scatter until 3800
    assert t["idle_while_nccl_runs_ms"] == pytest.approx(0.6 / 2)
    assert t["idle_with_nothing_running_ms"] == pytest.approx(0.2 / 2)
    assert t["largest_idle_gaps_ms"][:2] == [0.4, 0.4]
