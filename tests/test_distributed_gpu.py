"""The multi-rank cases of `dist_cases.py` on real GPUs: two NCCL ranks, one B200 each,
the CUDA kernels instead of the CPU stand-ins.  Skipped with fewer than two GPUs."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
WORLD = int(os.environ.get("F8_DIST_WORLD", "2"))  # ranks = GPUs used by every case


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, case, world, port, extra):
    os.environ["F8_DIST_DEVICE"] = "cuda"
    for p in (os.path.dirname(HERE), HERE, os.path.join(HERE, "golden")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import dist_cases

    getattr(dist_cases, case)(rank, world, port, *extra)


def _run(case, *extra):
    if torch.cuda.device_count() < WORLD:
        pytest.skip(f"needs {WORLD} GPUs")
    for attempt in range(3):  # the probed port can be taken again before rank 0 listens on it
        try:
            mp.spawn(_entry, args=(case, WORLD, _free_port(), extra), nprocs=WORLD, join=True)
            return
        except Exception as exc:  # noqa: BLE001
            if "EADDRINUSE" not in str(exc) or attempt == 2:
                raise


def test_sync_all_reduces_amaxes_once():
    _run("case_sync_all_reduce")


@pytest.mark.parametrize("precompute", [False, True])
def test_fsdp2_fp8_all_gather_matches_unsharded(precompute):
    _run("case_fsdp2_fp8_all_gather", precompute)


def test_fsdp2_precompute_that_also_casts_all_shards_at_once():
    """precompute(cast_now=True): one multi-tensor cast after the optimizer step, the all-gathers
    hand over the cached bytes; still loss for loss the unsharded model."""
    _run("case_fsdp2_fp8_all_gather", True, True)


def test_fsdp2_delayed_weight_scaling():
    _run("case_fsdp2_delayed")


@pytest.mark.parametrize("sequence_parallel", [False, True])
def test_tensor_parallel_matches_unsharded(sequence_parallel):
    _run("case_tensor_parallel", sequence_parallel)


def test_cast_all_gather_over_peer_memory():
    _run("case_cast_all_gather_over_peer_memory")


@pytest.mark.parametrize("name", ["fsdp2", "tp", "sp", "delayed_sync", "cast_all_gather", "sp_cast_all_gather",
                                  "sp_fused_reduce_scatter"])
def test_benchmark_parity_checks(name):
    """Each check of the block that `bench.py --gpus N` runs before timing (N > 1), here on two ranks."""
    _run("case_package_parity", name)


@pytest.mark.parametrize("weight_dynamic", [False, True])
def test_fsdp1_flat_parameter_wrapper_composes_with_float8_linear(weight_dynamic):
    _run("case_fsdp1_composition", weight_dynamic)
