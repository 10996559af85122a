"""Multi-rank host logic on CPU: two `gloo` ranks, kernels replaced by the oracle-backed
stand-ins.  Covers the delayed-scaling sync all-reduce, FSDP2 fp8 all-gather (dynamic with
and without precomputed scales, delayed) and DTensor tensor/sequence parallelism."""
import os
import socket
import sys

import pytest
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
WORLD = 2


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, case, world, port, extra):
    for p in (os.path.dirname(HERE), HERE, os.path.join(HERE, "golden")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import dist_cases

    getattr(dist_cases, case)(rank, world, port, *extra)


def _run(case, *extra):
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


def test_sequence_parallel_with_fused_reduce_scatter_route():
    """The row-parallel layer's fused GEMM + reduce-scatter route (host side; the peer-memory GEMM is
    replaced by a stand-in on CPU ranks) still equals the unsharded model."""
    _run("case_tensor_parallel", True, True)


@pytest.mark.parametrize("weight_dynamic", [False, True])
def test_fsdp1_flat_parameter_wrapper_composes_with_float8_linear(weight_dynamic):
    _run("case_fsdp1_composition", weight_dynamic)
