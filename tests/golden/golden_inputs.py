"""Seeded synthetic inputs shared by the fixture generator and the tests."""
from __future__ import annotations

import hashlib

import numpy as np
import torch


def sha256(arr: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(arr).tobytes()).hexdigest()


def config1_inputs():
    """The small reference configuration (one 4096x4096 layer, 2048 tokens): x bf16 [2048, 4096] ~ N(0,1) with 0.1 % of the elements (seeded
    positions) multiplied by 100; weight bf16 [4096, 4096] ~ N(0, 0.02); grad_output bf16
    [2048, 4096] ~ N(0, 1e-3).  CPU generators, so every machine with the same torch
    build produces the same bits (the fixture stores digests to detect drift)."""
    g = torch.Generator().manual_seed(20240801)
    x = torch.randn(2048, 4096, generator=g)
    n_out = x.numel() // 1000
    pos = torch.randperm(x.numel(), generator=g)[:n_out]
    x.view(-1)[pos] *= 100.0
    w = torch.randn(4096, 4096, generator=g) * 0.02
    go = torch.randn(2048, 4096, generator=g) * 1e-3
    return x.to(torch.bfloat16), w.to(torch.bfloat16), go.to(torch.bfloat16)
