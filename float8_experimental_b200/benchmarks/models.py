"""Model fragments the side measurements of the benchmark are run on."""
from __future__ import annotations

import torch.nn as nn


class Llama3Block(nn.Module):
    """The seven linears of a Llama-3-8B decoder block (dim 4096, 8 KV heads of 128, ffn 14336) in
    their data-flow order; attention itself and the norms are left out (they are not float8 work):
    the key / value projections are folded into the query so that every weight gets a gradient."""

    def __init__(self, dim=4096, kv_dim=1024, ffn=14336):
        super().__init__()
        self.wq = nn.Linear(dim, dim, bias=False)
        self.wk = nn.Linear(dim, kv_dim, bias=False)
        self.wv = nn.Linear(dim, kv_dim, bias=False)
        self.wo = nn.Linear(dim, dim, bias=False)
        self.w1 = nn.Linear(dim, ffn, bias=False)
        self.w3 = nn.Linear(dim, ffn, bias=False)
        self.w2 = nn.Linear(ffn, dim, bias=False)
        self.kv_dim = kv_dim

    def forward(self, x):
        q = self.wq(x)
        kv = self.wk(x) + self.wv(x)
        a = q + nn.functional.pad(kv, (0, q.shape[-1] - self.kv_dim))
        h = x + self.wo(a)
        return h + self.w2(nn.functional.silu(self.w1(h)) * self.w3(h))
