"""Row-parallel float8 GEMM fused with the reduce-scatter of its output, over peer memory.

The reference multiplies the local shards and then redistributes the partial products
(`outputs.redistribute(placements=output_layouts)`, float8_experimental/float8_tensor_parallel.py:
116-128): a GEMM that writes the whole [tokens, features] partial product, followed by a bf16
reduce-scatter that reads it again.  Here the GEMM's epilogue stores every row block of the
partial product straight into its owner's receive buffer (its own, or a peer's through mapped
symmetric memory: plain stores over NVLink, issued while later tiles are still being multiplied),
and each rank then adds up the slots it received:

    GEMM with scattered stores          slot `rank` of every owner's receive buffer
    1-element all-reduce                every rank's stores have landed
    sum of the slots (fp32, rank order) this rank's rows of the reduced output

Two receive buffers alternate, so no collective is needed before the GEMM: the buffer a call writes
was last read two calls ago, before the all-reduce of the call in between.

CUDA only (symmetric memory needs peer access between the ranks' GPUs), at most 16 ranks.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from . import _native as N
from ._ops import _gemm_operand
from .float8_tensor import Float8Tensor

__all__ = ["GemmReduceScatter", "rowwise_matmul_reduce_scatter"]


class GemmReduceScatter:
    """`rs = GemmReduceScatter(group, max_out_numel_per_rank, dtype)`;
    `y_local = rs(x8, w8_t, shard_dim)` with `x8` this rank's [..., K / tp] fp8 input shard and
    `w8_t` its [K / tp, N] fp8 weight shard (transposed view) returns this rank's shard, along
    dimension `shard_dim`, of the sum over the ranks of `x8 @ w8_t`."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None, max_out_numel_per_rank: int = 1 << 27,
                 dtype: torch.dtype = torch.bfloat16, device: Optional[torch.device] = None):
        import torch.distributed._symmetric_memory as symm_mem

        # plain peer mappings only: no NVLink multicast object is bound to the buffers
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > 16:
            raise RuntimeError("GemmReduceScatter supports at most 16 ranks")
        self.dtype = dtype
        self.capacity = int(max_out_numel_per_rank)  # elements of one rank's output shard
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.buffers, self.handles = [], []
        for _ in range(2):
            buf = symm_mem.empty(self.world * self.capacity, dtype=dtype, device=device)
            self.buffers.append(buf)
            self.handles.append(symm_mem.rendezvous(buf, self.group))
        self._flag = torch.zeros(1, dtype=torch.float32, device=device)
        self._turn = 0

    def __call__(self, x8: Float8Tensor, w8_t: Float8Tensor, shard_dim: int) -> torch.Tensor:
        lead = tuple(x8.shape[:-1])
        if shard_dim < 0 or shard_dim >= len(lead):
            raise RuntimeError("GemmReduceScatter: the output is sharded on one of the leading dimensions")
        if lead[shard_dim] % self.world != 0:
            raise RuntimeError("GemmReduceScatter: the sharded dimension must divide by the number of ranks")
        out_dtype = x8._orig_dtype
        if out_dtype != self.dtype:
            raise RuntimeError(f"GemmReduceScatter was built for {self.dtype} outputs, got {out_dtype}")
        a = x8._data.reshape(-1, x8.shape[-1])
        m, k = a.shape
        n = w8_t.shape[-1]
        b = w8_t._data.t()  # [N, K / tp]: the logical B operand of out = A . B^T
        inner = 1
        for d in lead[shard_dim + 1:]:
            inner *= d
        rows_per_block = (lead[shard_dim] // self.world) * inner
        shard_numel = (m // self.world) * n
        if shard_numel > self.capacity:
            raise RuntimeError(f"GemmReduceScatter: {shard_numel} output elements per rank, capacity {self.capacity}")
        turn = self._turn
        self._turn ^= 1
        esz = self.buffers[turn].element_size()
        # destination for owner o: slot `rank` of o's receive buffer
        ptrs = [int(self.handles[turn].buffer_ptrs[o]) + self.rank * shard_numel * esz for o in range(self.world)]
        a_op, lda, a_mn = _gemm_operand(a)
        b_op, ldb, b_mn = _gemm_operand(b)
        sa = x8._scale if x8._scale.dtype == torch.float32 else x8._scale.float()
        sb = w8_t._scale if w8_t._scale.dtype == torch.float32 else w8_t._scale.float()
        N.gemm_fp8_scatter_rows(a_op, lda, b_op, ldb, sa, sb, out_dtype, ptrs, rows_per_block, n, m, n, k,
                                a_mn_major=a_mn, b_mn_major=b_mn)
        dist.all_reduce(self._flag, group=self.group)  # every rank's stores into my buffer have landed
        out_shape = list(lead) + [n]
        out_shape[shard_dim] //= self.world
        out = torch.empty(out_shape, dtype=out_dtype, device=a.device)
        N.sum_slots(self.buffers[turn], self.world, shard_numel, shard_numel, out)
        return out


class _RowwiseMatmulReduceScatter(torch.autograd.Function):
    """`input_fp8 @ weight_fp8_t` of a row-parallel linear with the reduce-scatter of the result
    fused into the GEMM.  Inputs are float8 DTensors (input sharded on its last dimension, the
    transposed weight on its first); the output is a high-precision DTensor sharded on
    `shard_dim`.  Backward is the backward of matmul + redistribute: the incoming gradient (cast to
    e5m2 by the caller while still sharded) is all-gathered as fp8 bytes and enters the two float8
    products of `manual_float8_matmul`."""

    @staticmethod
    def forward(ctx, input_fp8, weight_fp8_t, rs: GemmReduceScatter, shard_dim: int):
        from torch.distributed._tensor import DTensor, Shard

        ctx.save_for_backward(input_fp8, weight_fp8_t)
        y = rs(input_fp8.to_local(), weight_fp8_t.to_local(), shard_dim)
        return DTensor.from_local(y, input_fp8.device_mesh, (Shard(shard_dim),), run_check=False)

    @staticmethod
    def backward(ctx, grad_output_fp8):
        from torch.distributed._tensor import Replicate

        input_fp8, weight_fp8_t = ctx.saved_tensors
        g = grad_output_fp8.redistribute(placements=(Replicate(),))
        lead = g.shape[:-1]
        go2d = g.reshape(-1, g.shape[-1])
        grad_input = torch.mm(go2d, weight_fp8_t.t())
        grad_input = grad_input.reshape(*lead, grad_input.shape[-1])
        x2d = input_fp8.reshape(-1, input_fp8.shape[-1])
        grad_weight = torch.mm(go2d.t(), x2d)
        return grad_input, grad_weight.t(), None, None


def rowwise_matmul_reduce_scatter(input_fp8, weight_fp8_t, rs: GemmReduceScatter, shard_dim: int):
    return _RowwiseMatmulReduceScatter.apply(input_fp8, weight_fp8_t, rs, shard_dim)
