"""Dynamic fp8 cast fused with the all-gather of its result, over peer memory.

The reference casts a sharded activation (or weight shard) to fp8 and then all-gathers the
bytes (float8_experimental/float8_tensor_parallel.py:49-60, fsdp_utils.py:168-207).  Here the
cast kernel itself stores every 8-byte group of its result into this rank's slot of the
gathered buffer on EVERY rank: its own buffer and, through peer-mapped symmetric memory,
plain stores over NVLink into the others'.  The bytes never make the round trip through a
local output, a collective's copy-in and a second kernel; two small NCCL collectives order
the stores against the readers:

    amax (local)  ->  all-reduce MAX          also: every rank has finished reading the buffers
    cast + scatter kernel                     writes slot `rank` of all gathered buffers
    1-element all-reduce                      every rank's stores have landed

CUDA only (symmetric memory needs peer access between the ranks' GPUs), at most 16 ranks.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from . import _native as N
from ._ops import _as_matrix, ops
from .float8_tensor import Float8Tensor, GemmInputRole, LinearMMConfig
from .float8_utils import _kind, e4m3_dtype

__all__ = ["CastAllGather", "CastAllGatherPool"]


class CastAllGather:
    """`gather = CastAllGather(group, max_numel_per_rank); y8 = gather(x_local)` returns the
    `Float8Tensor` of the row-wise concatenation of every rank's `x_local` ([rows, cols] each,
    same shape on all ranks), cast with the scale of the global amax.  The result aliases
    the object's gathered buffer: it is valid until the next call."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None, max_numel_per_rank: int = 1 << 27,
                 device: Optional[torch.device] = None):
        import torch.distributed._symmetric_memory as symm_mem

        # plain peer mappings only: no NVLink multicast object is bound to the buffers
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > 16:
            raise RuntimeError("CastAllGather supports at most 16 ranks")
        self.capacity = int(max_numel_per_rank)
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.buffer = symm_mem.empty(self.world * self.capacity, dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.buffer, self.group)
        self._flag = torch.zeros(1, dtype=torch.float32, device=device)
        count = getattr(torch._C, "_storage_Use_Count", None)
        self._idle_use_count = count(self.buffer.untyped_storage()._cdata) if count is not None else 0

    def __call__(self, x: torch.Tensor, float8_dtype: torch.dtype = e4m3_dtype,
                 linear_mm_config: Optional[LinearMMConfig] = None,
                 gemm_input_role: GemmInputRole = GemmInputRole.INPUT) -> Float8Tensor:
        xm, rows, cols, ld = _as_matrix(x)
        n = rows * cols
        if n == 0 or n > self.capacity:
            raise RuntimeError(f"CastAllGather: {n} elements per rank, capacity {self.capacity}")
        amax = ops.amax(xm)
        dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=self.group)
        # slot `rank` of every rank's buffer, this rank's own first
        order = [self.rank] + [p for p in range(self.world) if p != self.rank]
        ptrs = [int(self.handle.buffer_ptrs[p]) + self.rank * n for p in order]
        scale = torch.empty((), dtype=torch.float32, device=x.device)
        N.cast_scatter(xm, rows, cols, ld, amax, scale, _kind(float8_dtype), ptrs, cols)
        dist.all_reduce(self._flag, group=self.group)
        data = self.buffer[: self.world * n].view(float8_dtype).view(self.world * rows, cols)
        return Float8Tensor(data, scale, x.dtype, linear_mm_config or LinearMMConfig(), gemm_input_role)

    def gather_dim(self, x: torch.Tensor, dim: int, float8_dtype: torch.dtype = e4m3_dtype,
                   linear_mm_config: Optional[LinearMMConfig] = None,
                   gemm_input_role: GemmInputRole = GemmInputRole.INPUT) -> Float8Tensor:
        """The same for a shard of any rank-`dim` split: `x` is this rank's shard of a tensor
        sharded on dimension `dim` (same shape on every rank); returns the `Float8Tensor` of the
        whole tensor (dimension `dim` multiplied by the number of ranks).  One cast launch per
        index of the dimensions before `dim` (a [batch, seq / tp, features] activation sharded on
        the sequence takes `batch` launches)."""
        if x.dim() < 2 or dim < 0 or dim >= x.dim() - 1:
            raise RuntimeError("CastAllGather.gather_dim: the sharded dimension must not be the last one")
        x = x if x.is_contiguous() else x.contiguous()
        outer = 1
        for d in x.shape[:dim]:
            outer *= d
        cols = x.shape[-1]
        slab_rows = x.numel() // (outer * cols)  # rows of one contiguous [rows, cols] slab of this shard
        slab = slab_rows * cols
        n = x.numel()
        if n == 0 or n > self.capacity:
            raise RuntimeError(f"CastAllGather: {n} elements per rank, capacity {self.capacity}")
        if outer > 64:
            raise RuntimeError("CastAllGather.gather_dim: more than 64 slabs before the sharded dimension")
        amax = ops.amax(x)
        dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=self.group)
        order = [self.rank] + [p for p in range(self.world) if p != self.rank]
        scale = torch.empty((), dtype=torch.float32, device=x.device)
        flat = x.view(outer, slab_rows, cols)
        for o in range(outer):
            offset = (o * self.world + self.rank) * slab
            ptrs = [int(self.handle.buffer_ptrs[p]) + offset for p in order]
            N.cast_scatter(flat[o], slab_rows, cols, cols, amax, scale, _kind(float8_dtype), ptrs, cols)
        dist.all_reduce(self._flag, group=self.group)
        shape = list(x.shape)
        shape[dim] *= self.world
        data = self.buffer[: self.world * n].view(float8_dtype).view(shape)
        return Float8Tensor(data, scale, x.dtype, linear_mm_config or LinearMMConfig(), gemm_input_role)

    def in_use(self) -> bool:
        """True while a tensor handed out by an earlier call still references the gathered buffer."""
        count = getattr(torch._C, "_storage_Use_Count", None)
        if count is None:
            return False
        return count(self.buffer.untyped_storage()._cdata) > self._idle_use_count


class CastAllGatherPool:
    """`depth` gathered buffers used in turn, so that the bytes of one call stay valid for the next
    `depth - 1` calls.  A float8 linear keeps its fp8 input for the weight gradient, so a
    sequence-parallel input gathered in forward must outlive the call that gathered it: choose
    `depth` >= the number of gathered inputs that are alive at once (forward calls through this pool
    between a forward and its backward, plus one).  Reusing a buffer that a live tensor still
    references raises instead of overwriting it."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None, max_numel_per_rank: int = 1 << 27, depth: int = 2,
                 device: Optional[torch.device] = None):
        if depth < 1:
            raise ValueError("depth must be at least 1")
        self.gathers = [CastAllGather(group, max_numel_per_rank, device) for _ in range(depth)]
        self._next = 0

    def gather_dim(self, x: torch.Tensor, dim: int, **kw) -> Float8Tensor:
        g = self.gathers[self._next]
        if g.in_use():
            raise RuntimeError(
                f"CastAllGatherPool: all {len(self.gathers)} gathered buffers are still referenced by live tensors "
                "(saved for a backward pass that has not run yet); construct the pool with a larger depth")
        self._next = (self._next + 1) % len(self.gathers)
        return g.gather_dim(x, dim, **kw)
