"""Fully sharded data parallelism (ZeRO stage 3) for a stack of blocks: between uses every rank keeps 1/world of each
block's parameters, gradients and optimizer state.

    blocks = [Block(...) for _ in range(L)]
    fsdp = FullyShardedStack(blocks, comm)                   # shards the parameters, frees the full copies
    opt = torch.optim.AdamW(fsdp.shard_parameters(), lr=...)
    y = x
    for b in fsdp.blocks: y = b(y)                           # each block all-gathers its parameters just in time
    loss(y).backward()                                       # ... again before its backward; gradients are reduce-scattered
    opt.step(); opt.zero_grad()

One gather buffer (sized for the largest block) is shared by all blocks, so at most one block's full parameters exist
at a time.  The parameters of a wrapped block are views into that buffer: they hold valid numbers only while their
block is running forward or backward, which the hooks guarantee.  The all-gather writes the buffer from outside
autograd, so the tensors autograd saved for backward are refreshed in place when the block's backward begins.
Gradients are averaged over the ranks (reduce-scatter with the 1/world scale fused) into `.grad` of the shard.
The reference has no training code; this is ZeRO-3 expressed in its AllGather / ReduceScatter.
"""
from __future__ import annotations

from typing import Iterable, List

import torch
import torch.nn as nn

from ..comm import Communicator


class _ShardedBlock:
    def __init__(self, module: nn.Module, comm: Communicator, owner: "FullyShardedStack"):
        self.module, self.comm, self.owner = module, comm, owner
        self.params = [p for p in module.parameters() if p.requires_grad]
        if not self.params:
            raise ValueError("a block without trainable parameters cannot be sharded")
        dt, dev = self.params[0].dtype, self.params[0].device
        if any(p.dtype != dt or p.device != dev for p in self.params):
            raise ValueError("the parameters of a block must share dtype and device")
        n = comm.size
        self.offsets, numel = [], 0
        for p in self.params:
            self.offsets.append(numel)
            numel += (p.numel() + 7) // 8 * 8
        self.numel = (numel + 8 * n - 1) // (8 * n) * (8 * n)
        self.shard_len = self.numel // n
        full = torch.zeros(self.numel, dtype=dt, device=dev)
        for p, off in zip(self.params, self.offsets):
            full[off:off + p.numel()].copy_(p.data.reshape(-1))
        r = comm.rank
        self.shard = nn.Parameter(full[r * self.shard_len:(r + 1) * self.shard_len].clone())
        self.pending = 0
        self.gathered = False

    def attach(self, buffer: torch.Tensor) -> None:
        """Point the block's parameters into the shared gather buffer (their old storage is released)."""
        self.buffer = buffer[: self.numel]
        for p, off in zip(self.params, self.offsets):
            p.data = self.buffer[off:off + p.numel()].view(p.shape)

    def gather(self) -> None:
        self.owner._current = self
        r = self.comm.rank
        mine = self.buffer[r * self.shard_len:(r + 1) * self.shard_len]
        mine.copy_(self.shard.data)                          # in-place all-gather: own slice first
        if self.comm.size > 1:
            self.comm.all_gather(mine, self.buffer)
        self.gathered = True

    def reduce_grads(self) -> None:
        """All parameter gradients of the block exist: pack them, average over ranks, keep this rank's slice."""
        flat = torch.zeros(self.numel, dtype=self.shard.dtype, device=self.shard.device)
        for p, off in zip(self.params, self.offsets):
            if p.grad is not None:
                flat[off:off + p.numel()].copy_(p.grad.reshape(-1))
                p.grad = None
        out = torch.empty(self.shard_len, dtype=flat.dtype, device=flat.device)
        if self.comm.size > 1:
            self.comm.reduce_scatter(flat, out, op="avg")
        else:
            out.copy_(flat)
        self.shard.grad = out if self.shard.grad is None else self.shard.grad + out


class FullyShardedStack(nn.Module):
    """A stack of blocks whose parameters, gradients and optimizer state are sharded over the ranks (ZeRO stage 3)."""

    def __init__(self, blocks: Iterable[nn.Module], comm: Communicator):
        super().__init__()
        self.blocks = nn.ModuleList(list(blocks))
        self.comm = comm
        self._units: List[_ShardedBlock] = [_ShardedBlock(b, comm, self) for b in self.blocks]
        self._current = None
        biggest = max(u.numel for u in self._units)
        u0 = self._units[0]
        if u0.shard.is_cuda and comm.size > 1:
            self._buffer = comm.empty(biggest, u0.shard.dtype)   # symmetric memory: gathered in place by the NVLS / peer kernels
            self._buffer.zero_()
        else:
            self._buffer = torch.zeros(biggest, dtype=u0.shard.dtype, device=u0.shard.device)
        self._shards = nn.ParameterList([u.shard for u in self._units])
        for u, b in zip(self._units, self.blocks):
            u.attach(self._buffer)
            b.register_forward_pre_hook(lambda mod, args, u=u: u.gather())
            b.register_full_backward_pre_hook(lambda mod, grad_out, u=u: self._before_backward(u))
            for p in u.params:
                p.register_post_accumulate_grad_hook(lambda p, u=u: self._on_grad(u))

    def _before_backward(self, u: _ShardedBlock) -> None:
        u.pending = len(u.params)
        if self._current is not u:                           # another block has used the buffer since the forward pass
            u.gather()

    def _on_grad(self, u: _ShardedBlock) -> None:
        u.pending -= 1
        if u.pending == 0:
            u.reduce_grads()

    def forward(self, x):
        for b in self.blocks:
            x = b(x)
        return x

    def shard_parameters(self) -> List[nn.Parameter]:
        """What the optimizer updates: one flat parameter per block holding this rank's 1/world of it."""
        return [u.shard for u in self._units]

    def full_state(self) -> List[torch.Tensor]:
        """Every block's full flat parameter vector (gathered now); for checkpoints and tests."""
        out = []
        for u in self._units:
            u.gather()
            out.append(u.buffer.clone())
        return out
