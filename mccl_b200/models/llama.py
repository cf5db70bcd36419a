"""Llama-style decoder (RMSNorm, rotary position embedding, SwiGLU) with tensor parallelism built in: the q / k / v
and gate / up projections are column parallel, the output and down projections row parallel, so every rank holds
1/n of each block's matrices and n_head / n attention heads.  With `sequence_parallel` the residual stream between
the blocks is sharded over tokens (all-gather before a block's first projection, reduce-scatter after its last), as in
Megatron's sequence parallelism; otherwise it is replicated and the partial sums are all-reduced.

    comm = mccl.Communicator(world, uid, rank)                      # or a split of a larger one
    model = Llama(LlamaConfig.tiny(), comm)
    model.load_full(full_state)                                      # slices a single-process state dict
    loss = model(tokens, targets); loss.backward()

The embedding, the norms and the output head are replicated; their gradients (and those of sequence-parallel norms)
are per-rank shares that `reduce_replicated_grads` sums over the tensor-parallel group.  A communicator of size 1
gives the plain single-process model, which is what the tests compare against.  The reference has no models; this
one exists to exercise the tensor-parallel layers end to end.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..comm import Communicator
from ..parallel import functional as PF
from ..parallel.layers import ColumnParallelLinear, RowParallelLinear


@dataclass
class LlamaConfig:
    n_layer: int = 32
    d_model: int = 4096
    n_head: int = 32
    d_ff: int = 11008
    vocab_size: int = 32000
    seq_len: int = 2048
    rope_theta: float = 10000.0
    eps: float = 1e-5

    @staticmethod
    def tiny() -> "LlamaConfig":
        return LlamaConfig(n_layer=2, d_model=64, n_head=4, d_ff=128, vocab_size=256, seq_len=32)


class RMSNorm(nn.Module):
    """x / rms(x) * weight, statistics in fp32."""

    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        v = x.float()
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


def rope(x: torch.Tensor, theta: float) -> torch.Tensor:
    """x: [batch, seq, heads, d]; rotates pairs (i, i + d/2) by position-dependent angles."""
    b, s, h, d = x.shape
    half = d // 2
    freqs = theta ** (-torch.arange(half, device=x.device, dtype=torch.float32) / half)
    ang = torch.arange(s, device=x.device, dtype=torch.float32)[:, None] * freqs[None, :]
    cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    x1, x2 = x[..., :half].float(), x[..., half:].float()
    return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1).to(x.dtype)


class Block(nn.Module):
    """Pre-norm attention + SwiGLU block holding 1/n of every projection."""

    def __init__(self, cfg: LlamaConfig, comm: Communicator, sp: bool):
        super().__init__()
        n = comm.size
        if cfg.n_head % n or cfg.d_ff % n:
            raise ValueError("heads and d_ff must be divisible by the tensor-parallel size")
        self.cfg, self.comm, self.sp = cfg, comm, sp
        self.heads_local, self.head_dim = cfg.n_head // n, cfg.d_model // cfg.n_head
        d, f = cfg.d_model, cfg.d_ff
        self.norm1, self.norm2 = RMSNorm(d, cfg.eps), RMSNorm(d, cfg.eps)
        # the first projection of a group gathers (or marks) the input once; its siblings reuse the gathered tensor
        self.q = ColumnParallelLinear(comm, d, d, bias=False, sequence_parallel=sp)
        self.k = ColumnParallelLinear(comm, d, d, bias=False)
        self.v = ColumnParallelLinear(comm, d, d, bias=False)
        self.o = RowParallelLinear(comm, d, d, bias=False, sequence_parallel=sp)
        self.gate = ColumnParallelLinear(comm, d, f, bias=False, sequence_parallel=sp)
        self.up = ColumnParallelLinear(comm, d, f, bias=False)
        self.down = RowParallelLinear(comm, f, d, bias=False, sequence_parallel=sp)

    def _enter(self, x: torch.Tensor) -> torch.Tensor:
        """[batch*seq (/ n), d] -> the full token set every rank's weight shards are applied to."""
        return PF.all_gather_rows(x, self.comm) if self.sp else PF.copy_to_ranks(x, self.comm)

    def forward(self, x: torch.Tensor, batch: int, seq: int) -> torch.Tensor:
        h = self._enter(self.norm1(x))
        q, k, v = (F.linear(h, m.weight).view(batch, seq, self.heads_local, self.head_dim) for m in (self.q, self.k, self.v))
        q, k = rope(q, self.cfg.rope_theta), rope(k, self.cfg.rope_theta)
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        x = x + self.o(a.transpose(1, 2).reshape(batch * seq, -1))
        h = self._enter(self.norm2(x))
        return x + self.down(F.silu(F.linear(h, self.gate.weight)) * F.linear(h, self.up.weight))


class Llama(nn.Module):
    """Tensor-parallel Llama-style decoder on `comm`; forward(idx, targets) returns the mean cross-entropy over all
    tokens (the same value on every rank), forward(idx) the logits of this rank's tokens."""

    def __init__(self, cfg: LlamaConfig, comm: Communicator, sequence_parallel: bool = False):
        super().__init__()
        self.cfg, self.comm, self.sp = cfg, comm, sequence_parallel and comm.size > 1
        self.embed = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.blocks = nn.ModuleList([Block(cfg, comm, self.sp) for _ in range(cfg.n_layer)])
        self.norm = RMSNorm(cfg.d_model, cfg.eps)
        self.head = nn.Linear(cfg.d_model, cfg.vocab_size, bias=False)

    def forward(self, idx: torch.Tensor, targets: Optional[torch.Tensor] = None) -> torch.Tensor:
        b, s = idx.shape
        n, r = self.comm.size, self.comm.rank
        x = self.embed(idx).view(b * s, -1)
        if self.sp:                                       # this rank's rows of the flattened (batch, seq) tokens
            rows = b * s // n
            x = x[r * rows:(r + 1) * rows]
        for blk in self.blocks:
            x = blk(x, b, s)
        logits = self.head(self.norm(x))
        if targets is None:
            return logits
        t = targets.reshape(-1)
        if self.sp:
            t = t[r * rows:(r + 1) * rows]
            # mean over ALL tokens: every rank contributes the sum over its rows
            return PF.all_reduce_sum(F.cross_entropy(logits.float(), t, reduction="sum"), self.comm) / (b * s)
        return F.cross_entropy(logits.float(), t)

    # ---- weights
    @torch.no_grad()
    def load_full(self, state: Dict[str, torch.Tensor]) -> None:
        """Load a single-process state dict (as produced by a Llama on a communicator of size 1), slicing the
        column / row parallel matrices for this rank."""
        own = dict(self.named_parameters())
        n, r = self.comm.size, self.comm.rank
        for name, p in own.items():
            full = state[name]
            leaf = name.split(".")[-2] if "." in name else ""
            if leaf in ("q", "k", "v", "gate", "up"):
                m = full.shape[0] // n
                p.copy_(full[r * m:(r + 1) * m])
            elif leaf in ("o", "down"):
                m = full.shape[1] // n
                p.copy_(full[:, r * m:(r + 1) * m])
            else:
                p.copy_(full)

    def reduce_replicated_grads(self) -> None:
        """Sum over the tensor-parallel group the gradients that are per-rank shares: with sequence parallelism every
        replicated parameter (embedding, norms, head) sees only this rank's tokens."""
        if not self.sp:
            return
        for name, p in self.named_parameters():
            leaf = name.split(".")[-2] if "." in name else ""
            if leaf not in ("q", "k", "v", "gate", "up", "o", "down") and p.grad is not None:
                self.comm.all_reduce(p.grad.view(-1), op="sum")
