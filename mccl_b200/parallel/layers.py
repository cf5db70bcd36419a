"""Trainable model-parallel layers on top of the differentiable collectives (`functional.py`):

    ColumnParallelLinear / RowParallelLinear / TensorParallelMLP   tensor parallelism, optionally with the
                                                                   activations sharded over tokens between the two
                                                                   (Megatron-style sequence parallelism)
    UlyssesAttention                                               sequence parallel attention: all-to-all from
                                                                   token shards to head shards and back
    RingAttention                                                  context parallel attention: key / value blocks
                                                                   travel around the ring of ranks
    ExpertParallelMoE                                              top-1 routed experts spread over the ranks,
                                                                   dispatch and combine by all-to-all

They run on whatever device their tensors live on: cuda tensors use the library's kernels, cpu tensors the tcp
transport (which is how they are tested without a GPU).  The inference-only `TensorParallelFFN` in `tp.py` is the
fused-kernel form of TensorParallelMLP's forward pass.  The reference has none of this: its AllToAll and Send/Recv
(src/coll/coll.cc:90-106, src/p2p.cc:202-216) are the primitives these layers are made of.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..comm import Communicator
from . import functional as PF


class ColumnParallelLinear(nn.Module):
    """y[:, slice_r] = x @ W[slice_r].T: every rank holds out_features / n rows of the weight.  With
    `sequence_parallel` the input arrives sharded over tokens and is all-gathered first."""

    def __init__(self, comm: Communicator, in_features: int, out_features: int, bias: bool = True,
                 sequence_parallel: bool = False, device=None, dtype=None):
        super().__init__()
        if out_features % comm.size:
            raise ValueError("out_features must be divisible by the number of ranks")
        self.comm, self.sequence_parallel = comm, sequence_parallel
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features // comm.size, in_features, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_features // comm.size, device=device, dtype=dtype)) if bias else None
        nn.init.normal_(self.weight, std=in_features ** -0.5)

    @torch.no_grad()
    def load_full(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        """Copy this rank's rows of a full [out_features, in_features] weight (and bias)."""
        r, m = self.comm.rank, self.out_features // self.comm.size
        self.weight.copy_(weight[r * m:(r + 1) * m])
        if self.bias is not None and bias is not None:
            self.bias.copy_(bias[r * m:(r + 1) * m])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = PF.all_gather_rows(x, self.comm) if self.sequence_parallel else PF.copy_to_ranks(x, self.comm)
        return F.linear(x, self.weight, self.bias)


class RowParallelLinear(nn.Module):
    """y = sum_r x[:, slice_r] @ W[:, slice_r].T: every rank holds in_features / n columns of the weight and a
    matching slice of the input; the partial products are all-reduced, or reduce-scattered over tokens with
    `sequence_parallel`.  The bias is added once, after the reduction."""

    def __init__(self, comm: Communicator, in_features: int, out_features: int, bias: bool = True,
                 sequence_parallel: bool = False, device=None, dtype=None):
        super().__init__()
        if in_features % comm.size:
            raise ValueError("in_features must be divisible by the number of ranks")
        self.comm, self.sequence_parallel = comm, sequence_parallel
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features // comm.size, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None
        nn.init.normal_(self.weight, std=in_features ** -0.5)

    @torch.no_grad()
    def load_full(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        """Copy this rank's columns of a full [out_features, in_features] weight (and the whole bias)."""
        r, m = self.comm.rank, self.in_features // self.comm.size
        self.weight.copy_(weight[:, r * m:(r + 1) * m])
        if self.bias is not None and bias is not None:
            self.bias.copy_(bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = F.linear(x, self.weight)
        y = PF.reduce_scatter_rows(y, self.comm) if self.sequence_parallel else PF.all_reduce_sum(y, self.comm)
        return y if self.bias is None else y + self.bias


class TensorParallelMLP(nn.Module):
    """down(act(up(x))) with the hidden dimension split over the ranks.  With `sequence_parallel` input and output
    are [tokens / n, hidden] shards; otherwise they are replicated [tokens, hidden] tensors.  The gradient of a
    replicated bias of the down projection is the same on every rank; with sequence parallelism it is this rank's
    share and must be summed over the ranks by the caller's gradient reduction."""

    def __init__(self, comm: Communicator, hidden: int, ffn: int, act: Callable = F.silu, bias: bool = False,
                 sequence_parallel: bool = True, device=None, dtype=None):
        super().__init__()
        self.up = ColumnParallelLinear(comm, hidden, ffn, bias, sequence_parallel, device, dtype)
        self.down = RowParallelLinear(comm, ffn, hidden, bias, sequence_parallel, device, dtype)
        self.act = act

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down(self.act(self.up(x)))


class UlyssesAttention(nn.Module):
    """Self-attention over a sequence sharded across the ranks.  Every rank holds [tokens / n, heads, head_dim]
    of q, k and v; one all-to-all turns that into [tokens, heads / n, head_dim] (all tokens, a share of the heads),
    attention runs locally, and a second all-to-all restores the token sharding."""

    def __init__(self, comm: Communicator, heads: int, causal: bool = True):
        super().__init__()
        if heads % comm.size:
            raise ValueError("heads must be divisible by the number of ranks")
        self.comm, self.heads, self.causal = comm, heads, causal

    def _to_heads(self, t: torch.Tensor) -> torch.Tensor:
        n = self.comm.size
        s, h, d = t.shape
        t = t.view(s, n, h // n, d).permute(1, 0, 2, 3).contiguous()          # block j = head group j
        return PF.all_to_all_rows(t, self.comm).view(n * s, h // n, d)         # block i = rank i's tokens

    def _to_tokens(self, t: torch.Tensor) -> torch.Tensor:
        n = self.comm.size
        s_all, hl, d = t.shape
        t = PF.all_to_all_rows(t.view(n, s_all // n, hl, d).contiguous(), self.comm)   # block i = head group i
        return t.permute(1, 0, 2, 3).reshape(s_all // n, n * hl, d)

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        q, k, v = self._to_heads(q), self._to_heads(k), self._to_heads(v)      # [tokens, heads / n, d]
        o = F.scaled_dot_product_attention(q.transpose(0, 1).unsqueeze(0), k.transpose(0, 1).unsqueeze(0),
                                           v.transpose(0, 1).unsqueeze(0), is_causal=self.causal)
        return self._to_tokens(o.squeeze(0).transpose(0, 1).contiguous())


class RingAttention(nn.Module):
    """Context-parallel self-attention: the sequence stays sharded over the ranks and the key / value blocks travel
    around the ring (`functional.ring_attention`); memory per rank is independent of the number of ranks, and any
    number of heads works (Ulysses needs heads divisible by the ranks)."""

    def __init__(self, comm: Communicator, causal: bool = True):
        super().__init__()
        self.comm, self.causal = comm, causal

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        return PF.ring_attention(q, k, v, self.comm, self.causal)


class ExpertParallelMoE(nn.Module):
    """Top-1 routed mixture of experts, `experts_per_rank` experts on each of the n ranks.  A token goes to the
    expert with the largest router probability and is weighted by it.  Every (source rank, expert) pair has
    `capacity` slots per step; tokens beyond it are dropped (their output is zero), so the dispatch and the combine
    are all-to-alls of equal blocks."""

    def __init__(self, comm: Communicator, hidden: int, ffn: int, experts_per_rank: int, capacity: int, device=None, dtype=None,
                 fused: bool = False):
        super().__init__()
        self.comm, self.hidden, self.capacity = comm, hidden, capacity
        # fused: on cuda tensors the dispatch and the combine are single kernels that move each token row straight
        # between the activation tensor and its slot on the expert's rank (ops/moe.py) instead of pack + all-to-all + unpack
        self.fused = fused
        self._buf = self._grad_buf = None
        self.local, self.experts = experts_per_rank, experts_per_rank * comm.size
        self.router = nn.Linear(hidden, self.experts, bias=False, device=device, dtype=dtype)
        self.w_in = nn.Parameter(torch.empty(experts_per_rank, ffn, hidden, device=device, dtype=dtype))
        self.w_out = nn.Parameter(torch.empty(experts_per_rank, hidden, ffn, device=device, dtype=dtype))
        nn.init.normal_(self.w_in, std=hidden ** -0.5)
        nn.init.normal_(self.w_out, std=ffn ** -0.5)

    def route(self, x: torch.Tensor):
        """expert, gate, slot and keep-mask of every token of this rank."""
        probs = F.softmax(self.router(x).float(), dim=-1)
        gate, expert = probs.max(dim=-1)
        onehot = F.one_hot(expert, self.experts)
        slot = (onehot.cumsum(0) * onehot).sum(-1) - 1                         # position among the tokens of its expert
        return expert, gate.to(x.dtype), slot, slot < self.capacity

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        n, e, c, d = self.comm.size, self.local, self.capacity, self.hidden
        expert, gate, slot, keep = self.route(x)
        flat = expert * c + slot                                               # slot in the [experts, capacity] grid
        if self.fused and x.is_cuda:
            from ..ops import moe as M
            if self._buf is None:                                              # collective allocations, first call
                self._buf = M.ExchangeBuffer(self.comm, e, c, d, x.dtype)
                self._grad_buf = M.ExchangeBuffer(self.comm, e, c, d, x.dtype)
            flat32 = torch.where(keep, flat, torch.full_like(flat, -1)).to(torch.int32)
            recv = M.dispatch(x, flat32, self._buf, self._grad_buf)            # [n (source), e, c, d]
            tokens = recv.transpose(0, 1).reshape(e, n * c, d)
            hidden = F.silu(torch.einsum("etd,efd->etf", tokens, self.w_in))
            out = torch.einsum("etf,edf->etd", hidden, self.w_out)
            back = out.view(e, n, c, d).transpose(0, 1).contiguous()
            return M.combine(back, flat32, gate, self._buf, self._grad_buf)
        send = x.new_zeros(self.experts * c, d)
        send = send.index_put((flat[keep],), x[keep])
        recv = PF.all_to_all_rows(send, self.comm)                             # [n (source), e, c, d]
        tokens = recv.view(n, e, c, d).transpose(0, 1).reshape(e, n * c, d)    # per local expert: all sources' slots
        hidden = F.silu(torch.einsum("etd,efd->etf", tokens, self.w_in))
        out = torch.einsum("etf,edf->etd", hidden, self.w_out)
        back = out.view(e, n, c, d).transpose(0, 1).reshape(n * e * c, d)      # block j returns to source rank j
        got = PF.all_to_all_rows(back, self.comm)                              # [experts * c, d], this rank's slots
        y = x.new_zeros(x.shape)
        return y.index_put((keep.nonzero(as_tuple=True)[0],), got[flat[keep]] * gate[keep].unsqueeze(-1))


def moe_reference(x: torch.Tensor, router_w: torch.Tensor, w_in: torch.Tensor, w_out: torch.Tensor, capacity: int) -> torch.Tensor:
    """Dense restatement of ExpertParallelMoE for one rank's tokens: w_in / w_out hold ALL experts ([E, ffn, hidden],
    [E, hidden, ffn]); the capacity rule is applied to this rank's tokens as the layer applies it."""
    probs = F.softmax((x @ router_w.t()).float(), dim=-1)
    gate, expert = probs.max(dim=-1)
    onehot = F.one_hot(expert, router_w.shape[0])
    slot = (onehot.cumsum(0) * onehot).sum(-1) - 1
    keep = slot < capacity
    h = F.silu(torch.einsum("td,tfd->tf", x, w_in[expert]))
    y = torch.einsum("tf,tdf->td", h, w_out[expert]) * gate.to(x.dtype).unsqueeze(-1)
    return y * keep.unsqueeze(-1)


def attention_reference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True) -> torch.Tensor:
    """[tokens, heads, d] attention on one process."""
    o = F.scaled_dot_product_attention(q.transpose(0, 1).unsqueeze(0), k.transpose(0, 1).unsqueeze(0),
                                       v.transpose(0, 1).unsqueeze(0), is_causal=causal)
    return o.squeeze(0).transpose(0, 1)


__all__ = ["ColumnParallelLinear", "RowParallelLinear", "TensorParallelMLP", "UlyssesAttention", "RingAttention", "ExpertParallelMoE",
           "moe_reference", "attention_reference"]
