"""Collectives as differentiable functions of torch tensors: the forward pass calls the library's collective on
the tensor's device (cuda kernels or the tcp transport for cpu tensors), the backward pass calls its transpose.

    all_gather_rows       rows of every rank stacked              <->  reduce_scatter_rows of the gradient
    reduce_scatter_rows   sum over ranks, row block r to rank r   <->  all_gather_rows of the gradient
    all_reduce_sum        sum over ranks                          <->  identity   (the output is used by every rank)
    copy_to_ranks         identity                                <->  all_reduce_sum of the gradient
    all_to_all_rows       row block j goes to rank j              <->  all_to_all_rows of the gradient

These are the building blocks of the tensor-, sequence- and expert-parallel layers in this package.  The reference
offers the collectives only (src/include/coll.h:12-19); it has no model-parallel code.
"""
from __future__ import annotations

import torch

from ..comm import Communicator, group


def _ag(comm: Communicator, x: torch.Tensor) -> torch.Tensor:
    x = x.contiguous()
    out = torch.empty((x.shape[0] * comm.size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    comm.all_gather(x.view(-1), out.view(-1))
    return out


def _rs(comm: Communicator, x: torch.Tensor) -> torch.Tensor:
    x = x.contiguous()
    if x.shape[0] % comm.size:
        raise ValueError(f"{x.shape[0]} rows cannot be scattered over {comm.size} ranks")
    out = torch.empty((x.shape[0] // comm.size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    comm.reduce_scatter(x.view(-1), out.view(-1), op="sum")
    return out


def _ar(comm: Communicator, x: torch.Tensor) -> torch.Tensor:
    out = x.contiguous().clone()
    comm.all_reduce(out.view(-1), op="sum")
    return out


def _a2a(comm: Communicator, x: torch.Tensor) -> torch.Tensor:
    x = x.contiguous()
    if x.shape[0] % comm.size:
        raise ValueError(f"{x.shape[0]} rows cannot be exchanged between {comm.size} ranks")
    out = torch.empty_like(x)
    comm.all_to_all(x.view(-1), out.view(-1))
    return out


class _AllGatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        return _ag(comm, x)

    @staticmethod
    def backward(ctx, g):
        return _rs(ctx.comm, g), None


class _ReduceScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        return _rs(comm, x)

    @staticmethod
    def backward(ctx, g):
        return _ag(ctx.comm, g), None


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm):
        return _ar(comm, x)

    @staticmethod
    def backward(ctx, g):
        return g, None


class _CopyToRanks(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return _ar(ctx.comm, g), None


class _AllToAllRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        return _a2a(comm, x)

    @staticmethod
    def backward(ctx, g):
        return _a2a(ctx.comm, g), None


def all_gather_rows(x: torch.Tensor, comm: Communicator) -> torch.Tensor:
    """[r, ...] on every rank -> [n r, ...], rank order."""
    return x if comm.size == 1 else _AllGatherRows.apply(x, comm)


def reduce_scatter_rows(x: torch.Tensor, comm: Communicator) -> torch.Tensor:
    """[n r, ...] on every rank -> the sum over ranks of row block `rank`, [r, ...]."""
    return x if comm.size == 1 else _ReduceScatterRows.apply(x, comm)


def all_reduce_sum(x: torch.Tensor, comm: Communicator) -> torch.Tensor:
    """Sum over the ranks; the gradient passes through unchanged (every rank uses the result)."""
    return x if comm.size == 1 else _AllReduceSum.apply(x, comm)


def copy_to_ranks(x: torch.Tensor, comm: Communicator) -> torch.Tensor:
    """Marks a tensor that every rank of the group consumes with different weights: its gradient is the sum of the
    ranks' gradients."""
    return x if comm.size == 1 else _CopyToRanks.apply(x, comm)


def all_to_all_rows(x: torch.Tensor, comm: Communicator) -> torch.Tensor:
    """[n b, ...]: row block j goes to rank j; the result's row block i came from rank i."""
    return x if comm.size == 1 else _AllToAllRows.apply(x, comm)


def ring_shift(comm: Communicator, tensors):
    """Every tensor goes to rank + 1 and is replaced by the one from rank - 1 (one grouped Send / Recv pair per
    tensor, so the ring cannot stall on the transport's buffering).  Not differentiable: ring attention below
    moves its gradients around explicitly."""
    n, r = comm.size, comm.rank
    outs = [torch.empty_like(t) for t in tensors]
    with group():
        for t, o in zip(tensors, outs):
            comm.send(t.contiguous().view(-1), (r + 1) % n)
            comm.recv(o.view(-1), (r - 1) % n)
    return outs


class _RingAttention(torch.autograd.Function):
    """Blockwise attention over a sequence sharded across the ranks: the key / value blocks travel around the ring
    while every rank folds them into its queries' output with a running log-sum-exp, so no rank ever holds more
    than two blocks.  The backward pass sends the blocks around once more together with their gradients."""

    @staticmethod
    def forward(ctx, q, k, v, comm, causal):
        n, r = comm.size, comm.rank
        scale = q.shape[-1] ** -0.5
        qh = q.transpose(0, 1).float()                                   # [heads, s, d]
        out = torch.zeros_like(qh)
        lse = torch.full(qh.shape[:2], float("-inf"), device=q.device)
        kb, vb = k.contiguous(), v.contiguous()
        for step in range(n):
            src = (r - step) % n                                         # whose block this is
            if not causal or src <= r:
                s = torch.einsum("hqd,hkd->hqk", qh, kb.transpose(0, 1).float()) * scale
                if causal and src == r:
                    s = s.masked_fill(torch.ones(s.shape[-2:], dtype=torch.bool, device=s.device).triu(1), float("-inf"))
                blk_lse = torch.logsumexp(s, dim=-1)
                new_lse = torch.logaddexp(lse, blk_lse)
                p = torch.exp(s - new_lse.unsqueeze(-1))
                out = out * torch.exp(lse - new_lse).unsqueeze(-1) + torch.einsum("hqk,hkd->hqd", p, vb.transpose(0, 1).float())
                lse = new_lse
            if step + 1 < n:
                kb, vb = ring_shift(comm, [kb, vb])
        ctx.comm, ctx.causal, ctx.scale = comm, causal, scale
        o = out.transpose(0, 1).to(q.dtype)
        ctx.save_for_backward(q, k, v, o, lse)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        comm, causal, scale = ctx.comm, ctx.causal, ctx.scale
        n, r = comm.size, comm.rank
        qh, doh = q.transpose(0, 1).float(), do.transpose(0, 1).float()
        delta = (doh * o.transpose(0, 1).float()).sum(-1)                # [heads, s]
        dq = torch.zeros_like(qh)
        kb, vb = k.contiguous(), v.contiguous()
        dkb, dvb = torch.zeros_like(kb, dtype=torch.float32), torch.zeros_like(vb, dtype=torch.float32)
        for step in range(n):
            src = (r - step) % n
            if not causal or src <= r:
                kh, vh = kb.transpose(0, 1).float(), vb.transpose(0, 1).float()
                s = torch.einsum("hqd,hkd->hqk", qh, kh) * scale
                if causal and src == r:
                    s = s.masked_fill(torch.ones(s.shape[-2:], dtype=torch.bool, device=s.device).triu(1), float("-inf"))
                p = torch.exp(s - lse.unsqueeze(-1))
                dvb += torch.einsum("hqk,hqd->hkd", p, doh).transpose(0, 1)
                ds = p * (torch.einsum("hqd,hkd->hqk", doh, vh) - delta.unsqueeze(-1))
                dq += torch.einsum("hqk,hkd->hqd", ds, kh) * scale
                dkb += (torch.einsum("hqk,hqd->hkd", ds, qh) * scale).transpose(0, 1)
            # the block moves on with its gradients; after the last step it is back at its owner
            kb, vb, dkb, dvb = ring_shift(comm, [kb, vb, dkb, dvb])
        return dq.transpose(0, 1).to(q.dtype), dkb.to(k.dtype), dvb.to(v.dtype), None, None


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, comm: Communicator, causal: bool = True) -> torch.Tensor:
    """q, k, v: this rank's [tokens / n, heads, head_dim] block of the sequence (rank order = sequence order)."""
    return _RingAttention.apply(q, k, v, comm, causal)
