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

from ..comm import Communicator


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
    return x if comm.size == 1 else _AllReduceSum.apply(x, comm)


def copy_to_ranks(x: torch.Tensor, comm: Communicator) -> torch.Tensor:
    """Marks a tensor that every rank of the group consumes with different weights: its gradient is the sum of the
    ranks' gradients."""
    return x if comm.size == 1 else _CopyToRanks.apply(x, comm)


def all_to_all_rows(x: torch.Tensor, comm: Communicator) -> torch.Tensor:
    """[n b, ...]: row block j goes to rank j; the result's row block i came from rank i."""
    return x if comm.size == 1 else _AllToAllRows.apply(x, comm)
