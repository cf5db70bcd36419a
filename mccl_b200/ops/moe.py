"""Expert-parallel token exchange fused with the routing gather / scatter (csrc/device/moe.cu): one kernel moves
every token row straight between its place in the local activation tensor and its slot in the expert's rank, over
NVLink, instead of packing a send buffer, running an all-to-all and unpacking.

    buf, gbuf = (ExchangeBuffer(comm, experts_per_rank, capacity, hidden, dtype) for _ in range(2))   # symmetric, collective
    tokens_at_experts = dispatch(x, flat, buf, gbuf)                             # [n, e, c, d]: a copy of the filled buffer
    y = combine(expert_out, flat, gate, buf, gbuf)                               # [T, d]; gbuf carries gradients in backward

Both are differentiable: the backward pass of a dispatch is a combine of the gradient buffer and vice versa (the
gate's gradient is the dot product of the output gradient with the unscaled expert row).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import _lib as L
from ..comm import Communicator

_counter = {"launches": 0}
_DT = {torch.float32: L.FLOAT32, torch.bfloat16: L.BFLOAT16, torch.float16: L.FLOAT16}


def launches() -> int:
    return _counter["launches"]


def _lib():
    lib = L.load()
    if not getattr(lib, "_moe_declared", False):
        vp, i = C.c_void_p, C.c_int
        for f in (lib.mcclMoeScatter, lib.mcclMoeGather):
            f.restype = i
            f.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, vp]
        lib._moe_declared = True
    return lib


def _stream(t):
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


class ExchangeBuffer:
    """[ranks, experts_per_rank, capacity, hidden] in symmetric memory on every rank (a collective allocation)."""

    def __init__(self, comm: Communicator, experts_per_rank: int, capacity: int, hidden: int, dtype=torch.bfloat16):
        if hidden * torch.empty((), dtype=dtype).element_size() % 16:
            raise ValueError("a token row must be a multiple of 16 bytes")
        self.comm, self.e, self.c, self.d, self.dtype = comm, experts_per_rank, capacity, hidden, dtype
        self.data = comm.empty((comm.size, experts_per_rank, capacity, hidden), dtype)
        self.row_bytes = hidden * self.data.element_size()


def _scatter(buf: ExchangeBuffer, x: torch.Tensor, flat: torch.Tensor, scale: Optional[torch.Tensor]) -> None:
    assert x.is_cuda and x.is_contiguous() and x.dtype == buf.dtype and flat.dtype == torch.int32 and flat.is_contiguous()
    assert x.dim() == 2 and x.shape[1] == buf.d and flat.numel() == x.shape[0] and (scale is None or (scale.numel() == x.shape[0] and scale.dtype == torch.float32))
    sp = scale.data_ptr() if scale is not None else None
    L.check(_lib().mcclMoeScatter(C.c_void_p(buf.comm.handle), x.data_ptr(), flat.data_ptr(), sp, buf.data.data_ptr(), x.shape[0],
                                  buf.row_bytes, buf.e, buf.c, _DT[buf.dtype], _stream(x)), "mcclMoeScatter")
    _counter["launches"] += 1


def _gather(buf: ExchangeBuffer, flat: torch.Tensor, scale: Optional[torch.Tensor], n_tokens: int) -> torch.Tensor:
    assert flat.dtype == torch.int32 and flat.is_contiguous() and flat.numel() == n_tokens
    assert scale is None or (scale.numel() == n_tokens and scale.dtype == torch.float32 and scale.is_contiguous())
    out = torch.empty(n_tokens, buf.d, device=buf.data.device, dtype=buf.dtype)
    sp = scale.data_ptr() if scale is not None else None
    L.check(_lib().mcclMoeGather(C.c_void_p(buf.comm.handle), buf.data.data_ptr(), flat.data_ptr(), sp, out.data_ptr(), n_tokens,
                                 buf.row_bytes, buf.e, buf.c, _DT[buf.dtype], _stream(out)), "mcclMoeGather")
    _counter["launches"] += 1
    return out


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, flat, buf, grad_buf):
        ctx.buf, ctx.n = grad_buf, x.shape[0]
        ctx.save_for_backward(flat)
        _scatter(buf, x.contiguous(), flat, None)
        return buf.data.clone()                      # the buffer is reused by the next call; autograd keeps a copy

    @staticmethod
    def backward(ctx, g):
        (flat,) = ctx.saved_tensors
        ctx.buf.data.copy_(g)                        # the gradient of every slot, where the peers can read it
        return _gather(ctx.buf, flat, None, ctx.n), None, None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, expert_out, flat, gate, buf, grad_buf):
        buf.data.copy_(expert_out)
        ctx.buf, ctx.grad_buf = buf, grad_buf
        ctx.save_for_backward(flat, gate, expert_out)
        return _gather(buf, flat, gate, flat.shape[0])

    @staticmethod
    def backward(ctx, dy):
        flat, gate, expert_out = ctx.saved_tensors
        dy = dy.contiguous()
        # d gate[t] = <dy[t], unscaled row of t>: fetch the rows once more
        ctx.buf.data.copy_(expert_out)
        rows = _gather(ctx.buf, flat, None, flat.shape[0])
        d_gate = (dy.float() * rows.float()).sum(-1)
        # d expert_out[slot of t] = gate[t] * dy[t], scattered to the expert's rank
        _scatter(ctx.grad_buf, dy, flat, gate)
        return ctx.grad_buf.data.clone(), None, d_gate, None, None


def dispatch(x: torch.Tensor, flat: torch.Tensor, buf: ExchangeBuffer, grad_buf: ExchangeBuffer) -> torch.Tensor:
    """x [T, d], flat [T] int32 (expert * capacity + slot, negative = dropped) -> [ranks, experts_per_rank, capacity, d]:
    the tokens that every rank sent to this rank's experts (zero rows where a slot stayed empty)."""
    return _Dispatch.apply(x, flat, buf, grad_buf)


def combine(expert_out: torch.Tensor, flat: torch.Tensor, gate: torch.Tensor, buf: ExchangeBuffer, grad_buf: ExchangeBuffer) -> torch.Tensor:
    """expert_out [ranks, experts_per_rank, capacity, d] (this rank's experts' results per source rank), gate [T] fp32 ->
    y [T, d] = gate[t] * the row token t was sent to; zero for dropped tokens."""
    return _Combine.apply(expert_out, flat, gate.float().contiguous(), buf, grad_buf)
