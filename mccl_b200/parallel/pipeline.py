"""Pipeline parallelism over the library's Send / Recv: rank s of the communicator holds stage s of the model, the
batch is cut into micro-batches, and activations travel forward and gradients backward between neighbours.

    stage = PipelineStage(comm, module, act_shape, dtype)          # act_shape: shape of one micro-batch between stages
    loss = stage.run(micro_inputs, micro_targets, loss_fn)         # one step's forward + backward; grads are in .grad

Schedule: one-forward-one-backward (1F1B).  Stage s first runs `stages - 1 - s` forward passes, then alternates one
forward with one backward, then drains the remaining backward passes, so at most `stages - s` micro-batches are
alive on a stage.  In the steady state a stage has to send an activation to its successor while the successor wants
to send a gradient back; both transfers are issued inside one group (mcclGroupStart / mcclGroupEnd) so that they
progress together whatever the transport's buffering.

The reference provides the two primitives (mcclSend / mcclRecv, src/p2p.cc:202-216, grouped at :279-321) and no
scheduler.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.nn as nn

from ..comm import Communicator, group


class PipelineStage:
    """This rank's stage of a pipeline-parallel model and the 1F1B schedule that drives it."""

    def __init__(self, comm: Communicator, module: nn.Module, act_shape: Sequence[int], dtype=torch.float32, device=None):
        self.comm, self.module = comm, module
        self.stage, self.stages = comm.rank, comm.size
        self.first, self.last = self.stage == 0, self.stage == comm.size - 1
        self.shape, self.dtype = tuple(act_shape), dtype
        self.device = device if device is not None else next(module.parameters()).device

    # ---- neighbour exchanges (tensors of the agreed shape)
    def _buf(self) -> torch.Tensor:
        return torch.empty(self.shape, dtype=self.dtype, device=self.device)

    def _recv_forward(self) -> Optional[torch.Tensor]:
        if self.first:
            return None
        t = self._buf()
        self.comm.recv(t.view(-1), self.stage - 1)
        return t.requires_grad_(True)

    def _send_forward(self, y: torch.Tensor) -> None:
        if not self.last:
            self.comm.send(y.detach().contiguous().view(-1), self.stage + 1)

    def _recv_backward(self) -> Optional[torch.Tensor]:
        if self.last:
            return None
        g = self._buf()
        self.comm.recv(g.view(-1), self.stage + 1)
        return g

    def _send_backward(self, gx: Optional[torch.Tensor]) -> None:
        if not self.first:
            self.comm.send(gx.contiguous().view(-1), self.stage - 1)

    def _send_forward_recv_backward(self, y: torch.Tensor) -> Optional[torch.Tensor]:
        if self.last:
            return None
        g = self._buf()
        with group():
            self.comm.send(y.detach().contiguous().view(-1), self.stage + 1)
            self.comm.recv(g.view(-1), self.stage + 1)
        return g

    def _send_backward_recv_forward(self, gx: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        if self.first:
            return None
        t = self._buf()
        with group():
            self.comm.send(gx.contiguous().view(-1), self.stage - 1)
            self.comm.recv(t.view(-1), self.stage - 1)
        return t.requires_grad_(True)

    # ---- one micro-batch
    def _forward(self, x_in: Optional[torch.Tensor], micro_input, target, loss_fn, n_micro: int):
        x = micro_input if self.first else x_in
        y = self.module(x)
        if self.last:
            y = loss_fn(y, target) / n_micro
        return x_in, y

    def _backward(self, x_in: Optional[torch.Tensor], y: torch.Tensor, grad_out: Optional[torch.Tensor]):
        if self.last:
            y.backward()
        else:
            y.backward(grad_out)
        return None if self.first else x_in.grad

    def run(self, micro_inputs: Optional[List], micro_targets: Optional[List], loss_fn: Optional[Callable], n_micro: int) -> Optional[torch.Tensor]:
        """One training step over `n_micro` micro-batches.  The first stage passes `micro_inputs`, the last stage
        `micro_targets` and `loss_fn` (mean over the micro-batch); the others pass None.  Parameter gradients are
        accumulated into `.grad`; the last stage returns the mean loss."""
        warm = min(self.stages - 1 - self.stage, n_micro)
        steady = n_micro - warm
        alive: List = []                        # (input from the previous stage, output) of forward passes in flight
        total = None
        get_in = lambda i: micro_inputs[i] if self.first else None
        get_t = lambda i: micro_targets[i] if self.last else None
        fwd = 0
        for _ in range(warm):
            x_in, y = self._forward(self._recv_forward(), get_in(fwd), get_t(fwd), loss_fn, n_micro)
            self._send_forward(y)
            alive.append((x_in, y)); fwd += 1
        x_next = self._recv_forward() if steady > 0 else None
        for i in range(steady):
            x_in, y = self._forward(x_next, get_in(fwd), get_t(fwd), loss_fn, n_micro)
            alive.append((x_in, y)); fwd += 1
            if self.last:
                total = y.detach() if total is None else total + y.detach()
            grad_out = self._send_forward_recv_backward(y)
            x0, y0 = alive.pop(0)
            gx = self._backward(x0, y0, grad_out)
            if i + 1 < steady:
                x_next = self._send_backward_recv_forward(gx)
            else:
                self._send_backward(gx)
        for _ in range(warm):                   # drain
            x0, y0 = alive.pop(0)
            gx = self._backward(x0, y0, self._recv_backward())
            self._send_backward(gx)
        return total
