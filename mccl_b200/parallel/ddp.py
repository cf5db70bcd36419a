"""Data parallelism: gradient buckets in symmetric memory, all-reduced (fused 1/world average) by the
library's own kernels on a side stream while backward is still running, followed by a fused optimizer step
per bucket.

    ddp = DistributedDataParallel(model, comm, bucket_mb=25)
    loss = ddp(idx, targets); loss.backward(); ddp.step(lr=...)

Layout: parameters are walked in reverse registration order (roughly the order backward produces their
gradients) and packed into buckets of `bucket_mb`.  A bucket owns one flat bf16 gradient buffer allocated
with mcclMemAlloc (peer-mapped, multicast-bound: the all-reduce runs on it in place with no staging copy),
one flat bf16 parameter buffer the module's parameters are re-pointed into, and flat fp32 master / moment
buffers for the optimizer.  `param.grad` is a view of the gradient bucket, so autograd accumulates straight
into communication memory.

The reference publishes this workload only as a benchmark shape ("compute on batch + gradient all-reduce",
docs/perf-scaling.png, README.md:55-57); the wrapper itself has no counterpart there.
"""
from __future__ import annotations

import os
from contextlib import contextmanager
from typing import List, Optional

import torch
import torch.nn as nn

from ..comm import Communicator
from ..ops.optim import fused_adamw_, scratch_floats, sum_squares_


class _Bucket:
    def __init__(self, params: List[nn.Parameter], weight_decay: float):
        self.params = params
        self.weight_decay = weight_decay
        self.numel = 0
        self.offsets = []
        for p in params:
            self.offsets.append(self.numel)
            self.numel += (p.numel() + 7) // 8 * 8          # keep every view 16-byte aligned
        self.grad: Optional[torch.Tensor] = None
        self.param: Optional[torch.Tensor] = None
        self.master = self.exp_avg = self.exp_avg_sq = None
        self.pending = 0
        self.ready_event: Optional[torch.cuda.Event] = None
        self.done_event: Optional[torch.cuda.Event] = None
        self.launched = False


class DistributedDataParallel(nn.Module):
    def __init__(self, module: nn.Module, comm: Optional[Communicator] = None, bucket_mb: Optional[float] = None,
                 overlap: bool = True, comm_ctas: int = 16, weight_decay: float = 0.1, betas=(0.9, 0.95), eps: float = 1e-8):
        super().__init__()
        self.module = module
        self.comm = comm
        self.world = comm.size if comm is not None else 1
        self.overlap = overlap
        self.betas, self.eps = betas, eps
        self.step_count = 0
        self._norm_sq = None
        self._norm_scratch = None
        self._sync = True
        params = [p for p in module.parameters() if p.requires_grad]
        if not params:
            raise ValueError("module has no trainable parameters")
        self.device = params[0].device
        self.dtype = params[0].dtype
        if self.device.type == "cuda" and self.dtype != torch.bfloat16:
            raise ValueError("the fused optimizer path expects bf16 parameters")
        if bucket_mb is None:
            bucket_mb = float(os.environ.get("MCCL_BUCKET_MB", "25"))
        cap = int(bucket_mb * (1 << 20)) // params[0].element_size()
        # Matrices decay, vectors (biases, norms) do not: they live in separate buckets so a bucket has one setting.
        self.buckets: List[_Bucket] = []
        for decay in (True, False):
            cur: List[nn.Parameter] = []
            size = 0
            for p in reversed(params):
                if (p.dim() >= 2) != decay:
                    continue
                if cur and size + p.numel() > cap:
                    self.buckets.append(_Bucket(cur, weight_decay if decay else 0.0))
                    cur, size = [], 0
                cur.append(p)
                size += p.numel()
            if cur:
                self.buckets.append(_Bucket(cur, weight_decay if decay else 0.0))
        self._bucket_of = {}
        for b in self.buckets:
            self._materialize(b)
            for p in b.params:
                self._bucket_of[p] = b
        if self.world > 1:
            if comm_ctas:
                comm.set_max_ctas(comm_ctas)      # leave the SMs to the backward GEMMs
            self.comm_stream = torch.cuda.Stream(device=self.device, priority=-1) if self.device.type == "cuda" else None
            for p in params:
                p.register_post_accumulate_grad_hook(self._on_grad)
        self._reset()

    # ---- construction helpers
    def _materialize(self, b: _Bucket) -> None:
        dev, dt = self.device, self.dtype
        if self.world > 1 and dev.type == "cuda":
            b.grad = self.comm.empty(b.numel, dt)           # collective: same order on every rank
            b.grad.zero_()
        else:
            b.grad = torch.zeros(b.numel, device=dev, dtype=dt)
        b.param = torch.zeros(b.numel, device=dev, dtype=dt)
        b.master = torch.zeros(b.numel, device=dev, dtype=torch.float32)
        b.exp_avg = torch.zeros_like(b.master)
        b.exp_avg_sq = torch.zeros_like(b.master)
        for p, off in zip(b.params, b.offsets):
            n = p.numel()
            b.param[off:off + n].copy_(p.data.reshape(-1))
            b.master[off:off + n].copy_(p.data.reshape(-1).float())
            p.data = b.param[off:off + n].view(p.shape)
            p.grad = b.grad[off:off + n].view(p.shape)

    def _reset(self) -> None:
        for b in self.buckets:
            b.pending = len(b.params)
            b.launched = False

    # ---- backward-time communication
    def _launch(self, b: _Bucket) -> None:
        b.launched = True
        if self.world == 1 or not self._sync:
            return
        if self.overlap and self.comm_stream is not None:
            b.ready_event = torch.cuda.Event()
            b.ready_event.record()
            self.comm_stream.wait_event(b.ready_event)
            self.comm.all_reduce(b.grad, op="avg", stream=self.comm_stream)
            b.done_event = torch.cuda.Event()
            b.done_event.record(self.comm_stream)
        else:
            self.comm.all_reduce(b.grad, op="avg")
            b.done_event = None

    def _on_grad(self, p: nn.Parameter) -> None:
        b = self._bucket_of[p]
        b.pending -= 1
        if b.pending == 0 and not b.launched:
            self._launch(b)

    def forward(self, *args, **kwargs):
        if torch.is_grad_enabled():
            self._reset()                 # a new backward pass will count every parameter's gradient again
        return self.module(*args, **kwargs)

    @contextmanager
    def no_sync(self):
        """Gradient accumulation: backward passes inside this context add into the buckets without
        communicating; the first backward pass outside it all-reduces the accumulated gradients."""
        prev, self._sync = self._sync, False
        try:
            yield
        finally:
            self._sync = prev

    def finish_backward(self) -> None:
        """Launch whatever has not gone out yet (unused parameters) and make the current stream wait for all buckets."""
        for b in self.buckets:
            if not b.launched:
                self._launch(b)
        cur = torch.cuda.current_stream(self.device) if self.device.type == "cuda" else None
        for b in self.buckets:
            if b.done_event is not None and cur is not None:
                cur.wait_event(b.done_event)

    def step(self, lr: float = 3e-4, max_grad_norm: Optional[float] = None) -> None:
        """Wait for the gradient buckets, then one fused AdamW kernel per bucket (it also clears the gradients).
        With `max_grad_norm` the global gradient norm is accumulated bucket by bucket on the device and the
        optimizer kernels clip by it without a host round trip."""
        self.step_count += 1
        norm_sq = None
        if max_grad_norm is not None and self.device.type == "cuda":
            if self._norm_sq is None:
                self._norm_sq = torch.zeros(1, device=self.device, dtype=torch.float32)
                self._norm_scratch = torch.zeros(scratch_floats(max(b.numel for b in self.buckets)), device=self.device,
                                                 dtype=torch.float32)
            norm_sq = self._norm_sq
            cur0 = torch.cuda.current_stream(self.device)
            for i, b in enumerate(self.buckets):
                if not b.launched:
                    self._launch(b)
                if b.done_event is not None:
                    cur0.wait_event(b.done_event)
                sum_squares_(b.grad, norm_sq, self._norm_scratch, accumulate=i > 0)
        for b in self.buckets:
            if not b.launched:
                self._launch(b)
        cur = torch.cuda.current_stream(self.device) if self.device.type == "cuda" else None
        for b in self.buckets:
            if b.done_event is not None and cur is not None:
                cur.wait_event(b.done_event)
            if self.device.type == "cuda":
                fused_adamw_(b.param, b.master, b.exp_avg, b.exp_avg_sq, b.grad, lr=lr, betas=self.betas, eps=self.eps,
                             weight_decay=b.weight_decay, step=self.step_count, zero_grad=True, norm_sq=norm_sq,
                             max_norm=max_grad_norm or 0.0)
            else:  # CPU stand-in for tests of the bucket logic
                from ..ops.optim import adamw_reference
                new = adamw_reference(b.master, b.exp_avg, b.exp_avg_sq, b.grad, lr=lr, betas=self.betas, eps=self.eps,
                                      weight_decay=b.weight_decay, grad_scale=1.0, step=self.step_count)
                b.param.copy_(new.to(b.param.dtype))
                b.grad.zero_()
            b.done_event = None
        self._reset()

    def bucket_sizes_mb(self) -> List[float]:
        return [b.numel * b.grad.element_size() / (1 << 20) for b in self.buckets]
