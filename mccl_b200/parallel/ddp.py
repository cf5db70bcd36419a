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

With `shard_optimizer=True` (ZeRO stage 1) a bucket's gradients are reduce-scattered instead of all-reduced, each
rank keeps the fp32 master weights and Adam moments of its 1/world slice only and updates that slice, and the new
bf16 parameters are all-gathered in place: the same bytes cross NVLink as for an all-reduce, the optimizer kernels
shrink by the world size, and so does the optimizer state.

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
    def __init__(self, params: List[nn.Parameter], weight_decay: float, align: int = 8):
        self.params = params
        self.weight_decay = weight_decay
        self.numel = 0
        self.offsets = []
        for p in params:
            self.offsets.append(self.numel)
            self.numel += (p.numel() + 7) // 8 * 8          # keep every view 16-byte aligned
        self.numel = (self.numel + align - 1) // align * align   # sharded: equal 16-byte aligned slices
        self.gather_event: Optional[torch.cuda.Event] = None
        self.grad: Optional[torch.Tensor] = None
        self.param: Optional[torch.Tensor] = None
        self.master = self.exp_avg = self.exp_avg_sq = None
        self.pending = 0
        self.ready_event: Optional[torch.cuda.Event] = None
        self.done_event: Optional[torch.cuda.Event] = None
        self.launched = False


class DistributedDataParallel(nn.Module):
    """Wraps a module for data-parallel training over `comm`: gradients live in bucket buffers that are averaged over the
    ranks while backward runs; `step()` applies the fused (optionally sharded, optionally norm-clipped) AdamW update."""

    def __init__(self, module: nn.Module, comm: Optional[Communicator] = None, bucket_mb: Optional[float] = None,
                 overlap: bool = True, comm_ctas: Optional[int] = None, weight_decay: float = 0.1, betas=(0.9, 0.95),
                 eps: float = 1e-8, shard_optimizer: bool = False, sync_params: bool = True):
        super().__init__()
        self.module = module
        self.comm = comm
        self.world = comm.size if comm is not None else 1
        self.rank = comm.rank if comm is not None else 0
        self.sharded = bool(shard_optimizer) and self.world > 1
        self.overlap = overlap
        # CTAs a bucket's all-reduce may take while backward is still running (the rest stay with the GEMMs)
        self.comm_ctas = int(os.environ.get("MCCL_DDP_CTAS", "16")) if comm_ctas is None else int(comm_ctas)
        self._launched_count = 0
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
        align = 8 * self.world if self.sharded else 8
        self.buckets: List[_Bucket] = []
        for decay in (True, False):
            cur: List[nn.Parameter] = []
            size = 0
            for p in reversed(params):
                if (p.dim() >= 2) != decay:
                    continue
                if cur and size + p.numel() > cap:
                    self.buckets.append(_Bucket(cur, weight_decay if decay else 0.0, align))
                    cur, size = [], 0
                cur.append(p)
                size += p.numel()
            if cur:
                self.buckets.append(_Bucket(cur, weight_decay if decay else 0.0, align))
        self._bucket_of = {}
        if self.world > 1 and sync_params:
            self._sync_initial_state(module)
        # All communication buffers come from ONE symmetric allocation (one handle exchange, one multicast binding)
        # instead of one collective allocation per bucket.
        self._pool = None
        if self.world > 1 and self.device.type == "cuda":
            es = params[0].element_size()
            per = sum((b.numel * es + 255) // 256 * 256 for b in self.buckets)
            self._pool = comm.pool(per * (2 if self.sharded else 1) + 4096)
        for b in self.buckets:
            self._materialize(b)
            for p in b.params:
                self._bucket_of[p] = b
        if self.world > 1:
            if self.comm_ctas:
                comm.set_max_ctas(self.comm_ctas)      # leave the SMs to the backward GEMMs
            self.comm_stream = torch.cuda.Stream(device=self.device, priority=-1) if self.device.type == "cuda" else None
            for p in params:
                p.register_post_accumulate_grad_hook(self._on_grad)
        self._reset()

    # ---- construction helpers
    def _sync_initial_state(self, module: nn.Module) -> None:
        """Every replica starts from rank 0's parameters and buffers, whatever each rank was seeded with (only
        gradients are averaged afterwards, so replicas that start apart stay apart)."""
        with torch.no_grad():
            for t in list(module.parameters()) + list(module.buffers()):
                if t.numel() == 0:
                    continue
                flat = t.data.contiguous().view(-1)
                self.comm.broadcast(flat, flat, root=0)
                if flat.data_ptr() != t.data.data_ptr():
                    t.data.copy_(flat.view(t.shape))
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    def _materialize(self, b: _Bucket) -> None:
        dev, dt = self.device, self.dtype
        if self._pool is not None:
            b.grad = self._pool.empty(b.numel, dt)          # local bookkeeping: same order on every rank
            b.grad.zero_()
        else:
            b.grad = torch.zeros(b.numel, device=dev, dtype=dt)
        if self.sharded and self._pool is not None:
            b.param = self._pool.empty(b.numel, dt)         # all-gathered in place after the optimizer step
            b.param.zero_()
        else:
            b.param = torch.zeros(b.numel, device=dev, dtype=dt)
        for p, off in zip(b.params, b.offsets):
            n = p.numel()
            b.param[off:off + n].copy_(p.data.reshape(-1))
            p.data = b.param[off:off + n].view(p.shape)
            p.grad = b.grad[off:off + n].view(p.shape)
        # fp32 master weights and moments: the whole bucket, or this rank's slice of it when sharded
        b.lo, b.hi = 0, b.numel
        if self.sharded:
            shard = b.numel // self.world
            b.lo, b.hi = self.rank * shard, (self.rank + 1) * shard
        b.master = b.param[b.lo:b.hi].float()
        b.exp_avg = torch.zeros_like(b.master)
        b.exp_avg_sq = torch.zeros_like(b.master)

    def _reset(self) -> None:
        for b in self.buckets:
            b.pending = len(b.params)
            b.launched = False
        self._launched_count = 0

    # ---- backward-time communication
    def _launch(self, b: _Bucket) -> None:
        b.launched = True
        self._launched_count += 1
        if self.world == 1 or not self._sync:
            return
        if self.overlap and self.comm_stream is not None:
            b.ready_event = torch.cuda.Event()
            b.ready_event.record()
            self.comm_stream.wait_event(b.ready_event)
            # The bucket that closes last has nothing left to overlap with (backward is over when its last
            # gradient arrives): it gets the whole GPU, the others stay within comm_ctas.
            tail = self.comm_ctas and self._launched_count == len(self.buckets)
            if tail:
                self.comm.set_max_ctas(0)
            self._reduce(b, self.comm_stream)
            if tail:
                self.comm.set_max_ctas(self.comm_ctas)
            b.done_event = torch.cuda.Event()
            b.done_event.record(self.comm_stream)
        else:
            self._reduce(b, None)
            b.done_event = None

    def _reduce(self, b: _Bucket, stream) -> None:
        if not self.sharded:
            self.comm.all_reduce(b.grad, op="avg", stream=stream)
        elif self.device.type == "cuda":
            # in place: rank r reduces block r of every rank's bucket into block r of its own
            self.comm.reduce_scatter(b.grad, b.grad[b.lo:b.hi], op="avg", stream=stream)
        else:
            out = torch.empty(b.hi - b.lo, dtype=b.grad.dtype)
            self.comm.reduce_scatter(b.grad, out, op="avg")
            b.grad[b.lo:b.hi].copy_(out)

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

    def step(self, lr: float = 3e-4, max_grad_norm: Optional[float] = None, _hyper: Optional[torch.Tensor] = None) -> None:
        """Wait for the gradient buckets, then one fused AdamW kernel per bucket (it also clears the gradients).
        With `max_grad_norm` the global gradient norm is accumulated bucket by bucket on the device and the
        optimizer kernels clip by it without a host round trip."""
        self.step_count += 1
        norm_sq = None
        cuda = self.device.type == "cuda"
        if max_grad_norm is not None and cuda:
            if self._norm_sq is None:
                # four floats: a 16-byte message takes the one-shot all-reduce when the norm is summed over ranks
                self._norm_sq = (self._pool.empty(4, torch.float32) if self.sharded else
                                 torch.zeros(4, device=self.device, dtype=torch.float32))
                self._norm_sq.zero_()
                self._norm_scratch = torch.zeros(scratch_floats(max(b.hi - b.lo for b in self.buckets)), device=self.device,
                                                 dtype=torch.float32)
            norm_sq = self._norm_sq[:1]
            cur0 = torch.cuda.current_stream(self.device)
            for i, b in enumerate(self.buckets):
                if not b.launched:
                    self._launch(b)
                if b.done_event is not None:
                    cur0.wait_event(b.done_event)
                sum_squares_(b.grad[b.lo:b.hi], norm_sq, self._norm_scratch, accumulate=i > 0)
            if self.sharded:
                self.comm.all_reduce(self._norm_sq, op="sum")      # every rank summed its slices only
        for b in self.buckets:
            if not b.launched:
                self._launch(b)
        cur = torch.cuda.current_stream(self.device) if cuda else None
        side = self.comm_stream if (self.sharded and self.overlap and cuda) else None
        for b in self.buckets:
            if b.done_event is not None and cur is not None:
                cur.wait_event(b.done_event)
            p_slice, g_slice = b.param[b.lo:b.hi], b.grad[b.lo:b.hi]
            if cuda:
                fused_adamw_(p_slice, b.master, b.exp_avg, b.exp_avg_sq, g_slice, lr=lr, betas=self.betas, eps=self.eps,
                             weight_decay=b.weight_decay, step=self.step_count, zero_grad=not self.sharded, norm_sq=norm_sq,
                             max_norm=max_grad_norm or 0.0, hyper=_hyper)
                if self.sharded:
                    b.grad.zero_()                     # the other ranks' slices hold this rank's raw gradients
            else:  # CPU stand-in for tests of the bucket logic
                from ..ops.optim import adamw_reference
                new = adamw_reference(b.master, b.exp_avg, b.exp_avg_sq, g_slice, lr=lr, betas=self.betas, eps=self.eps,
                                      weight_decay=b.weight_decay, grad_scale=1.0, step=self.step_count)
                p_slice.copy_(new.to(b.param.dtype))
                b.grad.zero_()
            if self.sharded:
                # every rank's new slice into every rank's copy of the bucket, in place; on the side stream it
                # runs under the next bucket's optimizer kernel
                if side is not None:
                    ev = torch.cuda.Event()
                    ev.record()
                    side.wait_event(ev)
                    self.comm.all_gather(p_slice, b.param, stream=side)
                    b.gather_event = torch.cuda.Event()
                    b.gather_event.record(side)
                else:
                    self.comm.all_gather(p_slice, b.param)
            b.done_event = None
        if side is not None:
            for b in self.buckets:
                if b.gather_event is not None:
                    cur.wait_event(b.gather_event)
                    b.gather_event = None
        self._reset()

    def graphed_step(self, example_args, lr: float = 3e-4, max_grad_norm: Optional[float] = None, warmup: int = 1):
        """Record one whole training step (forward, backward with the bucket all-reduces on their side stream, gradient
        norm, optimizer) in a CUDA graph and return a callable that replays it:

            step = ddp.graphed_step((idx, targets), lr=3e-4, max_grad_norm=1.0)
            loss = step(idx, targets)            # a device tensor, overwritten by the next call

        `example_args` are the positional tensors of the module's forward (it must return the loss); later calls pass
        tensors of the same shapes and dtypes, which are copied into the graph's input buffers.  A replay costs the
        host one launch, so a step that is bound by the host issuing a few thousand small kernels becomes bound by the
        GPU.  The learning rate and Adam's bias corrections live in device memory and are refreshed before every replay
        (`step(..., lr=...)` changes the rate).  `warmup` eager steps on the example batch run first (they are ordinary
        training steps).  Every rank must record and replay in step with the others.  No autograd graph of an earlier
        step may still be alive when this is called (drop the last loss tensor): its gradient accumulators would run on
        the stream of that earlier step, which a recording cannot wait for."""
        return _GraphedStep(self, example_args, lr, max_grad_norm, warmup)

    # ---- checkpointing
    def optimizer_state_dict(self) -> dict:
        """The optimizer's state as host tensors: the step count and, per bucket, the fp32 master weights and the two
        Adam moments (this rank's slice of them when the optimizer is sharded).  Together with the module's own
        state_dict it resumes training exactly."""
        return {"step": self.step_count, "world": self.world, "sharded": self.sharded,
                "buckets": [{"numel": b.numel, "lo": b.lo, "hi": b.hi, "master": b.master.detach().cpu().clone(),
                             "exp_avg": b.exp_avg.detach().cpu().clone(), "exp_avg_sq": b.exp_avg_sq.detach().cpu().clone()}
                            for b in self.buckets]}

    def load_optimizer_state_dict(self, state: dict) -> None:
        """Restore what optimizer_state_dict returned (same model, bucket size, world size and sharding).  The bf16
        parameters are rewritten from the master weights, so the module needs no separate load."""
        if len(state["buckets"]) != len(self.buckets) or state["sharded"] != self.sharded or \
                (self.sharded and state["world"] != self.world):
            raise ValueError("the checkpoint was written with a different bucket layout, world size or sharding")
        self.step_count = int(state["step"])
        for b, sb in zip(self.buckets, state["buckets"]):
            if (sb["numel"], sb["lo"], sb["hi"]) != (b.numel, b.lo, b.hi):
                raise ValueError("bucket layout mismatch")
            b.master.copy_(sb["master"]); b.exp_avg.copy_(sb["exp_avg"]); b.exp_avg_sq.copy_(sb["exp_avg_sq"])
            b.param[b.lo:b.hi].copy_(b.master.to(b.param.dtype))
            if self.sharded:
                self.comm.all_gather(b.param[b.lo:b.hi], b.param)
        self._reset()

    def bucket_sizes_mb(self) -> List[float]:
        """Size of every gradient bucket in MB, in launch order."""
        return [b.numel * b.grad.element_size() / (1 << 20) for b in self.buckets]


class _GraphedStep:
    """See DistributedDataParallel.graphed_step."""

    def __init__(self, ddp: DistributedDataParallel, example_args, lr: float, max_grad_norm: Optional[float], warmup: int):
        if ddp.device.type != "cuda":
            raise RuntimeError("graphed_step needs a CUDA device")
        self.ddp, self.lr, self.max_grad_norm = ddp, lr, max_grad_norm
        if ddp.step_count == 0 and warmup < 1:
            warmup = 1                            # the first step allocates work buffers, which a recording cannot do
        self.inputs = [a.to(ddp.device).contiguous().clone() for a in example_args]
        self.hyper = torch.zeros(4, device=ddp.device, dtype=torch.float32)
        self.hyper_host = torch.zeros(4, dtype=torch.float32).pin_memory()
        cur = torch.cuda.current_stream(ddp.device)
        side = torch.cuda.Stream(device=ddp.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            for _ in range(max(0, warmup)):
                self._refresh(lr)
                loss = ddp(*self.inputs)
                loss.backward()
                ddp.step(lr=lr, max_grad_norm=max_grad_norm, _hyper=self.hyper)
        cur.wait_stream(side)
        torch.cuda.synchronize(ddp.device)
        from ..ops import loss as loss_ops
        from ..ops import norm as norm_ops
        from ..ops import optim
        count = lambda: ((ddp.comm.launch_count if ddp.comm is not None else 0) + optim.launches() + loss_ops.launches() +
                         norm_ops.launches())
        before, steps_before = count(), ddp.step_count
        self.graph = torch.cuda.CUDAGraph()
        try:
            with torch.cuda.graph(self.graph):
                self.loss = ddp(*self.inputs)
                self.loss.backward()
                ddp.step(lr=lr, max_grad_norm=max_grad_norm, _hyper=self.hyper)
        except RuntimeError as exc:
            raise RuntimeError("recording the step in a CUDA graph failed; if an earlier step's loss (and with it its autograd "
                               "graph) is still referenced, drop it before calling graphed_step") from exc
        ddp.step_count = steps_before            # recording ran no step
        self.launches_per_step = count() - before

    def _refresh(self, lr: float) -> None:
        d = self.ddp
        t = d.step_count + 1                     # the step about to run
        self.hyper_host[0] = lr
        self.hyper_host[1] = 1.0 - d.betas[0] ** t
        self.hyper_host[2] = (1.0 - d.betas[1] ** t) ** 0.5
        self.hyper.copy_(self.hyper_host, non_blocking=True)

    def __call__(self, *args, lr: Optional[float] = None) -> torch.Tensor:
        for dst, src in zip(self.inputs, args):
            dst.copy_(src, non_blocking=True)
        self._refresh(self.lr if lr is None else lr)
        self.graph.replay()
        self.ddp.step_count += 1
        return self.loss
