"""`torch.distributed` backend "mccl": the library's collectives behind the c10d interface, so that code written
for `backend="nccl"` (torch DDP, FSDP's flat all-gather / reduce-scatter, plain `dist.all_reduce` calls) runs on
this library by changing one string.

    import mccl_b200.c10d                      # registers the backend
    dist.init_process_group("mccl", rank=r, world_size=n, init_method="tcp://127.0.0.1:29500")
    dist.all_reduce(t)                         # cuda tensors -> the sm_100a kernels, cpu tensors -> the tcp transport

One communicator per device type is created on first use (the unique id travels through the c10d store).  CUDA
collectives are enqueued on a side stream that first waits for the caller's current stream; `Work.wait()` makes the
caller's stream wait for the collective, and the future returned by `get_future()` carries the same dependency,
which is what torch DDP's bucket hooks need to overlap communication with backward.  The reference has no
PyTorch binding; its C API (src/include/mccl.h:5-15) is what `mccl_b200.comm.Communicator` wraps underneath.
"""
from __future__ import annotations

import threading
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
from torch._C._distributed_c10d import Work as _WorkBase

from .comm import Communicator, get_unique_id

_OPS = {dist.ReduceOp.SUM: "sum", dist.ReduceOp.AVG: "avg", dist.ReduceOp.PRODUCT: "prod", dist.ReduceOp.MIN: "min",
        dist.ReduceOp.MAX: "max"}


def _op_name(op) -> str:
    op = getattr(op, "op", op) if not isinstance(op, dist.ReduceOp.RedOpType) else op
    for k, v in _OPS.items():
        if op == k:
            return v
    raise ValueError(f"the mccl backend supports sum, avg, product, min and max (got {op})")


class _Work(_WorkBase):
    """Completed on the host at once; on CUDA the device-side dependency is an event on the communication stream."""

    def __init__(self, result, device: torch.device, stream: Optional[torch.cuda.Stream]):
        super().__init__()
        self._result = result
        self._device = device
        self._stream = stream
        self._event = None
        if stream is not None:
            self._event = torch.cuda.Event()
            self._event.record(stream)
            self._future = torch.futures.Future(devices=[device])
            with torch.cuda.stream(stream):
                self._future.set_result(result)
        else:
            self._future = torch.futures.Future()
            self._future.set_result(result)

    def wait(self, timeout=None) -> bool:
        if self._event is not None:
            torch.cuda.current_stream(self._device).wait_event(self._event)
        return True

    def synchronize(self) -> None:
        self.wait()

    def is_completed(self) -> bool:
        return self._event is None or self._event.query()

    def is_success(self) -> bool:
        return True

    def get_future(self):
        return self._future

    def result(self):
        return self._result


class MCCLBackend(dist.ProcessGroup):
    """The c10d process group: every method maps one torch.distributed call onto the library's collective of the same
    name and returns a work object whose wait() / future carry the stream dependency."""

    def __init__(self, store, rank: int, size: int, timeout=None):
        super().__init__(rank, size)
        self._store = store
        self._rank, self._size = rank, size
        self._comms: Dict[str, Communicator] = {}
        self._streams: Dict[int, torch.cuda.Stream] = {}
        self._lock = threading.Lock()
        self._generation = 0

    # ---- plumbing
    def _comm(self, device: torch.device) -> Communicator:
        kind = device.type
        with self._lock:
            comm = self._comms.get(kind)
            if comm is None:
                key = f"mccl_uid_{kind}"            # the store is already prefixed per process group
                if self._rank == 0:
                    uid = get_unique_id()
                    self._store.set(key, uid)
                else:
                    uid = bytes(self._store.get(key))
                if kind == "cuda":
                    torch.cuda.set_device(device)
                comm = Communicator(self._size, uid, self._rank, transport="cuda" if kind == "cuda" else "tcp")
                self._comms[kind] = comm
            return comm

    def _enter(self, t: torch.Tensor):
        """Communicator and stream for a tensor; on CUDA the side stream first waits for the caller's work."""
        comm = self._comm(t.device)
        if t.device.type != "cuda":
            return comm, None
        idx = t.device.index if t.device.index is not None else torch.cuda.current_device()
        s = self._streams.get(idx)
        if s is None:
            s = self._streams[idx] = torch.cuda.Stream(device=t.device, priority=-1)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(t.device))
        s.wait_event(ev)
        return comm, s

    @staticmethod
    def _flat(t: torch.Tensor) -> torch.Tensor:
        if not t.is_contiguous():
            raise ValueError("the mccl backend needs contiguous tensors")
        return t.view(-1)

    def _done(self, result, t: torch.Tensor, stream) -> _Work:
        if stream is not None:
            for x in (result if isinstance(result, (list, tuple)) else [result]):
                for y in (x if isinstance(x, (list, tuple)) else [x]):
                    if isinstance(y, torch.Tensor):
                        y.record_stream(stream)
        return _Work(result, t.device, stream)

    # ---- collectives
    def allreduce(self, tensors: List[torch.Tensor], opts=None) -> _Work:
        op = _op_name(opts.reduceOp) if opts is not None else "sum"
        for t in tensors:
            comm, s = self._enter(t)
            comm.all_reduce(self._flat(t), op=op, stream=s)
        return self._done(tensors, tensors[0], s)

    def allreduce_coalesced(self, tensors, opts=None) -> _Work:
        return self.allreduce(tensors, opts)

    def broadcast(self, tensors: List[torch.Tensor], opts=None) -> _Work:
        root = opts.rootRank if opts is not None else 0
        for t in tensors:
            comm, s = self._enter(t)
            f = self._flat(t)
            comm.broadcast(f if self._rank == root else None, f, root=root, stream=s)
        return self._done(tensors, tensors[0], s)

    def reduce(self, tensors: List[torch.Tensor], opts=None) -> _Work:
        root = opts.rootRank if opts is not None else 0
        op = _op_name(opts.reduceOp) if opts is not None else "sum"
        for t in tensors:
            comm, s = self._enter(t)
            f = self._flat(t)
            if self._rank == root:
                comm.reduce(f, f, op=op, root=root, stream=s)
            else:                       # c10d leaves a non-root tensor untouched
                comm.reduce(f, None, op=op, root=root, stream=s)
        return self._done(tensors, tensors[0], s)

    def _allgather_base(self, out: torch.Tensor, inp: torch.Tensor, opts=None) -> _Work:
        comm, s = self._enter(inp)
        comm.all_gather(self._flat(inp), self._flat(out), stream=s)
        return self._done(out, out, s)

    def allgather(self, outputs: List[List[torch.Tensor]], inputs: List[torch.Tensor], opts=None) -> _Work:
        for outs, inp in zip(outputs, inputs):
            comm, s = self._enter(inp)
            flat = torch.empty(inp.numel() * self._size, dtype=inp.dtype, device=inp.device)
            ctx = torch.cuda.stream(s) if s is not None else _NullCtx()
            with ctx:
                comm.all_gather(self._flat(inp.contiguous()), flat, stream=s)
                for r, o in enumerate(outs):
                    o.copy_(flat[r * inp.numel():(r + 1) * inp.numel()].view_as(o))
            if s is not None:
                flat.record_stream(s)
        return self._done(outputs, inputs[0], s)

    def allgather_into_tensor_coalesced(self, outputs, inputs, opts=None) -> _Work:
        for o, i in zip(outputs, inputs):
            w = self._allgather_base(o, i, opts)
        return w

    def _reduce_scatter_base(self, out: torch.Tensor, inp: torch.Tensor, opts=None) -> _Work:
        op = _op_name(opts.reduceOp) if opts is not None else "sum"
        comm, s = self._enter(inp)
        comm.reduce_scatter(self._flat(inp), self._flat(out), op=op, stream=s)
        return self._done(out, out, s)

    def reduce_scatter(self, outputs: List[torch.Tensor], inputs: List[List[torch.Tensor]], opts=None) -> _Work:
        op = _op_name(opts.reduceOp) if opts is not None else "sum"
        for out, ins in zip(outputs, inputs):
            comm, s = self._enter(out)
            ctx = torch.cuda.stream(s) if s is not None else _NullCtx()
            with ctx:
                flat = torch.cat([self._flat(i.contiguous()) for i in ins])
                comm.reduce_scatter(flat, self._flat(out), op=op, stream=s)
            if s is not None:
                flat.record_stream(s)
        return self._done(outputs, outputs[0], s)

    def alltoall_base(self, out: torch.Tensor, inp: torch.Tensor, out_splits, in_splits, opts=None) -> _Work:
        comm, s = self._enter(inp)
        if out_splits or in_splits:
            # split sizes count rows of dim 0
            row_in = inp.numel() // max(inp.shape[0], 1) if inp.dim() else 1
            row_out = out.numel() // max(out.shape[0], 1) if out.dim() else 1
            n = self._size
            ins = list(in_splits) if in_splits else [inp.shape[0] // n] * n
            outs = list(out_splits) if out_splits else [out.shape[0] // n] * n
            comm.all_to_all_v(self._flat(inp), [c * row_in for c in ins], self._flat(out), [c * row_out for c in outs], stream=s)
        else:
            comm.all_to_all(self._flat(inp), self._flat(out), stream=s)
        return self._done(out, out, s)

    def alltoall(self, outputs: List[torch.Tensor], inputs: List[torch.Tensor], opts=None) -> _Work:
        n = inputs[0].numel()
        if any(t.numel() != n for t in list(inputs) + list(outputs)):
            raise NotImplementedError("the mccl backend exchanges equal blocks")
        comm, s = self._enter(inputs[0])
        ctx = torch.cuda.stream(s) if s is not None else _NullCtx()
        with ctx:
            flat_in = torch.cat([self._flat(i.contiguous()) for i in inputs])
            flat_out = torch.empty_like(flat_in)
            comm.all_to_all(flat_in, flat_out, stream=s)
            for r, o in enumerate(outputs):
                o.copy_(flat_out[r * n:(r + 1) * n].view_as(o))
        if s is not None:
            flat_in.record_stream(s); flat_out.record_stream(s)
        return self._done(outputs, inputs[0], s)

    def gather(self, outputs: List[List[torch.Tensor]], inputs: List[torch.Tensor], opts=None) -> _Work:
        root = opts.rootRank if opts is not None else 0
        inp = inputs[0]
        comm, s = self._enter(inp)
        if self._rank == root:
            bufs = [torch.empty_like(inp) for _ in range(self._size)]
            from .comm import group
            with group():
                for p in range(self._size):
                    if p != root:
                        comm.recv(self._flat(bufs[p]), p, stream=s)
            ctx = torch.cuda.stream(s) if s is not None else _NullCtx()
            with ctx:
                for p, o in enumerate(outputs[0]):
                    o.copy_(inp if p == root else bufs[p])
            if s is not None:
                for b in bufs:
                    b.record_stream(s)
        else:
            comm.send(self._flat(inp.contiguous()), root, stream=s)
        return self._done(outputs, inp, s)

    def scatter(self, outputs: List[torch.Tensor], inputs: List[List[torch.Tensor]], opts=None) -> _Work:
        root = opts.rootRank if opts is not None else 0
        out = outputs[0]
        comm, s = self._enter(out)
        if self._rank == root:
            from .comm import group
            srcs = [t.contiguous() for t in inputs[0]]
            with group():
                for p in range(self._size):
                    if p != root:
                        comm.send(self._flat(srcs[p]), p, stream=s)
            ctx = torch.cuda.stream(s) if s is not None else _NullCtx()
            with ctx:
                out.copy_(srcs[root])
            if s is not None:
                for t in srcs:
                    t.record_stream(s)
        else:
            comm.recv(self._flat(out), root, stream=s)
        return self._done(outputs, out, s)

    def reduce_scatter_tensor_coalesced(self, outputs, inputs, opts=None) -> _Work:
        for o, i in zip(outputs, inputs):
            w = self._reduce_scatter_base(o, i, opts)
        return w

    def send(self, tensors: List[torch.Tensor], dst: int, tag: int = 0) -> _Work:
        for t in tensors:
            comm, s = self._enter(t)
            comm.send(self._flat(t), dst, stream=s)
        return self._done(tensors, tensors[0], s)

    def recv(self, tensors: List[torch.Tensor], src: int, tag: int = 0) -> _Work:
        for t in tensors:
            comm, s = self._enter(t)
            comm.recv(self._flat(t), src, stream=s)
        return self._done(tensors, tensors[0], s)

    def barrier(self, opts=None) -> _Work:
        dev = torch.device("cpu")
        if torch.cuda.is_available() and "cuda" in self._comms:
            dev = torch.device("cuda", torch.cuda.current_device())
        t = torch.zeros(4, dtype=torch.float32, device=dev)
        w = self.allreduce([t])
        w.wait()
        if dev.type == "cuda":
            torch.cuda.current_stream(dev).synchronize()
        return w

    # ---- symmetric memory (no c10d counterpart at this level: reach it through dist.group.WORLD)
    def empty_symmetric(self, shape, dtype=torch.float32, device: Optional[torch.device] = None) -> torch.Tensor:
        """Collective: a cuda tensor in symmetric memory (peer-mapped, multicast-bound), which the collectives use in
        place; tensors from torch's allocator are staged through the communicator's scratch instead."""
        dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        return self._comm(dev).empty(shape, dtype)

    def communicator(self, device_type: str = "cuda") -> Communicator:
        """The library's communicator behind this process group (split, register, tuning knobs, ...)."""
        dev = torch.device("cuda", torch.cuda.current_device()) if device_type == "cuda" else torch.device("cpu")
        return self._comm(dev)

    def shutdown(self) -> None:
        for comm in self._comms.values():
            try:
                comm.finalize()
                comm.destroy()
            except Exception:
                pass
        self._comms.clear()

    def abort(self) -> None:
        for comm in self._comms.values():
            comm.abort()

    # The base class keeps a group's name inside its registered C++ backends; a process group written in Python has
    # none, so the name torch assigns is kept here (DeviceMesh and the functional collectives look groups up by it).
    def _set_group_name(self, name: str) -> None:
        self._name = name

    @property
    def group_name(self) -> str:
        return getattr(self, "_name", "")

    def _set_group_desc(self, desc: str) -> None:
        self._desc = desc

    @property
    def group_desc(self) -> str:
        return getattr(self, "_desc", "")

    def _get_backend_name(self) -> str:
        return "mccl"

    def getBackendName(self) -> str:
        return "mccl"

    def size(self) -> int:
        return self._size

    def rank(self) -> int:
        return self._rank


class _NullCtx:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def _create(store, rank: int, size: int, timeout=None):
    return MCCLBackend(store, rank, size, timeout)


def register() -> None:
    """Idempotent registration of the "mccl" backend for cpu and cuda tensors."""
    if not hasattr(dist.Backend, "MCCL"):
        dist.Backend.register_backend("mccl", _create, devices=["cpu", "cuda"])


register()
