"""Python face of the C API: Communicator and free functions over numpy arrays and torch tensors.

Host buffers (numpy arrays, CPU tensors) go with the "tcp" transport, CUDA tensors with "cuda"; the
pointer, element count and dtype are taken from the object and handed to libmccl unchanged.
"""
from __future__ import annotations

import atexit
import ctypes as C
import weakref
from contextlib import contextmanager
from typing import Optional

import numpy as np

from . import _lib as L

try:  # torch is optional for the tcp transport
    import torch
except Exception:  # pragma: no cover
    torch = None

_NP_DTYPES = {
    np.dtype(np.int8): L.INT8, np.dtype(np.uint8): L.UINT8, np.dtype(np.int32): L.INT32,
    np.dtype(np.uint32): L.UINT32, np.dtype(np.int64): L.INT64, np.dtype(np.uint64): L.UINT64,
    np.dtype(np.float16): L.FLOAT16, np.dtype(np.float32): L.FLOAT32, np.dtype(np.float64): L.FLOAT64,
}


def _torch_dtypes():
    return {
        torch.int8: L.INT8, torch.uint8: L.UINT8, torch.int32: L.INT32, torch.int64: L.INT64,
        torch.float16: L.FLOAT16, torch.bfloat16: L.BFLOAT16, torch.float32: L.FLOAT32, torch.float64: L.FLOAT64,
        **({torch.uint32: L.UINT32, torch.uint64: L.UINT64} if hasattr(torch, "uint32") else {}),
    }


def _describe(buf, dtype: Optional[int] = None):
    """(pointer, element count, mccl dtype, is_cuda) of a numpy array or torch tensor."""
    if buf is None:
        return None, 0, dtype, False
    if torch is not None and isinstance(buf, torch.Tensor):
        if not buf.is_contiguous():
            raise ValueError("mccl needs contiguous tensors")
        dt = dtype if dtype is not None else _torch_dtypes()[buf.dtype]
        return buf.data_ptr(), buf.numel(), dt, buf.is_cuda
    a = buf
    if not isinstance(a, np.ndarray):
        raise TypeError(f"unsupported buffer type {type(buf)}")
    if not a.flags["C_CONTIGUOUS"]:
        raise ValueError("mccl needs C-contiguous arrays")
    dt = dtype if dtype is not None else _NP_DTYPES[a.dtype]
    return a.ctypes.data, a.size, dt, False


def _check_pair(what: str, send, recv, num: int = 1, den: int = 1) -> None:
    """Refuse a send / recv pair before it reaches the library: the same kind of buffer, dtype and device, and a
    receive buffer of at least num/den times the send buffer's elements.  (A receive buffer that is too small would
    be written past its end on the device, where nothing can raise.)"""
    if send is None or recv is None:
        return
    is_t = torch is not None and isinstance(send, torch.Tensor)
    if is_t != (torch is not None and isinstance(recv, torch.Tensor)):
        raise TypeError(f"{what}: send and recv must both be torch tensors or both numpy arrays")
    if send.dtype != recv.dtype:
        raise ValueError(f"{what}: send is {send.dtype}, recv is {recv.dtype}")
    if is_t and send.device != recv.device:
        raise ValueError(f"{what}: send is on {send.device}, recv on {recv.device}")
    have = recv.numel() if is_t else recv.size
    give = send.numel() if is_t else send.size
    if have * den < give * num:
        raise ValueError(f"{what}: recv holds {have} elements, needs {give * num // den} for a send of {give}")


def _stream_of(buf, stream):
    if stream is not None:
        return C.c_void_p(stream if isinstance(stream, int) else stream.cuda_stream)
    if torch is not None and isinstance(buf, torch.Tensor) and buf.is_cuda:
        return C.c_void_p(torch.cuda.current_stream(buf.device).cuda_stream)
    return C.c_void_p(0)


def get_unique_id() -> bytes:
    """mcclGetUniqueId: 128 bytes to create on one rank and hand to the others (it names a listener of this process)."""
    uid = L.UniqueId()
    L.check(L.load().mcclGetUniqueId(C.byref(uid)), "mcclGetUniqueId")
    return C.string_at(C.byref(uid), 128)      # the raw 128 bytes (a c_char array would stop at the first NUL)


def unique_id_from_env(ip: str, port: int) -> bytes:
    """The shared-by-convention id every rank can build from (ip, port) without talking to anyone."""
    raw = ip.encode().ljust(64, b"\0") + int(port).to_bytes(2, "little") + b"\0" * 6 + (0).to_bytes(8, "little")
    return raw.ljust(128, b"\0")


def set_forced_algo(algo) -> None:
    """Force one algorithm ("ring", "tree", "oneshot", "twoshot", "nvls") for this thread's next calls; "auto" restores the tuner."""
    a = L.ALGOS[algo] if isinstance(algo, str) else int(algo)
    L.check(L.load().mcclSetForcedAlgo(a), "mcclSetForcedAlgo")


@contextmanager
def forced_algo(algo):
    """`with forced_algo("ring"): ...` — set_forced_algo for the duration of the block."""
    set_forced_algo(algo)
    try:
        yield
    finally:
        set_forced_algo("auto")


@contextmanager
def group():
    """mcclGroupStart / mcclGroupEnd around the block: the calls inside are recorded and issued together at its end."""
    lib = L.load()
    L.check(lib.mcclGroupStart())
    try:
        yield
    except BaseException:
        lib.mcclGroupAbort()
        raise
    L.check(lib.mcclGroupEnd(), "mcclGroupEnd")


_live = weakref.WeakSet()


@atexit.register
def _destroy_live_communicators() -> None:
    # A process that exits with peer mappings and multicast bindings still in place leaves the tear-down to
    # the driver at an arbitrary moment; destroying explicitly unbinds and unmaps in order.
    for comm in list(_live):
        try:
            comm.destroy()
        except Exception:
            pass


class Communicator:
    """One rank's handle on a communicator (wraps mcclComm_t)."""

    def __init__(self, n_ranks: int, unique_id: bytes, rank: int, blocking: bool = True,
                 transport: Optional[str] = None, _handle: Optional[int] = None):
        self._lib = L.load()
        self._h = C.c_void_p(_handle) if _handle is not None else C.c_void_p()
        self._transport_keepalive = transport.encode() if transport else None
        if _handle is None:
            uid = L.UniqueId()
            C.memmove(C.byref(uid), bytes(unique_id).ljust(128, b"\0")[:128], 128)
            cfg = L.Config(1 if blocking else 0, self._transport_keepalive)
            L.check(self._lib.mcclCommInitRankConfig(C.byref(self._h), n_ranks, uid, rank, C.byref(cfg)),
                    "mcclCommInitRankConfig")
        self._sym = {}
        _live.add(self)

    # ---- queries
    @property
    def handle(self) -> int:
        """The mcclComm_t as an integer (for ctypes calls into the C API)."""
        return self._h.value

    def _q(self, fn) -> int:
        v = C.c_int()
        L.check(fn(self._h, C.byref(v)))
        return v.value

    @property
    def rank(self) -> int:
        """This process's rank in the communicator."""
        return self._q(self._lib.mcclCommUserRank)

    @property
    def size(self) -> int:
        """Number of ranks."""
        return self._q(self._lib.mcclCommCount)

    @property
    def device(self) -> int:
        """CUDA device ordinal of the cuda transport (-1 on tcp)."""
        return self._q(self._lib.mcclCommDevice)

    @property
    def transport(self) -> str:
        """"tcp" or "cuda"."""
        return self._lib.mcclCommTransport(self._h).decode()

    @property
    def nvls(self) -> bool:
        """Whether NVSwitch multicast (NVLS) is mapped for this communicator."""
        return bool(self._q(self._lib.mcclCommNvlsEnabled))

    @property
    def last_algo(self) -> str:
        """Algorithm the most recent collective ran with ("ring", "tree", "oneshot", "twoshot", "nvls")."""
        return L.ALGO_NAMES.get(self._q(self._lib.mcclCommLastAlgo), "none")

    @property
    def launch_count(self) -> int:
        """Device kernels this communicator has launched so far."""
        v = C.c_uint64()
        L.check(self._lib.mcclCommLaunchCount(self._h, C.byref(v)))
        return v.value

    def guards_intact(self) -> bool:
        """Debug aid: the guard word behind the device flag arrays is untouched."""
        return bool(self._q(self._lib.mcclCommCheckGuards))

    def async_error(self) -> int:
        """mcclCommGetAsyncError: 0, mcclInProgress while non-blocking tcp work runs, or the latched fatal error."""
        return self._q(self._lib.mcclCommGetAsyncError)

    def pick_algo(self, coll: str, nbytes: int, dtype: int = L.FLOAT32, op: str = "sum") -> str:
        """The algorithm the tuner would choose for this call."""
        a = C.c_int()
        L.check(self._lib.mcclCommPickAlgo(self._h, L.COLLS[coll], nbytes, dtype, L.OPS[op], C.byref(a)))
        return L.ALGO_NAMES[a.value]

    def set_max_ctas(self, n: int) -> None:
        """Cap the CTAs of every collective kernel (0 = tuner default), leaving SMs to overlapped compute."""
        L.check(self._lib.mcclCommSetMaxCtas(self._h, n))

    def set_ctas(self, n: int) -> None:
        """Tuning aid: exactly n CTAs for every collective kernel (0 = planner's choice)."""
        L.check(self._lib.mcclCommSetCtas(self._h, n))

    def topo_xml(self) -> str:
        """Topology, per-algorithm plans and tuner constants as XML."""
        p = C.c_void_p()
        L.check(self._lib.mcclCommTopoXml(self._h, C.byref(p)))
        s = C.string_at(p).decode()
        self._lib.mcclFreeString(p)
        return s

    # ---- lifecycle
    def split(self, color: int, key: int = 0, blocking: Optional[bool] = None) -> Optional["Communicator"]:
        """mcclCommSplit: collective over this communicator; ranks with one color form a new communicator ordered by
        (key, rank); color mccl_b200.SPLIT_NOCOLOR returns None."""
        h = C.c_void_p()
        cfg = None
        if blocking is not None:
            cfg = C.byref(L.Config(1 if blocking else 0, self._transport_keepalive or self.transport.encode()))
        L.check(self._lib.mcclCommSplit(self._h, color, key, C.byref(h), cfg), "mcclCommSplit")
        if not h.value:
            return None
        return Communicator(0, b"", 0, _handle=h.value)

    def synchronize(self) -> None:
        """Wait for queued non-blocking tcp work (the cuda transport is synchronised through its stream)."""
        L.check(self._lib.mcclCommSynchronize(self._h), "mcclCommSynchronize")

    def finalize(self) -> None:
        """Drain outstanding work and pass a barrier; call before destroy on a healthy communicator."""
        L.check(self._lib.mcclCommFinalize(self._h), "mcclCommFinalize")

    def abort(self) -> None:
        """Unblock every thread parked in this communicator and refuse further work; frees nothing."""
        L.check(self._lib.mcclCommAbort(self._h), "mcclCommAbort")

    def destroy(self) -> None:
        """Free the communicator and its symmetric memory."""
        _live.discard(self)
        if self._h:
            self._sym.clear()
            self._lib.mcclCommDestroy(self._h)
            self._h = C.c_void_p()

    def host_barrier(self) -> None:
        """Barrier over the control plane (host side only; says nothing about GPU work)."""
        L.check(self._lib.mcclCommHostBarrier(self._h), "mcclCommHostBarrier")

    def host_all_gather(self, payload: bytes) -> list:
        """All-gather of equal-size byte strings over the control plane."""
        n = self.size
        out = C.create_string_buffer(len(payload) * n)
        L.check(self._lib.mcclCommHostAllGather(self._h, payload, out, len(payload)), "mcclCommHostAllGather")
        raw = out.raw
        return [raw[i * len(payload):(i + 1) * len(payload)] for i in range(n)]

    # ---- collectives
    def all_reduce(self, send, recv=None, op: str = "sum", dtype: Optional[int] = None, stream=None) -> None:
        """recv (default: in place) = op over the ranks' `send`; torch tensors, numpy arrays, or raw pointers with `dtype`."""
        recv = send if recv is None else recv
        _check_pair("all_reduce", send, recv)
        sp, cnt, dt, _ = _describe(send, dtype)
        rp, _, _, _ = _describe(recv, dtype)
        L.check(self._lib.mcclAllReduce(self._h, sp, rp, cnt, dt, L.OPS[op], _stream_of(send, stream)), "mcclAllReduce")

    def all_gather(self, send, recv, dtype: Optional[int] = None, stream=None) -> None:
        """recv = the ranks' `send` concatenated in rank order (`send` may be this rank's slot of `recv`)."""
        _check_pair("all_gather", send, recv, self.size)
        sp, cnt, dt, _ = _describe(send, dtype)
        rp, _, _, _ = _describe(recv, dtype)
        L.check(self._lib.mcclAllGather(self._h, sp, rp, cnt, dt, _stream_of(send, stream)), "mcclAllGather")

    def reduce_scatter(self, send, recv, op: str = "sum", dtype: Optional[int] = None, stream=None) -> None:
        """recv = block `rank` of op over the ranks' `send` (n blocks of recv's size)."""
        _check_pair("reduce_scatter", recv, send, self.size)      # send holds one block of recv's size per rank
        sp, _, dt, _ = _describe(send, dtype)
        rp, cnt, _, _ = _describe(recv, dtype)
        L.check(self._lib.mcclReduceScatter(self._h, sp, rp, cnt, dt, L.OPS[op], _stream_of(send, stream)),
                "mcclReduceScatter")

    def broadcast(self, send, recv, root: int = 0, dtype: Optional[int] = None, stream=None) -> None:
        """recv on every rank = the root's `send` (may be None elsewhere)."""
        _check_pair("broadcast", recv, send)                      # the root sends as many elements as everyone receives
        rp, cnt, dt, _ = _describe(recv, dtype)
        sp = _describe(send, dtype)[0] if send is not None else None
        L.check(self._lib.mcclBroadcast(self._h, sp, rp, cnt, dt, root, _stream_of(recv, stream)), "mcclBroadcast")

    def reduce(self, send, recv, op: str = "sum", root: int = 0, dtype: Optional[int] = None, stream=None) -> None:
        """The root's recv = op over the ranks' `send` (`recv` may be None elsewhere)."""
        _check_pair("reduce", send, recv)
        sp, cnt, dt, _ = _describe(send, dtype)
        rp = _describe(recv, dtype)[0] if recv is not None else None
        L.check(self._lib.mcclReduce(self._h, sp, rp, cnt, dt, L.OPS[op], root, _stream_of(send, stream)), "mcclReduce")

    def all_to_all(self, send, recv, dtype: Optional[int] = None, stream=None) -> None:
        """Block j of `send` goes to rank j; block i of `recv` came from rank i (equal blocks)."""
        _check_pair("all_to_all", send, recv)
        if _describe(send, dtype)[1] % self.size:
            raise ValueError(f"all_to_all: {_describe(send, dtype)[1]} elements do not split into {self.size} equal blocks")
        sp, cnt, dt, _ = _describe(send, dtype)
        rp, _, _, _ = _describe(recv, dtype)
        L.check(self._lib.mcclAllToAll(self._h, sp, rp, cnt // self.size, dt, _stream_of(send, stream)), "mcclAllToAll")

    def all_to_all_v(self, send, send_counts, recv, recv_counts, stream=None) -> None:
        """All-to-all with a different element count per peer: `send_counts[j]` elements of flat `send` (consecutive
        segments, rank order) go to rank j, `recv_counts[i]` elements arrive from rank i into consecutive segments of
        flat `recv`.  Issued as one group of Send / Recv pairs (plus a local copy of the own segment)."""
        n = self.size
        if len(send_counts) != n or len(recv_counts) != n:
            raise ValueError("one count per rank is required")
        _check_pair("all_to_all_v", send, recv, 0)
        sp, ns, dt, _ = _describe(send)
        rp, nr, _, _ = _describe(recv)
        if sum(int(c) for c in send_counts) > ns or sum(int(c) for c in recv_counts) > nr:
            raise ValueError("all_to_all_v: the counts add up to more elements than the buffers hold")
        arr = C.c_size_t * n
        sc, rc = arr(*[int(c) for c in send_counts]), arr(*[int(c) for c in recv_counts])
        sd, rd = arr(), arr()
        for i in range(1, n):
            sd[i], rd[i] = sd[i - 1] + sc[i - 1], rd[i - 1] + rc[i - 1]
        L.check(self._lib.mcclAllToAllv(self._h, sp, sc, sd, rp, rc, rd, dt, _stream_of(send, stream)), "mcclAllToAllv")

    def gather(self, send, recv, root: int = 0, dtype: Optional[int] = None, stream=None) -> None:
        """The root's `recv` = every rank's `send` in rank order (`recv` may be None elsewhere)."""
        _check_pair("gather", send, recv, self.size)
        sp, cnt, dt, _ = _describe(send, dtype)
        rp = _describe(recv, dtype)[0] if recv is not None else None
        L.check(self._lib.mcclGather(self._h, sp, rp, cnt, dt, root, _stream_of(send, stream)), "mcclGather")

    def scatter(self, send, recv, root: int = 0, dtype: Optional[int] = None, stream=None) -> None:
        """`recv` on rank p = block p of the root's `send` (`send` may be None elsewhere)."""
        _check_pair("scatter", recv, send, self.size)
        rp, cnt, dt, _ = _describe(recv, dtype)
        sp = _describe(send, dtype)[0] if send is not None else None
        L.check(self._lib.mcclScatter(self._h, sp, rp, cnt, dt, root, _stream_of(recv, stream)), "mcclScatter")

    def send(self, buf, peer: int, dtype: Optional[int] = None, stream=None) -> None:
        """Send `buf` to `peer`; inside `with mccl_b200.group():` it is batched with the other calls."""
        p, cnt, dt, _ = _describe(buf, dtype)
        L.check(self._lib.mcclSend(self._h, p, cnt, dt, peer, _stream_of(buf, stream)), "mcclSend")

    def recv(self, buf, peer: int, dtype: Optional[int] = None, stream=None) -> None:
        """Receive into `buf` from `peer`."""
        p, cnt, dt, _ = _describe(buf, dtype)
        L.check(self._lib.mcclRecv(self._h, p, cnt, dt, peer, _stream_of(buf, stream)), "mcclRecv")

    def recv_any(self, buf, dtype: Optional[int] = None, stream=None) -> int:
        """Receive into `buf` from whichever rank sends first; returns its rank."""
        p, cnt, dt, _ = _describe(buf, dtype)
        src = C.c_int(-1)
        L.check(self._lib.mcclRecvAny(self._h, p, cnt, dt, C.byref(src), _stream_of(buf, stream)), "mcclRecvAny")
        return src.value

    # ---- symmetric memory (cuda transport)
    def alloc_raw(self, nbytes: int) -> int:
        p = C.c_void_p()
        L.check(self._lib.mcclMemAlloc(self._h, nbytes, C.byref(p)), "mcclMemAlloc")
        return p.value

    def free_raw(self, ptr: int) -> None:
        self._sym.pop(ptr, None)
        L.check(self._lib.mcclMemFree(self._h, C.c_void_p(ptr)), "mcclMemFree")

    def empty(self, shape, dtype=None):
        """A CUDA tensor in symmetric memory (collective: every rank calls with the same shape)."""
        if torch is None:
            raise RuntimeError("torch is required for symmetric tensors")
        dtype = dtype or torch.float32
        numel = int(np.prod(shape)) if not isinstance(shape, int) else int(shape)
        nbytes = max(numel * torch.empty((), dtype=dtype).element_size(), 16)
        ptr = self.alloc_raw(nbytes)
        holder = _SymBlock(self, ptr, nbytes)
        t = torch.as_tensor(holder, device=f"cuda:{self.device}").view(dtype)[:numel].view(shape)
        self._sym[t.data_ptr()] = holder
        return t

    def pool(self, nbytes: int) -> "SymmetricPool":
        """Collective: one symmetric allocation of `nbytes` to carve tensors from without further collectives (see
        SymmetricPool)."""
        return SymmetricPool(self, nbytes)

    def register(self, tensor) -> int:
        """Collective: map an existing CUDA tensor (cudaMalloc memory, e.g. from torch's allocator) into every
        peer through CUDA IPC so the peer-load algorithms use it in place.  Returns a handle for deregister()."""
        h = C.c_void_p()
        nbytes = tensor.numel() * tensor.element_size()
        L.check(self._lib.mcclCommRegister(self._h, C.c_void_p(tensor.data_ptr()), nbytes, C.byref(h)), "mcclCommRegister")
        return h.value

    def deregister(self, handle: int) -> None:
        L.check(self._lib.mcclCommDeregister(self._h, C.c_void_p(handle)), "mcclCommDeregister")

    def peer_pointer(self, tensor_or_ptr, peer: int) -> int:
        p = tensor_or_ptr.data_ptr() if hasattr(tensor_or_ptr, "data_ptr") else int(tensor_or_ptr)
        out = C.c_void_p()
        L.check(self._lib.mcclMemPeerPointer(self._h, C.c_void_p(p), peer, C.byref(out)))
        return out.value or 0

    def multicast_pointer(self, tensor_or_ptr) -> int:
        p = tensor_or_ptr.data_ptr() if hasattr(tensor_or_ptr, "data_ptr") else int(tensor_or_ptr)
        out = C.c_void_p()
        L.check(self._lib.mcclMemMulticastPointer(self._h, C.c_void_p(p), C.byref(out)))
        return out.value or 0


class _SymBlock:
    """Exposes a symmetric allocation through __cuda_array_interface__ so torch can wrap it without a copy."""

    def __init__(self, comm: Communicator, ptr: int, nbytes: int):
        self.comm, self.ptr, self.nbytes = comm, ptr, nbytes
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
        }


class SymmetricPool:
    """Tensors carved from ONE symmetric allocation (mcclSymPool*).  Creating and destroying the pool are collective;
    `empty` and `free` are local bookkeeping, so they cost microseconds instead of a handle exchange, but every rank
    must make the same sequence of `empty` / `free` calls (a tensor is then the same part of the allocation on every
    rank, which is what the kernels assume of symmetric buffers)."""

    def __init__(self, comm: Communicator, nbytes: int):
        self.comm = comm
        self._lib = comm._lib
        self._p = C.c_void_p()
        self._declare()
        L.check(self._lib.mcclSymPoolCreate(comm._h, C.c_size_t(nbytes), C.byref(self._p)), "mcclSymPoolCreate")
        self._holders = {}

    def _declare(self) -> None:
        lib = self._lib
        if getattr(lib, "_sympool_declared", False):
            return
        vp, sz = C.c_void_p, C.c_size_t
        lib.mcclSymPoolCreate.restype = C.c_int; lib.mcclSymPoolCreate.argtypes = [vp, sz, C.POINTER(vp)]
        lib.mcclSymPoolAlloc.restype = C.c_int; lib.mcclSymPoolAlloc.argtypes = [vp, sz, C.POINTER(vp)]
        lib.mcclSymPoolFree.restype = C.c_int; lib.mcclSymPoolFree.argtypes = [vp, vp]
        lib.mcclSymPoolStats.restype = C.c_int; lib.mcclSymPoolStats.argtypes = [vp, C.POINTER(sz), C.POINTER(sz), C.POINTER(sz)]
        lib.mcclSymPoolDestroy.restype = C.c_int; lib.mcclSymPoolDestroy.argtypes = [vp]
        lib._sympool_declared = True

    def alloc_raw(self, nbytes: int) -> int:
        p = C.c_void_p()
        L.check(self._lib.mcclSymPoolAlloc(self._p, C.c_size_t(nbytes), C.byref(p)), "mcclSymPoolAlloc")
        return p.value

    def free_raw(self, ptr: int) -> None:
        self._holders.pop(ptr, None)
        L.check(self._lib.mcclSymPoolFree(self._p, C.c_void_p(ptr)), "mcclSymPoolFree")

    def empty(self, shape, dtype=None):
        """A tensor from the pool (CUDA on the cuda transport, host memory on tcp); local, same call order on every rank."""
        dtype = dtype or torch.float32
        numel = int(np.prod(shape)) if not isinstance(shape, int) else int(shape)
        nbytes = max(numel * torch.empty((), dtype=dtype).element_size(), 16)
        ptr = self.alloc_raw(nbytes)
        if self.comm.transport == "cuda":
            holder = _SymBlock(self.comm, ptr, nbytes)
            t = torch.as_tensor(holder, device=f"cuda:{self.comm.device}").view(dtype)[:numel].view(shape)
        else:
            holder = (C.c_char * nbytes).from_address(ptr)
            t = torch.frombuffer(holder, dtype=torch.uint8).view(dtype)[:numel].view(shape)
        self._holders[ptr] = holder
        return t

    def free(self, tensor) -> None:
        self.free_raw(tensor.data_ptr())

    def stats(self) -> dict:
        """{'total', 'in_use', 'largest_free'} in bytes."""
        a, b, c = C.c_size_t(), C.c_size_t(), C.c_size_t()
        L.check(self._lib.mcclSymPoolStats(self._p, C.byref(a), C.byref(b), C.byref(c)))
        return {"total": a.value, "in_use": b.value, "largest_free": c.value}

    def destroy(self) -> None:
        """Collective: give the allocation back (no tensor from the pool may be used afterwards)."""
        if self._p:
            self._holders.clear()
            L.check(self._lib.mcclSymPoolDestroy(self._p), "mcclSymPoolDestroy")
            self._p = C.c_void_p()
