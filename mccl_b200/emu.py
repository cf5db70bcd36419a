"""Single-GPU emulation of a multi-rank all-reduce: n buffers on one device stand for n ranks and one
cooperative launch runs every rank's CTAs through the production kernel bodies (two-shot, one-shot, ring,
double-binary tree).  For tests on machines with one GPU and for profiling the collective kernels."""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import torch

from . import _lib as L
from .comm import _torch_dtypes


def all_reduce(tensors: Sequence[torch.Tensor], op: str = "sum", algo: str = "twoshot", ctas: int = 0, stream=None) -> None:
    """In-place all-reduce across `tensors` (same shape and dtype, all on the current CUDA device)."""
    lib = L.load()
    f = lib.mcclEmuAllReduce
    f.restype = C.c_int
    f.argtypes = [C.c_int, C.POINTER(C.c_void_p), C.c_uint64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    n = len(tensors)
    assert all(t.is_cuda and t.is_contiguous() and t.shape == tensors[0].shape and t.dtype == tensors[0].dtype for t in tensors)
    ptrs = (C.c_void_p * n)(*[t.data_ptr() for t in tensors])
    s = stream.cuda_stream if stream is not None else torch.cuda.current_stream(tensors[0].device).cuda_stream
    L.check(f(n, ptrs, tensors[0].numel(), _torch_dtypes()[tensors[0].dtype], L.OPS[op], L.ALGOS[algo], ctas, C.c_void_p(s)),
            "mcclEmuAllReduce")


def phases(tensors: Sequence[torch.Tensor], algo: str, phase_mask: int, shift: int = 0, op: str = "sum", ctas: int = 0) -> None:
    """Run only part of the ring kernel (1 = reduce steps, 2 = gather steps) or of the tree kernel (1 = up,
    2 = down) in place over `tensors`; `shift=1` makes ring rank r own / start with the r-th part."""
    lib = L.load()
    f = lib.mcclEmuPhases
    f.restype = C.c_int
    f.argtypes = [C.c_int, C.POINTER(C.c_void_p), C.c_uint64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    n = len(tensors)
    ptrs = (C.c_void_p * n)(*[t.data_ptr() for t in tensors])
    s = torch.cuda.current_stream(tensors[0].device).cuda_stream
    L.check(f(n, ptrs, tensors[0].numel(), _torch_dtypes()[tensors[0].dtype], L.OPS[op], L.ALGOS[algo], phase_mask, shift, ctas,
              C.c_void_p(s)), "mcclEmuPhases")


def one_shot_counters(rank: int, ctas: int = 8) -> list[int]:
    """One-shot call counters of the first `ctas` CTAs of emulated rank `rank` (equal after every call)."""
    lib = L.load()
    f = lib.mcclEmuOneShotCounters
    f.restype = C.c_int
    f.argtypes = [C.c_int, C.POINTER(C.c_uint64), C.c_int]
    out = (C.c_uint64 * ctas)()
    L.check(f(rank, out, ctas), "mcclEmuOneShotCounters")
    return list(out)


def destroy() -> None:
    L.load().mcclEmuDestroy()
