"""ctypes loader for libmccl.so and the prototypes of the C API (include/mccl.h)."""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libmccl.so"

# enums (values fixed by include/mccl.h)
SUCCESS, ERROR, SYSTEM_ERROR, INTERNAL_ERROR, INVALID_ARGUMENT, INVALID_USAGE, REMOTE_ERROR, IN_PROGRESS = range(8)
INT8, UINT8, INT32, UINT32, INT64, UINT64, FLOAT16, BFLOAT16, FLOAT32, FLOAT64 = range(10)
SUM, PROD, MAX, MIN, AVG = range(5)
ALGO_RING, ALGO_TREE, ALGO_ONESHOT, ALGO_TWOSHOT, ALGO_NVLS = range(5)
ALGO_AUTO = -1
COLL_ALLREDUCE, COLL_ALLGATHER, COLL_REDUCESCATTER, COLL_BROADCAST, COLL_REDUCE, COLL_ALLTOALL = range(6)
SPLIT_NOCOLOR = -1

OPS = {"sum": SUM, "prod": PROD, "max": MAX, "min": MIN, "avg": AVG}
ALGOS = {"ring": ALGO_RING, "tree": ALGO_TREE, "oneshot": ALGO_ONESHOT, "twoshot": ALGO_TWOSHOT,
         "nvls": ALGO_NVLS, "auto": ALGO_AUTO}
ALGO_NAMES = {v: k for k, v in ALGOS.items()}
COLLS = {"allreduce": 0, "allgather": 1, "reducescatter": 2, "broadcast": 3, "reduce": 4, "alltoall": 5}


class UniqueId(C.Structure):
    _fields_ = [("internal", C.c_char * 128)]


class Config(C.Structure):
    _fields_ = [("blocking", C.c_int), ("transport", C.c_char_p)]


class Buf(C.Structure):
    _fields_ = [("host", C.c_void_p), ("size", C.c_size_t)]


_lib = None


def load(build_if_missing: bool = True) -> C.CDLL:
    """Load libmccl.so, building it in-tree first if it is not there yet."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        if not build_if_missing:
            raise OSError(f"{_LIB_PATH} is missing; run `python -m mccl_b200._build`")
        from . import _build
        _build.build()
    lib = C.CDLL(str(_LIB_PATH), mode=os.RTLD_NOW | os.RTLD_GLOBAL)
    _declare(lib)
    _lib = lib
    return lib


def _declare(lib: C.CDLL) -> None:
    vp, sz, i, u64 = C.c_void_p, C.c_size_t, C.c_int, C.c_uint64
    P = C.POINTER

    def fn(name, res, *args):
        f = getattr(lib, name)
        f.restype = res
        f.argtypes = list(args)

    fn("mcclGetVersion", i, P(i))
    for s in ("mcclGetErrorString", "mcclResultStr", "mcclDataTypeStr", "mcclRedOpStr", "mcclAlgoStr", "mcclCollStr"):
        fn(s, C.c_char_p, i)
    fn("mcclDataSize", sz, i)
    fn("mcclGetLastError", i, vp)
    fn("mcclGetUniqueId", i, P(UniqueId))
    fn("mcclCommInitRank", i, P(vp), i, UniqueId, i)
    fn("mcclCommInitRankConfig", i, P(vp), i, UniqueId, i, P(Config))
    fn("mcclCommSplit", i, vp, i, i, P(vp), P(Config))
    for s in ("mcclCommFinalize", "mcclCommDestroy", "mcclCommAbort", "mcclCommSynchronize", "mcclCommHostBarrier"):
        fn(s, i, vp)
    for s in ("mcclCommCount", "mcclCommUserRank", "mcclCommDevice", "mcclCommGetAsyncError", "mcclCommNvlsEnabled",
              "mcclCommLastAlgo", "mcclCommCheckGuards"):
        fn(s, i, vp, P(i))
    fn("mcclCommHostAllGather", i, vp, vp, vp, sz)
    fn("mcclCommTransport", C.c_char_p, vp)
    fn("mcclAllReduce", i, vp, vp, vp, sz, i, i, vp)
    fn("mcclAllGather", i, vp, vp, vp, sz, i, vp)
    fn("mcclReduceScatter", i, vp, vp, vp, sz, i, i, vp)
    fn("mcclBroadcast", i, vp, vp, vp, sz, i, i, vp)
    fn("mcclReduce", i, vp, vp, vp, sz, i, i, i, vp)
    fn("mcclAllToAll", i, vp, vp, vp, sz, i, vp)
    psz = C.POINTER(C.c_size_t)
    fn("mcclAllToAllv", i, vp, vp, psz, psz, vp, psz, psz, i, vp)
    fn("mcclGather", i, vp, vp, vp, sz, i, i, vp)
    fn("mcclScatter", i, vp, vp, vp, sz, i, i, vp)
    fn("mcclSend", i, vp, vp, sz, i, i, vp)
    fn("mcclRecv", i, vp, vp, sz, i, i, vp)
    fn("mcclRecvAny", i, vp, vp, sz, i, P(i), vp)
    fn("mcclGroupStart", i)
    fn("mcclGroupEnd", i)
    fn("mcclGroupAbort", i)
    fn("mcclMemAlloc", i, vp, sz, P(vp))
    fn("mcclMemFree", i, vp, vp)
    fn("mcclCommRegister", i, vp, vp, sz, P(vp))
    fn("mcclCommDeregister", i, vp, vp)
    fn("mcclMemPeerPointer", i, vp, vp, i, P(vp))
    fn("mcclMemMulticastPointer", i, vp, vp, P(vp))
    fn("mcclPageAlloc", i, sz, P(vp))
    fn("mcclPageFree", None, vp)
    fn("mcclMemPoolCreate", i, sz, i, P(vp))
    fn("mcclMemPoolAlloc", i, vp, P(Buf))
    fn("mcclMemPoolFree", i, vp, P(Buf))
    fn("mcclMemPoolStats", i, vp, P(i), P(i))
    fn("mcclMemPoolDestroy", i, vp)
    fn("mcclCommPickAlgo", i, vp, i, sz, i, i, P(i))
    fn("mcclSetForcedAlgo", i, i)
    fn("mcclCommLaunchCount", i, vp, P(u64))
    fn("mcclCommSetMaxCtas", i, vp, i)
    fn("mcclCommSetCtas", i, vp, i)
    fn("mcclCommTopoXml", i, vp, P(C.c_void_p))
    fn("mcclFreeString", None, vp)
    # debug / test hooks (csrc/graph/debug.cc)
    fn("mcclDbgBtree", None, i, i, P(i))
    fn("mcclDbgDtree", None, i, i, P(i))
    fn("mcclDbgSyntheticTopoXml", i, i, i, C.c_float, i, P(C.c_void_p))
    fn("mcclDbgSyntheticChannel", i, i, i, i, i, P(i), i)
    fn("mcclDbgTunerPick", i, i, i, i, sz, i, i, C.c_char_p, P(i), P(C.c_float))
    fn("mcclDbgParseList", i, C.c_char_p, P(i))
    fn("mcclDbgHostReduce", i, vp, vp, sz, i, i)
    fn("mcclDbgHostScale", i, vp, sz, i, i)
    fn("mcclDbgXmlRoundTrip", i, C.c_char_p, P(C.c_void_p))
    fn("mcclDbgParam", C.c_int64, C.c_char_p, C.c_int64)
    fn("mcclDbgPaths", i, i, i, P(i), P(i))


class MCCLError(RuntimeError):
    def __init__(self, code: int, what: str = ""):
        self.code = code
        name = load().mcclResultStr(code).decode()
        super().__init__(f"mccl: {name} (code {code}){': ' + what if what else ''}")


def check(code: int, what: str = "") -> None:
    if code != SUCCESS and code != IN_PROGRESS:
        raise MCCLError(code, what)
