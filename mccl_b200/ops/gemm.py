"""bf16 GEMM on the 5th-generation tensor cores (tcgen05 + TMEM + TMA, csrc/device/gemm) and its fused
tensor-parallel forms.  `y = act(x @ w.T)` with x [M, K], w [N, K] (the nn.Linear weight layout)."""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib as L

_counter = {"launches": 0}
EPI = {"none": 0, "silu": 1}


def launches() -> int:
    return _counter["launches"]


def _lib():
    lib = L.load()
    if not getattr(lib, "_gemm_declared", False):
        vp, i = C.c_void_p, C.c_int
        lib.mcclTpGemm.restype = i
        lib.mcclTpGemm.argtypes = [vp, vp, vp, i, i, i, i, i, vp]
        lib.mcclTpGemm2.restype = i
        lib.mcclTpGemm2.argtypes = [vp, vp, vp, i, i, i, i, i, vp]
        lib.mcclTpAllGatherGemm.restype = i
        lib.mcclTpAllGatherGemm.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, i, vp]
        lib.mcclTpGemmReduceScatter.restype = i
        lib.mcclTpGemmReduceScatter.argtypes = [vp, vp, vp, vp, vp, vp, vp, i, i, i, C.c_uint64, vp]
        lib.mcclTpGemmLastError.restype = i
        lib.mcclTpGemmLastError.argtypes = []
        lib._gemm_declared = True
    return lib


def _stream(t, stream):
    return C.c_void_p(stream.cuda_stream if stream is not None else torch.cuda.current_stream(t.device).cuda_stream)


def supported(M: int, N: int, K: int, ranks: int = 1) -> bool:
    return M % (128 * ranks) == 0 and N % 64 == 0 and K % 64 == 0 and min(M, N, K) > 0


def gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None, epilogue: str = "none", max_ctas: int = 0,
         stream=None, two_sm: bool | None = None) -> torch.Tensor:
    """out[M, N] = act(x[M, K] @ w[N, K].T) in bf16 with fp32 accumulation, by the library's own tcgen05 kernel.
    `two_sm` selects the form in which pairs of SMs share a 256-row tile (needs M % 256 == 0); by default it is
    used whenever the shape allows it."""
    if not x.is_cuda:
        raise RuntimeError("mccl gemm runs on CUDA (sm_100a) only")
    assert x.dtype == w.dtype == torch.bfloat16 and x.is_contiguous() and w.is_contiguous()
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K
    if not supported(M, N, K):
        raise ValueError(f"unsupported GEMM shape {M}x{N}x{K}: M % 128, N % 64 and K % 64 must be 0")
    if out is None:
        out = torch.empty(M, N, device=x.device, dtype=torch.bfloat16)
    if two_sm is None:
        two_sm = M % 256 == 0
    if two_sm and M % 256:
        raise ValueError(f"the two-SM GEMM needs M % 256 == 0 (got {M})")
    fn = _lib().mcclTpGemm2 if two_sm else _lib().mcclTpGemm
    L.check(fn(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, EPI[epilogue], max_ctas, _stream(x, stream)),
            "mcclTpGemm2" if two_sm else "mcclTpGemm")
    _counter["launches"] += 1
    return out


def last_error() -> int:
    """Error code a GEMM kernel recorded on the current device since the last call (0 = none)."""
    return _lib().mcclTpGemmLastError()
