"""LayerNorm with the library's fused forward / backward kernels (csrc/ops/layer_norm.cu) for bf16 rows of
256, 512 or 1024 elements on CUDA; anything else goes through torch.nn.functional.layer_norm."""
from __future__ import annotations

import ctypes as C

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _lib as L

_counter = {"launches": 0}
_WIDTHS = (256, 512, 1024)


def launches() -> int:
    return _counter["launches"]


def _lib():
    lib = L.load()
    if not getattr(lib, "_ln_declared", False):
        vp, i64, i = C.c_void_p, C.c_int64, C.c_int
        lib.mcclLayerNormForward.restype = i
        lib.mcclLayerNormForward.argtypes = [vp, vp, vp, vp, vp, vp, i64, i, C.c_float, vp]
        lib.mcclLayerNormBackward.restype = i
        lib.mcclLayerNormBackward.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i, vp]
        lib.mcclLayerNormPartials.restype = i
        lib.mcclLayerNormPartials.argtypes = [i64]
        lib._ln_declared = True
    return lib


class _FusedLayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).contiguous()
        rows, d = x2.shape
        y = torch.empty_like(x2)
        mean = torch.empty(rows, device=x.device, dtype=torch.float32)
        rstd = torch.empty_like(mean)
        s = C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)
        L.check(_lib().mcclLayerNormForward(x2.data_ptr(), weight.data_ptr(), bias.data_ptr(), y.data_ptr(), mean.data_ptr(),
                                            rstd.data_ptr(), rows, d, eps, s), "mcclLayerNormForward")
        _counter["launches"] += 1
        ctx.save_for_backward(x2, weight, mean, rstd)
        ctx.shape = shape
        return y.view(shape)

    @staticmethod
    def backward(ctx, dy: torch.Tensor):
        x2, weight, mean, rstd = ctx.saved_tensors
        rows, d = x2.shape
        dy2 = dy.reshape(rows, d).contiguous()
        dx = torch.empty_like(x2)
        dgamma = torch.empty_like(weight)
        dbeta = torch.empty_like(weight)
        lib = _lib()
        partial = torch.empty(lib.mcclLayerNormPartials(rows) * 2 * d, device=x2.device, dtype=torch.float32)
        s = C.c_void_p(torch.cuda.current_stream(x2.device).cuda_stream)
        L.check(lib.mcclLayerNormBackward(x2.data_ptr(), dy2.data_ptr(), weight.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                          dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), partial.data_ptr(), rows, d, s),
                "mcclLayerNormBackward")
        _counter["launches"] += 2
        return dx.view(ctx.shape), dgamma, dbeta, None


def fused_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[-1] in _WIDTHS
            and weight.is_contiguous() and weight.data_ptr() % 16 == 0)


class FusedLayerNorm(nn.Module):
    """Drop-in for nn.LayerNorm over the last dimension (same parameter names)."""

    def __init__(self, d: int, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))
        self.bias = nn.Parameter(torch.zeros(d))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if fused_supported(x, self.weight) and self.bias.data_ptr() % 16 == 0:
            return _FusedLayerNorm.apply(x, self.weight, self.bias, self.eps)
        return F.layer_norm(x, x.shape[-1:], self.weight, self.bias, self.eps)
