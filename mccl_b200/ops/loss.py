"""Fused softmax cross-entropy for bf16 logits (csrc/ops/cross_entropy.cu): one read of the logits in the
forward pass, the gradient written in bf16 over the logits in the backward pass, no fp32 copy of the
rows x vocab matrix."""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib as L

_counter = {"launches": 0}


def launches() -> int:
    return _counter["launches"]


def _lib():
    lib = L.load()
    if not getattr(lib, "_ce_declared", False):
        vp, i64, i = C.c_void_p, C.c_int64, C.c_int
        lib.mcclCrossEntropyForward.restype = i
        lib.mcclCrossEntropyForward.argtypes = [vp, i64, i64, i, vp, vp, vp, vp]
        lib.mcclCrossEntropyBackward.restype = i
        lib.mcclCrossEntropyBackward.argtypes = [vp, i64, i64, i, i, vp, vp, vp, vp]
        lib._ce_declared = True
    return lib


class _FusedCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits: torch.Tensor, targets: torch.Tensor, vocab: int):
        rows, width = logits.shape
        loss = torch.empty(rows, device=logits.device, dtype=torch.float32)
        lse = torch.empty_like(loss)
        s = C.c_void_p(torch.cuda.current_stream(logits.device).cuda_stream)
        L.check(_lib().mcclCrossEntropyForward(logits.data_ptr(), rows, logits.stride(0), vocab, targets.data_ptr(),
                                               loss.data_ptr(), lse.data_ptr(), s), "mcclCrossEntropyForward")
        _counter["launches"] += 1
        ctx.save_for_backward(logits, targets, lse)
        ctx.vocab = vocab
        return loss.mean()

    @staticmethod
    def backward(ctx, grad_out: torch.Tensor):
        logits, targets, lse = ctx.saved_tensors
        rows, width = logits.shape
        g = grad_out.to(torch.float32).contiguous()
        s = C.c_void_p(torch.cuda.current_stream(logits.device).cuda_stream)
        # The gradient overwrites the logits: nothing downstream of the output projection reads them again.
        L.check(_lib().mcclCrossEntropyBackward(logits.data_ptr(), rows, logits.stride(0), ctx.vocab, width, targets.data_ptr(),
                                                lse.data_ptr(), g.data_ptr(), s), "mcclCrossEntropyBackward")
        _counter["launches"] += 1
        return logits, None, None


def fused_cross_entropy(logits: torch.Tensor, targets: torch.Tensor, vocab: int | None = None) -> torch.Tensor:
    """Mean cross-entropy of bf16 `logits` [rows, width] against int64 `targets` [rows]; columns at or beyond
    `vocab` (padding of the output projection) take no probability mass and get zero gradient."""
    if not logits.is_cuda:
        raise RuntimeError("fused_cross_entropy runs on CUDA (sm_100a) only")
    assert logits.dim() == 2 and logits.dtype == torch.bfloat16 and logits.stride(1) == 1
    assert targets.dtype == torch.int64 and targets.is_contiguous() and targets.numel() == logits.shape[0]
    return _FusedCrossEntropy.apply(logits, targets, vocab if vocab is not None else logits.shape[1])
