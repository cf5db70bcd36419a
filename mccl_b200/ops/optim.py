"""Fused AdamW over flat buckets (one CUDA kernel per bucket, csrc/ops/fused_adamw.cu)."""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib as L

_counter = {"launches": 0}


def launches() -> int:
    """Number of fused optimizer kernels launched by this process so far."""
    return _counter["launches"]


def _fn():
    lib = L.load()
    f = lib.mcclFusedAdamW
    if not getattr(f, "_declared", False):
        f.restype = C.c_int
        f.argtypes = [C.c_void_p] * 5 + [C.c_uint64] + [C.c_float] * 6 + [C.c_int, C.c_int, C.c_void_p, C.c_float, C.c_void_p]
        f._declared = True
    return f


def fused_adamw_(param: torch.Tensor, master: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor,
                 grad: torch.Tensor, *, lr: float, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.0,
                 grad_scale: float = 1.0, step: int = 1, zero_grad: bool = True, norm_sq: torch.Tensor | None = None,
                 max_norm: float = 0.0, stream=None, hyper: torch.Tensor | None = None) -> None:
    """In-place AdamW step on flat tensors: bf16 `param`/`grad`, fp32 `master`/`exp_avg`/`exp_avg_sq`.  With `hyper` (three
    fp32 values on the device: lr, 1 - beta1^t, sqrt(1 - beta2^t)) the kernel reads the schedule when it runs instead of
    taking `lr` and `step` from this call, which is what a launch recorded in a CUDA graph needs."""
    if not param.is_cuda:
        raise RuntimeError("fused_adamw_ needs CUDA tensors (the kernel is sm_100a code)")
    assert param.dtype == torch.bfloat16 and grad.dtype == torch.bfloat16
    assert master.dtype == exp_avg.dtype == exp_avg_sq.dtype == torch.float32
    n = param.numel()
    assert master.numel() == n and grad.numel() == n and exp_avg.numel() == n and exp_avg_sq.numel() == n
    s = stream.cuda_stream if stream is not None else torch.cuda.current_stream(param.device).cuda_stream
    if hyper is not None:
        assert hyper.is_cuda and hyper.dtype == torch.float32 and hyper.numel() >= 3
        lib = L.load()
        g = lib.mcclFusedAdamWDeviceHyper
        if not getattr(g, "_declared", False):
            g.restype = C.c_int
            g.argtypes = [C.c_void_p] * 5 + [C.c_uint64, C.c_void_p] + [C.c_float] * 5 + [C.c_int, C.c_void_p, C.c_float, C.c_void_p]
            g._declared = True
        L.check(g(param.data_ptr(), master.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(), grad.data_ptr(), n,
                  hyper.data_ptr(), betas[0], betas[1], eps, weight_decay, grad_scale, 1 if zero_grad else 0,
                  norm_sq.data_ptr() if norm_sq is not None else None, max_norm, C.c_void_p(s)), "mcclFusedAdamWDeviceHyper")
        _counter["launches"] += 1
        return
    L.check(_fn()(param.data_ptr(), master.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(), grad.data_ptr(), n,
                  lr, betas[0], betas[1], eps, weight_decay, grad_scale, step, 1 if zero_grad else 0,
                  norm_sq.data_ptr() if norm_sq is not None else None, max_norm, C.c_void_p(s)),
            "mcclFusedAdamW")
    _counter["launches"] += 1


def sum_squares_(x: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor, accumulate: bool = False, stream=None) -> None:
    """out (one fp32 on the device) = [out +] sum(x**2) for a flat bf16 tensor; `scratch` is fp32 work memory
    (see scratch_floats) whose first element is zero."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and out.dtype == torch.float32 and scratch.dtype == torch.float32
    lib = L.load()
    f = lib.mcclSumSquaresBf16
    if not getattr(f, "_declared", False):
        f.restype = C.c_int
        f.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64, C.c_void_p, C.c_int, C.c_void_p]
        lib.mcclSumSquaresScratchFloats.restype = C.c_uint64
        lib.mcclSumSquaresScratchFloats.argtypes = [C.c_uint64]
        f._declared = True
    s = stream.cuda_stream if stream is not None else torch.cuda.current_stream(x.device).cuda_stream
    L.check(f(x.data_ptr(), x.numel(), scratch.data_ptr(), scratch.numel(), out.data_ptr(), 1 if accumulate else 0,
              C.c_void_p(s)), "mcclSumSquaresBf16")
    _counter["launches"] += 1


def scratch_floats(n: int) -> int:
    lib = L.load()
    lib.mcclSumSquaresScratchFloats.restype = C.c_uint64
    lib.mcclSumSquaresScratchFloats.argtypes = [C.c_uint64]
    return int(lib.mcclSumSquaresScratchFloats(n))


def adamw_reference(master, exp_avg, exp_avg_sq, grad, *, lr, betas, eps, weight_decay, grad_scale, step):
    """Plain PyTorch fp32 restatement of the kernel, for tests."""
    g = grad.float() * grad_scale
    exp_avg.mul_(betas[0]).add_(g, alpha=1 - betas[0])
    exp_avg_sq.mul_(betas[1]).addcmul_(g, g, value=1 - betas[1])
    bc1 = 1 - betas[0] ** step
    bc2 = 1 - betas[1] ** step
    denom = exp_avg_sq.sqrt() / (bc2 ** 0.5) + eps
    master.mul_(1 - lr * weight_decay).addcdiv_(exp_avg, denom, value=-lr / bc1)
    return master.to(torch.bfloat16)
