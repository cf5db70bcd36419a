"""Tensor-parallel FFN with sequence-sharded activations (Megatron-style sequence parallelism):

    h   = silu(all_gather(x_shard) @ W_up_shard.T)        fused: all-gather -> GEMM -> SiLU, one kernel
    out = reduce_scatter(h @ W_down_shard.T)              fused: GEMM -> reduce-scatter, one kernel

x_shard is this rank's [tokens/n, hidden] slice of the activations, W_up_shard [ffn/n, hidden] the rank's
rows of the up projection, W_down_shard [hidden, ffn/n] its columns of the down projection.  Both kernels
are the library's tcgen05 GEMM with communication warps inside (csrc/device/gemm/gemm_core.cuh); the
communicator may be a split of a larger one (TP=4 x DP=2).  The reference has no tensor-parallel code.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib as L
from ..comm import Communicator
from ..ops import gemm as G
from . import functional as PF


class TensorParallelFFN:
    """Forward-only SiLU FFN on the two fused kernels (all-gather -> GEMM -> SiLU, GEMM -> reduce-scatter); owns the
    symmetric buffers for one fixed (tokens, hidden, ffn) shape."""

    def __init__(self, comm: Communicator, tokens: int, hidden: int, ffn: int, w_up: torch.Tensor, w_down: torch.Tensor):
        n = comm.size
        if not G.supported(tokens, ffn // n, hidden, n) or not G.supported(tokens, hidden, ffn // n, n):
            raise ValueError("shapes must satisfy tokens % (128 n) == 0 and hidden, ffn/n % 64 == 0")
        assert w_up.shape == (ffn // n, hidden) and w_down.shape == (hidden, ffn // n)
        assert w_up.dtype == w_down.dtype == torch.bfloat16 and w_up.is_contiguous() and w_down.is_contiguous()
        self.comm, self.n, self.tokens, self.hidden, self.ffn = comm, n, tokens, hidden, ffn
        self.w_up, self.w_down = w_up, w_down
        dev = w_up.device
        # symmetric buffers (collective allocations, same order on every rank)
        self.x_shard = comm.empty((tokens // n, hidden), torch.bfloat16)
        self.partial = comm.empty((tokens, hidden), torch.bfloat16)
        stripes = tokens // 128
        self.flags = comm.empty(16 + stripes + n * (stripes // n) + 16, torch.int64)
        self.flags.zero_()
        self.ag_flags = torch.zeros(16, device=dev, dtype=torch.int64)
        self.x_full = torch.empty(tokens, hidden, device=dev, dtype=torch.bfloat16)
        self.h = torch.empty(tokens, ffn // n, device=dev, dtype=torch.bfloat16)
        self.out = torch.empty(tokens // n, hidden, device=dev, dtype=torch.bfloat16)
        self.accum = torch.empty(tokens // n, hidden, device=dev, dtype=torch.float32)
        self.calls = 0
        torch.cuda.synchronize(dev)
        comm.host_barrier()

    def forward(self, x_shard: torch.Tensor | None = None, stream=None) -> torch.Tensor:
        """x_shard [tokens/n, hidden] -> out [tokens/n, hidden] (this rank's rows of the FFN output)."""
        lib = G._lib()
        if x_shard is not None and x_shard.data_ptr() != self.x_shard.data_ptr():
            self.x_shard.copy_(x_shard)
        s = G._stream(self.h, stream)
        h = C.c_void_p(self.comm.handle)
        L.check(lib.mcclTpAllGatherGemm(h, self.x_shard.data_ptr(), self.x_full.data_ptr(), self.w_up.data_ptr(), self.h.data_ptr(),
                                        self.ag_flags.data_ptr(), self.tokens, self.ffn // self.n, self.hidden, G.EPI["silu"], s),
                "mcclTpAllGatherGemm")
        self.calls += 1
        L.check(lib.mcclTpGemmReduceScatter(h, self.h.data_ptr(), self.w_down.data_ptr(), self.partial.data_ptr(),
                                            self.flags.data_ptr(), self.out.data_ptr(), self.accum.data_ptr(), self.tokens, self.hidden,
                                            self.ffn // self.n, self.calls, s), "mcclTpGemmReduceScatter")
        G._counter["launches"] += 2
        return self.out

    def reference(self, x_shards: list[torch.Tensor], w_ups: list[torch.Tensor], w_downs: list[torch.Tensor]) -> torch.Tensor:
        """fp32 PyTorch restatement over every rank's inputs; returns this rank's rows of the output."""
        x = torch.cat([t.float() for t in x_shards])
        acc = torch.zeros(self.tokens, self.hidden, device=x.device)
        for wu, wd in zip(w_ups, w_downs):
            hcol = torch.nn.functional.silu(x @ wu.float().t()).to(torch.bfloat16).float()
            acc += (hcol @ wd.float().t()).to(torch.bfloat16).float()      # partial sums travel as bf16
        blk = self.tokens // self.n
        return acc[self.comm.rank * blk:(self.comm.rank + 1) * blk]


class _FusedMLPFunction(torch.autograd.Function):
    """Forward through the two fused kernels; backward with the collectives and plain matrix products.  The
    pre-activation is not kept: the backward pass recomputes it from the gathered input (one extra GEMM) instead of
    storing a [tokens, ffn / n] tensor per layer."""

    @staticmethod
    def forward(ctx, x_shard, w_up, w_down, layer):
        out = layer.forward(x_shard).clone()                       # the layer's buffers are reused by the next call
        ctx.layer = layer
        ctx.save_for_backward(layer.x_full.clone(), w_up, w_down)
        return out

    @staticmethod
    def backward(ctx, dy):
        x_full, w_up, w_down = ctx.saved_tensors
        comm = ctx.layer.comm
        dy_full = PF._ag(comm, dy.contiguous())                    # [tokens, hidden]
        u = (x_full @ w_up.t()).float()
        sig = torch.sigmoid(u)
        h = (u * sig).to(x_full.dtype)
        d_w_down = dy_full.t() @ h
        dh = (dy_full @ w_down).float()
        du = (dh * (sig * (1.0 + u * (1.0 - sig)))).to(x_full.dtype)
        d_w_up = du.t() @ x_full
        dx = PF._rs(comm, du @ w_up)                               # this rank's rows of the input gradient
        return dx, d_w_up, d_w_down, None


class FusedTensorParallelMLP(torch.nn.Module):
    """Trainable sequence-parallel SiLU MLP whose forward pass is the pair of fused kernels of TensorParallelFFN
    (all-gather -> GEMM -> SiLU, GEMM -> reduce-scatter).  Shapes are fixed at construction (the symmetric buffers
    are sized for them): x [tokens / n, hidden] -> [tokens / n, hidden], bf16, cuda."""

    def __init__(self, comm: Communicator, tokens: int, hidden: int, ffn: int, device=None):
        super().__init__()
        n = comm.size
        dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.w_up = torch.nn.Parameter(torch.randn(ffn // n, hidden, device=dev).mul_(hidden ** -0.5).to(torch.bfloat16))
        self.w_down = torch.nn.Parameter(torch.randn(hidden, ffn // n, device=dev).mul_(ffn ** -0.5).to(torch.bfloat16))
        self.layer = TensorParallelFFN(comm, tokens, hidden, ffn, self.w_up.data, self.w_down.data)

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        # the kernels read the parameters' current storage (an optimizer may have re-pointed .data)
        self.layer.w_up, self.layer.w_down = self.w_up.data, self.w_down.data
        return _FusedMLPFunction.apply(x_shard, self.w_up, self.w_down, self.layer)
