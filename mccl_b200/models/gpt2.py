"""GPT-2 style decoder used as the data-parallel workload (24 layers, d_model 1024, 16 heads, FFN 4096,
vocab 50257, sequence 1024 for the "medium" shape, ~355M parameters).

The model is plain PyTorch in bf16: attention goes through scaled_dot_product_attention, the linear layers
through cuBLAS.  What this library adds around it is the communication (gradient buckets in symmetric
memory, all-reduced by the library's own kernels while backward still runs) and the fused optimizer step.
The token embedding is padded to a multiple of 64 rows so the tied output projection is tensor-core
friendly; the padding rows never receive probability mass (their logits are cut before the loss).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.norm import FusedLayerNorm


@dataclass
class GPT2Config:
    n_layer: int = 24
    d_model: int = 1024
    n_head: int = 16
    d_ff: int = 4096
    vocab_size: int = 50257
    seq_len: int = 1024
    dropout: float = 0.0

    @property
    def padded_vocab(self) -> int:
        return (self.vocab_size + 63) // 64 * 64

    @staticmethod
    def medium() -> "GPT2Config":
        return GPT2Config()

    @staticmethod
    def tiny() -> "GPT2Config":
        return GPT2Config(n_layer=2, d_model=128, n_head=4, d_ff=512, vocab_size=1000, seq_len=64)


class Block(nn.Module):
    def __init__(self, cfg: GPT2Config, fused: bool = True):
        super().__init__()
        norm = FusedLayerNorm if fused else nn.LayerNorm
        self.n_head = cfg.n_head
        self.ln1 = norm(cfg.d_model)
        # Separate q / k / v projections: same parameters and math as one 3d-wide projection, but the
        # backward pass gets three gradient GEMMs that accumulate into dx instead of a concatenation of
        # dq, dk, dv into one packed tensor (a pure copy that cost 7 % of the step).
        self.split_qkv = fused
        if fused:
            self.q = nn.Linear(cfg.d_model, cfg.d_model)
            self.k = nn.Linear(cfg.d_model, cfg.d_model)
            self.v = nn.Linear(cfg.d_model, cfg.d_model)
        else:
            self.qkv = nn.Linear(cfg.d_model, 3 * cfg.d_model)
        self.proj = nn.Linear(cfg.d_model, cfg.d_model)
        self.ln2 = norm(cfg.d_model)
        self.fc = nn.Linear(cfg.d_model, cfg.d_ff)
        self.out = nn.Linear(cfg.d_ff, cfg.d_model)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b, s, d = x.shape
        h = self.ln1(x)
        if self.split_qkv:
            q, k, v = (p(h).view(b, s, self.n_head, d // self.n_head).transpose(1, 2) for p in (self.q, self.k, self.v))
        else:
            q, k, v = self.qkv(h).view(b, s, 3, self.n_head, d // self.n_head).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(b, s, d))
        x = x + self.out(F.gelu(self.fc(self.ln2(x)), approximate="tanh"))
        return x


class GPT2(nn.Module):
    """Decoder-only transformer with learned positions, pre-LayerNorm blocks and a tied output projection;
    forward(idx, targets) returns the mean cross-entropy, forward(idx) the logits."""

    def __init__(self, cfg: GPT2Config, fused_loss: bool = True):
        super().__init__()
        self.cfg = cfg
        self.fused_loss = fused_loss      # the library's cross-entropy and LayerNorm kernels (CUDA, bf16); False = stock PyTorch
        self.wte = nn.Embedding(cfg.padded_vocab, cfg.d_model)
        self.wpe = nn.Embedding(cfg.seq_len, cfg.d_model)
        self.blocks = nn.ModuleList(Block(cfg, fused_loss) for _ in range(cfg.n_layer))
        self.ln_f = (FusedLayerNorm if fused_loss else nn.LayerNorm)(cfg.d_model)
        self.apply(self._init)
        for blk in self.blocks:  # GPT-2's scaled init of the residual projections
            nn.init.normal_(blk.proj.weight, std=0.02 / math.sqrt(2 * cfg.n_layer))
            nn.init.normal_(blk.out.weight, std=0.02 / math.sqrt(2 * cfg.n_layer))

    @staticmethod
    def _init(m: nn.Module) -> None:
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)
            if isinstance(m, nn.Linear) and m.bias is not None:
                nn.init.zeros_(m.bias)

    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def forward(self, idx: torch.Tensor, targets: torch.Tensor | None = None):
        b, s = idx.shape
        pos = torch.arange(s, device=idx.device)
        x = self.wte(idx) + self.wpe(pos)
        for blk in self.blocks:
            x = blk(x)
        x = self.ln_f(x)
        logits = F.linear(x, self.wte.weight)            # tied output projection, padded vocab
        if targets is None:
            return logits[..., : self.cfg.vocab_size]
        flat = logits.view(b * s, -1)
        if self.fused_loss and flat.is_cuda and flat.dtype == torch.bfloat16:
            from ..ops.loss import fused_cross_entropy
            return fused_cross_entropy(flat, targets.reshape(-1).contiguous(), self.cfg.vocab_size)
        return F.cross_entropy(flat[:, : self.cfg.vocab_size].float(), targets.reshape(-1))
