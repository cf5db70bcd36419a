#!/usr/bin/env python
"""Two training steps of the flagship workload (GPT-2-medium shape, micro-batch 8, bf16, one GPU) with as
little around them as possible: the command to put under `ncu --metrics gpu__time_duration.sum` for a
per-kernel launch list of one step (the first step warms up, capture the second with -s/-c).

    python bench/step_launches.py            # prints the number of CUDA kernels it expects per step
"""
from __future__ import annotations

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mccl_b200.models.gpt2 import GPT2, GPT2Config  # noqa: E402
from mccl_b200.ops import optim  # noqa: E402
from mccl_b200.parallel.ddp import DistributedDataParallel  # noqa: E402


def main() -> int:
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    torch.manual_seed(1234)
    cfg = GPT2Config.medium()
    model = GPT2(cfg).to(device=dev, dtype=torch.bfloat16)
    ddp = DistributedDataParallel(model, None, bucket_mb=25.0)
    tokens = torch.randint(0, cfg.vocab_size, (8, cfg.seq_len + 1), device=dev)
    for step in range(2):
        before = optim.launches()
        loss = ddp(tokens[:, :-1], tokens[:, 1:])
        loss.backward()
        ddp.step(lr=3e-4, max_grad_norm=1.0)
        torch.cuda.synchronize()
        print(f"step {step}: loss {loss.item():.4f}, {optim.launches() - before} launches of this library's kernels", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
