"""Data-parallel training of the GPT-2 workload with this library's DDP wrapper.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/train_gpt2_ddp.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mccl_b200 import dist  # noqa: E402
from mccl_b200.models.gpt2 import GPT2, GPT2Config  # noqa: E402
from mccl_b200.parallel.ddp import DistributedDataParallel  # noqa: E402

comm = dist.init_process_group()                     # cuda transport, device = LOCAL_RANK
dev = torch.device("cuda", torch.cuda.current_device())
torch.manual_seed(comm.rank)                         # the wrapper starts every replica from rank 0's weights
cfg = GPT2Config.medium()
model = GPT2(cfg).to(device=dev, dtype=torch.bfloat16)
ddp = DistributedDataParallel(model, comm if comm.size > 1 else None, bucket_mb=25)
g = torch.Generator().manual_seed(100 + comm.rank)   # every rank its own data
for step in range(20):
    tokens = torch.randint(0, cfg.vocab_size, (8, cfg.seq_len + 1), generator=g).to(dev, non_blocking=True)
    loss = ddp(tokens[:, :-1], tokens[:, 1:])
    loss.backward()                                  # gradient buckets are all-reduced while this runs
    ddp.step(lr=3e-4, max_grad_norm=1.0)             # fused clip + AdamW per bucket
    if comm.rank == 0 and step % 5 == 0:
        print(f"step {step}: loss {loss.item():.4f}", flush=True)
del loss                                             # no autograd graph of an eager step may outlive the recording below

# The same step recorded once in a CUDA graph and replayed: the host issues one launch per step instead of a few
# thousand, which is worth about 10 % on this model (the eager step is bound by the host).
tokens = torch.randint(0, cfg.vocab_size, (8, cfg.seq_len + 1), generator=g).to(dev)
train = ddp.graphed_step((tokens[:, :-1], tokens[:, 1:]), lr=3e-4, max_grad_norm=1.0, warmup=0)
for step in range(20, 40):
    tokens = torch.randint(0, cfg.vocab_size, (8, cfg.seq_len + 1), generator=g).pin_memory()
    loss = train(tokens[:, :-1], tokens[:, 1:])      # copied into the graph's input buffers, then one replay
    if comm.rank == 0 and step % 5 == 0:
        print(f"step {step}: loss {loss.item():.4f} (graph replay)", flush=True)
dist.destroy_process_group()
