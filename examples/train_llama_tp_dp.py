"""Two-dimensional parallel training: tensor parallel inside groups of `--tp` ranks, data parallel across the groups.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        examples/train_llama_tp_dp.py --tp 4 [--sequence-parallel] [--cpu]

The world communicator is split twice (mcclCommSplit): ranks with the same `rank // tp` form a tensor-parallel group,
ranks with the same `rank % tp` a data-parallel group.  The Llama-style model lives on the tensor-parallel group; the
DDP wrapper buckets its gradients and averages them over the data-parallel group while backward runs.  `--cpu` runs
the same program on the tcp transport (fp32), which is how it is exercised on machines without a GPU.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mccl_b200 import dist  # noqa: E402
from mccl_b200.models.llama import Llama, LlamaConfig  # noqa: E402
from mccl_b200.parallel.ddp import DistributedDataParallel  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--tp", type=int, default=2)
ap.add_argument("--sequence-parallel", action="store_true")
ap.add_argument("--cpu", action="store_true")
ap.add_argument("--steps", type=int, default=10)
args = ap.parse_args()

world = dist.init_process_group(transport="tcp" if args.cpu else None)
if world.size % args.tp:
    raise SystemExit(f"world size {world.size} is not a multiple of --tp {args.tp}")
tp = world.split(world.rank // args.tp, world.rank)
dp = world.split(world.rank % args.tp, world.rank)
dev = torch.device("cpu") if args.cpu else torch.device("cuda", torch.cuda.current_device())
dtype = torch.float32 if args.cpu else torch.bfloat16

cfg = LlamaConfig.tiny() if args.cpu else LlamaConfig(n_layer=8, d_model=2048, n_head=16, d_ff=5632, vocab_size=32000, seq_len=1024)
torch.manual_seed(1000 + tp.rank)                    # replicas of one shard start equal; shards differ
model = Llama(cfg, tp, sequence_parallel=args.sequence_parallel).to(device=dev, dtype=dtype)
ddp = DistributedDataParallel(model, dp if dp.size > 1 else None, bucket_mb=25)
g = torch.Generator().manual_seed(100 + dp.rank)     # a tensor-parallel group shares its batch
for step in range(args.steps):
    tokens = torch.randint(0, cfg.vocab_size, (2 * tp.size, cfg.seq_len + 1), generator=g).to(dev)
    loss = ddp(tokens[:, :-1], tokens[:, 1:])
    loss.backward()
    ddp.finish_backward()                            # the data-parallel buckets are done before anything else touches the gradients
    model.reduce_replicated_grads()                  # shares of the replicated parameters under sequence parallelism
    ddp.step(lr=3e-4)
    if world.rank == 0:
        print(f"step {step}: loss {loss.item():.4f}", flush=True)
for c in (tp, dp):
    c.finalize(); c.destroy()
dist.destroy_process_group()
