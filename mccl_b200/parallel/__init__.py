"""Parallel training on the library's communicators.

    ddp         DistributedDataParallel: gradient buckets in symmetric memory reduced during backward, fused optimizer
                step, gradient accumulation, sharded optimizer (ZeRO-1), checkpointing
    fsdp        FullyShardedStack: parameters, gradients and optimizer state sharded per block (ZeRO-3)
    tp          TensorParallelFFN / FusedTensorParallelMLP: the fused all-gather -> GEMM and GEMM -> reduce-scatter kernels
    functional  the collectives as differentiable functions, ring attention
    layers      column / row parallel linear, sequence-parallel MLP, Ulysses and ring attention, expert-parallel MoE
    pipeline    PipelineStage: 1F1B over grouped Send / Recv

Submodules are imported on demand (`from mccl_b200.parallel import layers`): `tp` needs CUDA at call time, the others
run on cpu tensors over the tcp transport as well.
"""
