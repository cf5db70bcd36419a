"""Process-group style convenience on top of Communicator: one default communicator per process, created
from the launcher's environment (RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT as set by
torchrun, or MCCL_RANK / MCCL_WORLD_SIZE / MCCL_BOOTSTRAP_IP / MCCL_BOOTSTRAP_PORT)."""
from __future__ import annotations

import os
from typing import Optional

from .comm import Communicator, unique_id_from_env

_default: Optional[Communicator] = None


def init_process_group(transport: Optional[str] = None, port_offset: int = 23, blocking: bool = True) -> Communicator:
    """Create (once) the default communicator.  Every rank derives the same rendezvous id from the environment,
    so no id has to be passed around; the bootstrap listens on MASTER_PORT + port_offset to stay clear of the
    launcher's own store."""
    global _default
    if _default is not None:
        return _default
    rank = int(os.environ.get("RANK", os.environ.get("MCCL_RANK", "0")))
    world = int(os.environ.get("WORLD_SIZE", os.environ.get("MCCL_WORLD_SIZE", "1")))
    if "MASTER_PORT" in os.environ:
        ip, port = os.environ.get("MASTER_ADDR", "127.0.0.1"), int(os.environ["MASTER_PORT"]) + port_offset
    else:
        ip, port = os.environ.get("MCCL_BOOTSTRAP_IP", "127.0.0.1"), int(os.environ.get("MCCL_BOOTSTRAP_PORT", "53700"))
    if transport != "tcp":
        try:
            import torch
            if torch.cuda.is_available():
                torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", str(rank))) % torch.cuda.device_count())
        except ImportError:
            pass
    _default = Communicator(world, unique_id_from_env(ip, port), rank, blocking=blocking, transport=transport)
    return _default


def default_group() -> Communicator:
    """The communicator init_process_group created."""
    if _default is None:
        raise RuntimeError("call mccl_b200.dist.init_process_group() first")
    return _default


def get_rank() -> int:
    """Rank in the default communicator."""
    return default_group().rank


def get_world_size() -> int:
    """Size of the default communicator."""
    return default_group().size


def all_reduce(tensor, op: str = "sum") -> None:
    """In-place all-reduce on the default communicator."""
    default_group().all_reduce(tensor, op=op)


def broadcast(tensor, src: int = 0) -> None:
    """In-place broadcast from rank `src`."""
    g = default_group()
    g.broadcast(tensor if g.rank == src else None, tensor, root=src)


def all_gather_into_tensor(out, inp) -> None:
    """out = every rank's `inp`, concatenated in rank order."""
    default_group().all_gather(inp, out)


def reduce_scatter_tensor(out, inp, op: str = "sum") -> None:
    """out = block `rank` of the reduction of every rank's `inp`."""
    default_group().reduce_scatter(inp, out, op=op)


def barrier() -> None:
    """Host-side barrier over the control plane."""
    default_group().host_barrier()


def destroy_process_group() -> None:
    """Finalize and destroy the default communicator."""
    global _default
    if _default is not None:
        _default.finalize()
        _default.destroy()
        _default = None
