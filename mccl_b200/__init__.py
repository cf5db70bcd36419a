"""mccl-b200: a collective communication library for one NVSwitch box of B200 GPUs, with a TCP/CPU path.

    import mccl_b200 as mccl
    uid = mccl.get_unique_id()            # on one rank, then share it
    comm = mccl.Communicator(world, uid, rank)
    comm.all_reduce(tensor, op="avg")
"""
from ._lib import (ALGOS, ALGO_NAMES, COLLS, OPS, MCCLError, load,  # noqa: F401
                   INT8, UINT8, INT32, UINT32, INT64, UINT64, FLOAT16, BFLOAT16, FLOAT32, FLOAT64, SPLIT_NOCOLOR)
from .comm import (Communicator, forced_algo, get_unique_id, group, set_forced_algo,  # noqa: F401
                   unique_id_from_env)

__version__ = "0.1.0"
