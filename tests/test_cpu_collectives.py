"""Multi-process tests of the tcp transport on loopback (no GPU): the reference's MCCL_COLL_MAIN,
MCCL_BOOTSTRAP_MAIN and MCCL_COMM_MAIN probes (src/coll/coll.cc:110-237, src/bootstrap.cc:88-109,
src/comm.cc:360-389) grown into a matrix."""
import os

import pytest

from _mp import assert_all_ok, run_ranks


def test_baseline_config_two_ranks():
    assert_all_ok(run_ranks(2, "baseline_config"))


@pytest.mark.parametrize("world", [2, 3, 5])
def test_matrix(world):
    args = {"counts": [1, 7, 4099, 70001]} if world != 3 else {"counts": [1000, 300001], "dtypes": ["float32", "int32"]}
    assert_all_ok(run_ranks(world, "matrix", args=args, timeout=300))


def test_matrix_double_binary_tree():
    assert_all_ok(run_ranks(6, "matrix", env={"MCCL_DTREE": "1"},
                            args={"algos": ["tree"], "dtypes": ["float32"], "counts": [3, 5000]}))


def test_matrix_single_ring_no_direct():
    assert_all_ok(run_ranks(4, "matrix", env={"MCCL_DUAL_RINGS": "0", "MCCL_DIRECT_MAX_BYTES": "0", "MCCL_NSOCKS": "1"},
                            args={"algos": ["auto", "ring"], "dtypes": ["float32"], "counts": [9, 400001]}))


def test_matrix_striped_dual_ring_large():
    assert_all_ok(run_ranks(3, "matrix", env={"MCCL_NSOCKS": "4", "MCCL_PIPELINE_CHUNKS": "3"},
                            args={"algos": ["ring", "tree"], "dtypes": ["float32"], "counts": [1 << 20]}))


def test_bf16():
    assert_all_ok(run_ranks(3, "bf16"))


def test_p2p_group_alltoall_recvany():
    assert_all_ok(run_ranks(4, "p2p_group"))


def test_nonblocking_worker():
    assert_all_ok(run_ranks(2, "nonblocking"))


def test_split():
    assert_all_ok(run_ranks(5, "split_groups"))


def test_usage_errors_do_not_latch():
    assert_all_ok(run_ranks(2, "usage_errors"))


def test_ddp_matches_single_process():
    assert_all_ok(run_ranks(2, "ddp_cpu"))


def test_striped_transfer_integrity():
    assert_all_ok(run_ranks(2, "stripe_integrity", env={"MCCL_NSOCKS": "4"}))
    assert_all_ok(run_ranks(2, "stripe_integrity", env={"MCCL_NSOCKS": "1"}))


def test_ddp_gradient_accumulation():
    assert_all_ok(run_ranks(2, "ddp_accumulate"))


@pytest.mark.parametrize("world", [2, 3])
def test_fully_sharded_stack(world):
    assert_all_ok(run_ranks(world, "fsdp_stack"))


@pytest.mark.parametrize("world", [2, 3])
def test_gather_scatter_alltoallv(world):
    assert_all_ok(run_ranks(world, "rooted_and_ragged"))


def test_ddp_checkpoint_and_resume():
    assert_all_ok(run_ranks(2, "ddp_checkpoint"))


@pytest.mark.parametrize("world", [2, 3])
def test_ddp_sharded_optimizer(world):
    assert_all_ok(run_ranks(world, "ddp_zero"))


@pytest.mark.parametrize("world", [2, 3])
def test_torch_distributed_backend(world, tmp_path):
    assert_all_ok(run_ranks(world, "c10d_backend", args={"rendezvous": str(tmp_path / "rdv")}))


@pytest.mark.parametrize("world", [2, 4])
def test_model_parallel_layers(world):
    assert_all_ok(run_ranks(world, "parallel_layers"))


@pytest.mark.parametrize("world", [2, 3])
def test_tensor_parallel_llama(world):
    assert_all_ok(run_ranks(world, "llama_tp"))


def test_tensor_parallel_times_data_parallel():
    assert_all_ok(run_ranks(4, "tp_dp_2d"))


@pytest.mark.parametrize("world", [2, 4])
def test_pipeline_schedule(world):
    assert_all_ok(run_ranks(world, "pipeline_1f1b"))


def test_distributed_probes_on_loopback():
    """The bootstrap, m2m and discover probes (MCCL_BOOTSTRAP_MAIN, MCCL_M2M_MAIN, MCCL_DISCOVER_MAIN of the
    reference) as separate processes that find each other through MCCL_RANK / MCCL_WORLD_SIZE / MCCL_BOOTSTRAP_PORT."""
    import socket
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for world, args in ((3, ["bootstrap"]), (2, ["m2m", "--bytes", "1000003"]), (2, ["discover", "--transport", "tcp"])):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        procs = []
        for r in range(world):
            env = dict(os.environ, MCCL_RANK=str(r), MCCL_WORLD_SIZE=str(world), MCCL_BOOTSTRAP_PORT=str(port),
                       MCCL_BOOTSTRAP_IP="127.0.0.1")
            procs.append(subprocess.Popen([sys.executable, "-m", "mccl_b200.probe", *args], cwd=root, env=env,
                                          stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
        outs = []
        for p in procs:
            try:
                out, _ = p.communicate(timeout=120)
            except subprocess.TimeoutExpired:
                p.kill()
                out, _ = p.communicate()
            outs.append(out)
        assert all(p.returncode == 0 for p in procs), (args, outs)
        assert "FAIL" not in "".join(outs), (args, outs)
