"""Failure detection, tested on the host only: a rank that exits, a rank that never joins, an injected
socket error, abort from a second thread.  Nothing here touches a GPU."""
from _mp import assert_all_ok, free_port, run_ranks


def test_abort_unblocks_parked_receive():
    assert_all_ok(run_ranks(2, "abort_unblocks", timeout=60))


def test_peer_exit_is_an_error_not_a_hang():
    # short data-path deadlines: the survivors' connection attempts to the dead rank give up in seconds
    res = run_ranks(3, "peer_dies", env={"MCCL_ACCEPT_TIMEOUT_MS": "3000", "MCCL_CONNECT_TIMEOUT_MS": "1500"}, timeout=90)
    assert_all_ok([r for r in res if r[0] != 1])


def test_missing_rank_fails_rendezvous():
    assert_all_ok(run_ranks(3, "never_joins", env={"MCCL_BOOTSTRAP_TIMEOUT_SEC": "3"}, timeout=60))


def test_injected_send_fault_surfaces():
    res = run_ranks(2, "inject_socket_fault", per_rank_env={0: {"MCCL_FAULT_INJECT": "send:9"}}, timeout=90)
    assert_all_ok(res)


def test_survivors_restart_as_a_smaller_world():
    res = run_ranks(3, "recover_smaller", args={"port2": free_port()},
                    env={"MCCL_ACCEPT_TIMEOUT_MS": "3000", "MCCL_CONNECT_TIMEOUT_MS": "1500"}, timeout=180)
    assert_all_ok([r for r in res if r[0] != 2])
