"""Multi-process CPU ranks over the host-memory transport: bootstrap, C API signatures, p2p, sub-communicators,
consistency checking, and the failure paths (all failures are produced on the host)."""
import pytest

from mp_util import run_ranks


def test_baseline_config_a_allreduce_ring_8mb_world2():
    res = run_ranks(2, "allreduce_ring_8mb")
    assert all("check_result: success" in out for _, out in res)


@pytest.mark.parametrize("p", [2, 3, 4])
def test_c_api_sweep(p):
    res = run_ranks(p, "sweep")
    assert all("sweep ok" in out for _, out in res)


@pytest.mark.parametrize("p", [2, 4])
def test_send_recv_batch(p):
    res = run_ranks(p, "sendrecv")
    assert all("sendrecv ok" in out for _, out in res)


def test_alltoallv_count_matrix_cross_check():
    res = run_ranks(3, "a2av_mismatch")
    assert all("a2av_mismatch ok" in out for _, out in res)


def test_staged_abort_with_budgets():
    env = {"HCCL_EXEC_TIMEOUT_MS": "20000", "HCCL_FAULT_INJECT": "stall_rank:rank=1,op=2,ms=3000"}
    res = run_ranks(2, "staged_abort", env=env)
    assert all("staged abort ok" in out for _, out in res)


def test_sub_communicator():
    res = run_ranks(4, "subcomm")
    assert all("subcomm ok" in out for _, out in res)


def test_hcom_groups_and_grad_fusion():
    res = run_ranks(4, "hcom")
    assert all("hcom ok" in out for _, out in res)


def test_one_sided_topology_overflow(tmp_path):
    dump = str(tmp_path / "stats.jsonl")
    res = run_ranks(3, "onesided", env={"HCCL_OVERFLOW_CHECK": "1", "HCCL_NVTX": "1", "HCCL_STATS_DUMP": dump})
    assert all("onesided ok" in out for _, out in res)
    import json
    lines = [json.loads(x) for x in open(dump).read().splitlines() if x.strip()]
    assert len(lines) == 3 and all(d["ops"]["AllReduce"]["calls"] >= 2 for d in lines)


def test_connection_whitelist(tmp_path):
    """HCCL_WHITELIST_DISABLE=0: the bootstrap hub only serves addresses listed under "host_ip" in HCCL_WHITELIST_FILE."""
    good = tmp_path / "wl_ok.json"
    good.write_text('{"host_ip": ["10.1.2.3", "127.0.0.1"]}')
    env = {"HCCL_WHITELIST_DISABLE": "0", "HCCL_WHITELIST_FILE": str(good), "HCCL_IF_IP": "127.0.0.1"}
    res = run_ranks(2, "sweep", env=env)
    assert all(code == 0 for code, _ in res)
    bad = tmp_path / "wl_other.json"
    bad.write_text('{"host_ip": ["10.1.2.3"]}')
    env["HCCL_WHITELIST_FILE"] = str(bad)
    env["HCCL_CONNECT_TIMEOUT"] = "5"
    res = run_ranks(2, "sweep", env=env, expect_fail_ranks=(0, 1), timeout=60)
    assert all(code != 0 for code, _ in res)
    assert "not in the whitelist" in res[0][1]
    # a hub that cannot load its list refuses to start
    env["HCCL_WHITELIST_FILE"] = str(tmp_path / "missing.json")
    res = run_ranks(1, "sweep", env=env, expect_fail_ranks=(0,), timeout=60)
    assert res[0][0] != 0 and "whitelist file" in res[0][1]


def test_param_mismatch_detected():
    res = run_ranks(3, "mismatch")
    assert all("mismatch detected" in out for _, out in res)


def test_bounded_wait_times_out_when_peer_absent():
    res = run_ranks(3, "timeout_absent_peer", env={"HCCL_EXEC_TIMEOUT_MS": "400", "HCCL_CONSISTENCY_CHECK": "0"}, args=[2.0])
    assert "timeout after" in res[0][1] and "timeout after" in res[2][1]
    assert "waiting for rank 1" in res[0][1]


def test_operator_retry_after_stall():
    env = {"HCCL_EXEC_TIMEOUT_MS": "500", "HCCL_OP_RETRY_ENABLE": "L0:1", "HCCL_OP_RETRY_PARAMS": "MaxCnt:3,HoldTime:3000,IntervalTime:50",
           "HCCL_FAULT_INJECT": "stall_rank:rank=1,op=2,ms=1500", "HCCL_CONSISTENCY_CHECK": "0"}
    res = run_ranks(2, "retry", env=env)
    assert all("retries:" in out for _, out in res)


def test_peer_exit_is_reported():
    env = {"HCCL_EXEC_TIMEOUT_MS": "3000", "HCCL_FAULT_INJECT": "exit_rank:rank=2,op=2", "HCCL_HEARTBEAT_LOST_MS": "300",
           "HCCL_HEARTBEAT_INTERVAL_MS": "50", "HCCL_CONSISTENCY_CHECK": "0"}
    res = run_ranks(3, "peer_exit", env=env, expect_fail_ranks=(2,))
    assert res[2][0] == 17
    assert "peer loss seen" in res[0][1] and "peer loss seen" in res[1][1]


def test_suspend_resume():
    res = run_ranks(2, "suspend_resume")
    assert all("suspend/resume ok" in out for _, out in res)


def test_stuck_detection_via_heartbeat():
    env = {"HCCL_EXEC_TIMEOUT_MS": "4000", "HCCL_STUCK_DETECT_MS": "500", "HCCL_HEARTBEAT_INTERVAL_MS": "50",
           "HCCL_CONSISTENCY_CHECK": "0"}
    res = run_ranks(2, "stuck", env=env)
    assert "stuck peer reported" in res[1][1]


@pytest.mark.parametrize("argv", [
    ["all_reduce_test", "-b", "8K", "-e", "128K", "-f", "4", "-d", "fp32", "-o", "sum", "-p", "3"],
    ["reduce_scatter_test", "-b", "1K", "-e", "16K", "-f", "4", "-d", "bfp16", "-o", "max", "-p", "2"],
    ["all_gather_test", "-b", "1000", "-e", "3000", "-f", "0", "-i", "1000", "-d", "int8", "-p", "4", "--algo", "ring"],
    ["broadcast_test", "-b", "4K", "-e", "4K", "-d", "int64", "-p", "3", "-r", "1"],
    ["alltoallv_test", "-b", "2K", "-e", "32K", "-f", "4", "-d", "fp32", "-p", "3", "--algo", "mesh,pairwise"],
    ["reduce_test", "-b", "4K", "-e", "64K", "-f", "4", "-d", "fp32", "-o", "sum", "-p", "4", "-r", "2", "--algo", "mesh_pipe"],
])
def test_hccl_test_command_line(argv):
    """The hccl_test-shaped CLI prints the reference tool's columns and reports success for every size (CPU ranks)."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "cann_hccl_b200.utils.hccl_test"] + argv + ["--host", "-n", "3", "-w", "1"]
    r = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = [ln.split() for ln in r.stdout.splitlines() if ln and ln[0].isdigit()]
    assert "aveg_time(us):" in r.stdout and "alg_bandwidth(GB/s):" in r.stdout and "check_result:" in r.stdout
    assert lines and all(ln[3] == "success" and float(ln[1]) > 0 for ln in lines), r.stdout
