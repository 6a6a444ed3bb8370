"""Public C API contracts: result codes, argument validation, configuration, rank table, selector, env parsing."""
import ctypes as C
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import cann_hccl_b200 as H
from cann_hccl_b200 import _lib as L


@pytest.fixture(scope="module")
def one():
    c = H.Communicator.init_local(1, device=False)
    yield c
    c.destroy()


def test_error_strings():
    lib = L.lib()
    want = {0: "no error", 1: "parameter error", 2: "empty pointer", 5: "not support feature", 9: "timeout", 20: "try again",
            21: "error cqe", 22: "error communicator suspending", 99: "unknow error"}
    for code, text in want.items():
        assert lib.HcclGetErrorString(code).decode() == text


def test_enum_values_match_hccl():
    assert (L.INT8, L.INT16, L.INT32, L.FP16, L.FP32, L.INT64, L.UINT64, L.UINT8, L.UINT16, L.UINT32, L.FP64, L.BFP16) == tuple(range(12))
    assert (L.SUM, L.PROD, L.MAX, L.MIN) == (0, 1, 2, 3)
    assert C.sizeof(L.RootInfo) == 4108
    assert C.sizeof(L.CommConfig) == 24 + 4 + 4 + 128 + 128 + 12


def test_null_and_zero_count(one):
    lib = L.lib()
    a = np.zeros(4, np.float32)
    assert lib.HcclAllReduce(None, a.ctypes.data, 4, L.FP32, L.SUM, one.handle, None) == L.E_PTR
    assert lib.HcclAllReduce(a.ctypes.data, None, 4, L.FP32, L.SUM, one.handle, None) == L.E_PTR
    assert lib.HcclAllReduce(a.ctypes.data, a.ctypes.data, 4, L.FP32, L.SUM, None, None) == L.E_PTR
    # count 0 succeeds before pointers are looked at (reference: early return with a warning)
    assert lib.HcclAllReduce(None, None, 0, L.FP32, L.SUM, one.handle, None) == L.SUCCESS
    assert lib.HcclAllGather(None, None, 0, L.FP32, one.handle, None) == L.SUCCESS
    assert lib.HcclBatchSendRecv(None, 0, one.handle, None) == L.SUCCESS
    assert lib.HcclGetRankSize(one.handle, None) == L.E_PTR
    assert lib.HcclGetRootInfo(None) == L.E_PTR


def test_dtype_and_op_checks(one):
    lib = L.lib()
    a = np.zeros(16, np.float32)
    p = a.ctypes.data
    assert lib.HcclAllReduce(p, p, 4, 77, L.SUM, one.handle, None) == L.E_PARA
    assert lib.HcclAllReduce(p, p, 4, L.FP32, 9, one.handle, None) == L.E_PARA
    assert lib.HcclAllReduce(p, p, 1, L.INT128, L.SUM, one.handle, None) == L.E_NOT_SUPPORT  # transport-only type
    assert lib.HcclAllReduce(p, p, 4, L.FP8E4M3, L.SUM, one.handle, None) == L.E_NOT_SUPPORT
    assert lib.HcclAllGather(p, p, 1, L.INT128, one.handle, None) == L.SUCCESS  # copies are fine
    assert lib.HcclBroadcast(p, 4, L.FP32, 5, one.handle, None) == L.E_PARA  # root outside the communicator
    assert lib.HcclAllReduce(p, p, 1 << 40, L.FP32, L.SUM, one.handle, None) == L.E_PARA  # above SYS_MAX_COUNT


def test_alltoall_contract(one):
    lib = L.lib()
    a, b = np.zeros(4, np.float32), np.zeros(4, np.float32)
    assert lib.HcclAlltoAll(a.ctypes.data, 4, L.FP32, b.ctypes.data, 3, L.FP32, one.handle, None) == L.E_PARA
    assert lib.HcclAlltoAll(a.ctypes.data, 4, L.FP32, b.ctypes.data, 4, L.FP16, one.handle, None) == L.E_PARA
    assert lib.HcclAlltoAll(a.ctypes.data, 4, L.FP32, a.ctypes.data, 4, L.FP32, one.handle, None) == L.E_PARA
    a[:] = [1, 2, 3, 4]
    assert lib.HcclAlltoAll(a.ctypes.data, 4, L.FP32, b.ctypes.data, 4, L.FP32, one.handle, None) == L.SUCCESS
    np.testing.assert_array_equal(a, b)


def test_reduce_scatter_v_contract(one):
    lib = L.lib()
    a, b = np.arange(4, dtype=np.float32), np.zeros(4, np.float32)
    counts, displs = np.array([4], np.uint64), np.array([0], np.uint64)
    assert lib.HcclReduceScatterV(a.ctypes.data, counts.ctypes.data, displs.ctypes.data, b.ctypes.data, 3, L.FP32, L.SUM,
                                  one.handle, None) == L.E_PARA  # recvCount != sendCounts[rank]
    assert lib.HcclReduceScatterV(a.ctypes.data, counts.ctypes.data, displs.ctypes.data, b.ctypes.data, 4, L.FP32, L.SUM,
                                  one.handle, None) == L.SUCCESS
    np.testing.assert_array_equal(a, b)


def test_comm_config_validation():
    lib = L.lib()
    h = C.c_void_p()
    bad = L.CommConfig()  # not initialised: magic word missing
    assert lib.HcclB200CommInitLocal(2, 0, 0, C.byref(bad), C.byref(h)) == L.E_PARA
    cfg = L.CommConfig.default()
    cfg.hcclDeterministic = 5
    assert lib.HcclB200CommInitLocal(2, 0, 0, C.byref(cfg), C.byref(h)) == L.E_PARA
    cfg = L.CommConfig.default()
    cfg.hcclOpExpansionMode = 9
    assert lib.HcclB200CommInitLocal(2, 0, 0, C.byref(cfg), C.byref(h)) == L.E_PARA
    cfg = L.CommConfig.default()
    cfg.hcclCommName = b"my_group"
    cfg.hcclBufferSize = 2
    assert lib.HcclB200CommInitLocal(2, 0, 0, C.byref(cfg), C.byref(h)) == L.SUCCESS
    c = H.Communicator(h.value, False)
    assert c.name() == "my_group"
    assert c.destroy() == L.SUCCESS
    assert lib.HcclB200CommInitLocal(0, 0, 0, None, C.byref(h)) == L.E_PARA
    assert lib.HcclB200CommInitLocal(99, 0, 0, None, C.byref(h)) == L.E_PARA
    assert lib.HcclGetCommConfigCapability() & 0xF == 0xF


def test_set_get_config_and_unknown_comm():
    lib = L.lib()
    v = C.c_int32(7)
    assert lib.HcclGetConfig(0, C.byref(v)) == L.SUCCESS and v.value in (0, 1)
    assert lib.HcclSetConfig(0, 3) == L.E_PARA
    assert lib.HcclSetConfig(5, 1) == L.E_NOT_SUPPORT
    assert lib.HcclSetConfig(0, 1) == L.SUCCESS
    assert lib.HcclGetConfig(0, C.byref(v)) == L.SUCCESS and v.value == 1
    assert lib.HcclSetConfig(0, 0) == L.SUCCESS
    bogus = C.c_void_p(0x1234)
    assert lib.HcclCommDestroy(bogus) == L.E_PARA
    a = np.zeros(2, np.float32)
    assert lib.HcclAllReduce(a.ctypes.data, a.ctypes.data, 2, L.FP32, L.SUM, bogus, None) == L.E_PARA


def test_memory_range_api(one):
    lib = L.lib()
    buf = np.zeros(1024, np.uint8)
    base = buf.ctypes.data
    assert lib.HcclCommSetMemoryRange(one.handle, base, 1024, 0, 0) == L.SUCCESS
    assert lib.HcclCommSetMemoryRange(one.handle, base + 10, 100, 0, 0) == L.E_PARA  # overlap
    assert lib.HcclCommActivateCommMemory(one.handle, base + 4096, 16, 0, None, 0) == L.E_PARA  # outside
    assert lib.HcclCommActivateCommMemory(one.handle, base, 512, 0, None, 0) == L.SUCCESS
    assert lib.HcclCommUnsetMemoryRange(one.handle, base) == L.E_PARA  # still active
    assert lib.HcclCommDeactivateCommMemory(one.handle, base) == L.SUCCESS
    assert lib.HcclCommUnsetMemoryRange(one.handle, base) == L.SUCCESS
    assert lib.HcclCommUnsetMemoryRange(one.handle, base) == L.E_NOT_FOUND


def test_deterministic_mode_is_bitwise_reproducible():
    cfg = L.CommConfig.default()
    cfg.hcclDeterministic = 1
    c = H.Communicator.init_local(5, device=False, config=cfg)
    ins = [np.random.default_rng(r).standard_normal(10001).astype(np.float32) for r in range(5)]
    outs1 = [np.zeros(10001, np.float32) for _ in range(5)]
    outs2 = [np.zeros(10001, np.float32) for _ in range(5)]
    c.all_reduce(ins, outs1)
    c.all_reduce(ins, outs2)
    for a, b in zip(outs1, outs2):
        assert a.tobytes() == b.tobytes()
    for o in outs1[1:]:
        assert o.tobytes() == outs1[0].tobytes()  # every rank reduces in the same fixed order
    c.destroy()


def test_selector_model():
    c = H.Communicator.init_local(8, device=False)
    small = c.select(L.ALLREDUCE, 256, L.FP32)
    big = c.select(L.ALLREDUCE, 64 << 20, L.FP32)
    assert small[0] == "mesh_oneshot" and small[1] == 1
    assert big[0] in ("mesh", "ring", "rhd") and big[2] > small[2]
    assert c.select(L.BROADCAST, 1 << 20, L.FP32)[0] in ("star", "tree", "ring")
    assert c.select(L.ALLTOALL, 1 << 20, L.FP32)[0] in ("mesh", "pairwise")
    # a slower flag hop pushes mid sizes towards fewer steps; a huge alpha makes one-shot win longer
    c.set_cost_model(alpha_us=50.0)
    assert c.select(L.ALLREDUCE, 64 << 10, L.FP32)[0] == "mesh_oneshot"
    c.destroy()


def test_hccl_algo_env_override_and_env_validation():
    code = """
import numpy as np, cann_hccl_b200 as H
from cann_hccl_b200 import _lib as L
c = H.Communicator.init_local(4, device=False)
print('SEL', c.select(L.ALLREDUCE, 1000, L.FP32)[0], c.select(L.ALLGATHER, 1000, L.FP32)[0], c.select(L.BROADCAST, 1000, L.FP32)[0])
ins=[np.ones(1000,np.float32) for _ in range(4)]; outs=[np.zeros(1000,np.float32) for _ in range(4)]
c.all_reduce(ins, outs); assert outs[0][0]==4
print('ALGOS', c.stats()['algos'])
"""
    env = dict(os.environ, HCCL_ALGO="allreduce=ring;allgather=rhd;broadcast=ring")
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, cwd=os.path.dirname(os.path.dirname(__file__)))
    assert "SEL ring rhd ring" in out.stdout, out.stdout + out.stderr
    assert "'ring': 1" in out.stdout
    env = dict(os.environ, HCCL_RDMA_TC="7")
    code2 = "import cann_hccl_b200 as H\nfrom cann_hccl_b200 import _lib as L\nimport ctypes as C\ni=L.RootInfo()\nprint('RC', L.lib().HcclGetRootInfo(C.byref(i)))"
    out = subprocess.run([sys.executable, "-c", code2], env=env, capture_output=True, text=True, cwd=os.path.dirname(os.path.dirname(__file__)))
    assert "RC 1" in out.stdout, out.stdout + out.stderr  # invalid HCCL_RDMA_TC is rejected like the reference does


def test_rank_table_init(tmp_path):
    table = {"version": "1.0", "status": "completed", "server_count": "1",
             "server_list": [{"server_id": "127.0.0.1", "host_ip": "127.0.0.1", "host_port": "0",
                              "device": [{"device_id": "0", "rank_id": "0"}]}]}
    path = tmp_path / "ranktable.json"
    table["server_list"][0]["host_port"] = str(61000 + os.getpid() % 2000)
    path.write_text(json.dumps(table))
    env_backup = os.environ.get("HCCL_TRANSPORT")
    os.environ["HCCL_TRANSPORT"] = "host"
    try:
        L.lib().HcclB200ReloadEnv()
        c = H.Communicator.init_cluster_info(str(path), 0, device=False)
        assert c.nranks == 1 and c.rank == 0
        c.destroy()
        bad = tmp_path / "bad.json"
        bad.write_text('{"server_list": [{"device": [{"device_id": "0", "rank_id": "3"}]}]}')
        h = C.c_void_p()
        assert L.lib().HcclCommInitClusterInfo(str(bad).encode(), 0, C.byref(h)) == L.E_PARA
        assert L.lib().HcclCommInitClusterInfo(b"/nonexistent/file.json", 0, C.byref(h)) == L.E_OPEN_FILE_FAILURE
    finally:
        if env_backup is None:
            del os.environ["HCCL_TRANSPORT"]
        else:
            os.environ["HCCL_TRANSPORT"] = env_backup
        L.lib().HcclB200ReloadEnv()


def test_comm_init_all_threads_host():
    code = """
import ctypes as C, numpy as np, threading
import cann_hccl_b200 as H
from cann_hccl_b200 import _lib as L
n=3
devs=(C.c_int32*n)(0,1,2); comms=(C.c_void_p*n)()
L.check(L.lib().HcclCommInitAll(n, devs, comms), 'HcclCommInitAll')
cs=[H.Communicator(comms[i], False) for i in range(n)]
assert [c.rank for c in cs]==[0,1,2]
outs=[np.zeros(10,np.float32) for _ in range(n)]
def run(i):
    cs[i].all_reduce(np.full(10,i+1,np.float32), outs[i])
ts=[threading.Thread(target=run,args=(i,)) for i in range(n)]
[t.start() for t in ts]; [t.join() for t in ts]
assert all((o==6).all() for o in outs), outs
ts=[threading.Thread(target=lambda c=c: c.destroy()) for c in cs]
[t.start() for t in ts]; [t.join() for t in ts]
print('INITALL OK')
"""
    env = dict(os.environ, HCCL_TRANSPORT="host")
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, cwd=os.path.dirname(os.path.dirname(__file__)), timeout=60)
    assert "INITALL OK" in out.stdout, out.stdout + out.stderr


def test_plan_verifier_accepts_schedules_and_catches_a_skewed_step():
    """Every plan passes a static bounds check before its first run; a destination offset pushed past the staging area
    (or the caller's buffer) is reported with the step, at plan build time."""
    lib = L.lib()
    msg = C.create_string_buffer(512)
    n = 100_003
    for coll, algos in ((L.ALLREDUCE, (L.ALGO_MESH, L.ALGO_RING, L.ALGO_RHD, L.ALGO_MESH_ONESHOT)), (L.ALLGATHER, (L.ALGO_MESH, L.ALGO_RING)),
                        (L.REDUCE_SCATTER, (L.ALGO_MESH, L.ALGO_RING, L.ALGO_RHD)), (L.BROADCAST, (L.ALGO_STAR, L.ALGO_RING, L.ALGO_TREE))):
        for algo in algos:
            for p in (2, 3, 5, 8):
                rc = lib.HcclB200PlanCheck(coll, algo, p, n, L.FP32, 4, 64 << 20, -1, 0, msg, 512)
                assert rc == L.SUCCESS, msg.value
    # staging half too small for the declared need
    assert lib.HcclB200PlanCheck(L.ALLREDUCE, L.ALGO_MESH, 4, n, L.FP32, 4, 4096, -1, 0, msg, 512) == L.E_INTERNAL
    assert b"staging" in msg.value
    # a step whose destination runs 1 GiB past its buffer
    bad = 0
    for step in range(6):
        rc = lib.HcclB200PlanCheck(L.ALLREDUCE, L.ALGO_RING, 4, n, L.FP32, 4, 64 << 20, step, 1 << 30, msg, 512)
        if rc == L.E_INTERNAL:
            bad += 1
            assert b"step %d" % step in msg.value and b"reaches byte" in msg.value, msg.value
    assert bad >= 4


def test_headers_compile_as_c99_and_library_runs_from_c(tmp_path):
    """The public headers are C: a C99 program (-pedantic -Werror) includes hccl.h, hccl_b200.h and hcom.h, links the shared
    library and runs collectives on four CPU ranks."""
    import shutil
    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    pkg = os.path.join(root, "cann_hccl_b200")
    L.lib()  # builds the library when missing
    exe = str(tmp_path / "c_consumer")
    cmd = ["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I" + os.path.join(pkg, "include"),
           os.path.join(root, "tests", "c_api", "hccl_c_consumer.c"), "-o", exe, "-L" + os.path.join(pkg, "lib"), "-lhccl_b200",
           "-Wl,-rpath," + os.path.join(pkg, "lib")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    env = dict(os.environ, HCCL_TRANSPORT="host")
    r = subprocess.run([exe], capture_output=True, text=True, env=env, timeout=120)
    assert r.returncode == 0 and "c consumer ok" in r.stdout, r.stdout + r.stderr


def test_plan_verifier_property_sweep():
    """Random (collective, algorithm, ranks, count, dtype, channels): every schedule the generators emit stays inside its
    buffers (hypothesis drives the static verifier; no communicator involved)."""
    hyp = pytest.importorskip("hypothesis")
    from hypothesis import given, settings, strategies as st
    lib = L.lib()
    table = {
        L.ALLREDUCE: [L.ALGO_MESH, L.ALGO_MESH_ONESHOT, L.ALGO_RING, L.ALGO_RHD],
        L.ALLGATHER: [L.ALGO_MESH, L.ALGO_RING, L.ALGO_RHD, L.ALGO_PAIRWISE],
        L.REDUCE_SCATTER: [L.ALGO_MESH, L.ALGO_RING, L.ALGO_RHD],
        L.BROADCAST: [L.ALGO_STAR, L.ALGO_RING, L.ALGO_TREE],
        L.REDUCE: [L.ALGO_STAR, L.ALGO_RING, L.ALGO_TREE, L.ALGO_RHD],
        L.SCATTER: [L.ALGO_STAR, L.ALGO_RING],
        L.GATHER: [L.ALGO_STAR, L.ALGO_RING],
        L.ALLTOALL: [L.ALGO_MESH, L.ALGO_PAIRWISE],
    }
    pairs = [(c, a) for c, algos in table.items() for a in algos]
    msg = C.create_string_buffer(512)

    @settings(max_examples=400, deadline=None)
    @given(st.sampled_from(pairs), st.integers(2, 16), st.integers(1, 200_000), st.sampled_from([L.INT8, L.FP16, L.FP32, L.FP64]),
           st.integers(1, 16))
    def run(pair, p, count, dtype, nchan):
        coll, algo = pair
        rc = lib.HcclB200PlanCheck(coll, algo, p, count, dtype, nchan, 1 << 30, -1, 0, msg, 512)
        assert rc == L.SUCCESS, (coll, L.ALGO_NAMES[algo], p, count, dtype, nchan, msg.value)

    run()


def test_library_override_and_sanitizer_build_names(tmp_path):
    """HCCL_B200_LIB makes the Python layer load another build of the library (a sanitizer build, for one); the build script
    names those builds after the sanitizer and refuses anything but address and thread."""
    import subprocess
    import sys
    from cann_hccl_b200 import build as B
    assert B.lib_path().endswith("libhccl_b200.so")
    assert B.lib_path("thread").endswith("libhccl_b200_thread.so")
    with pytest.raises(ValueError):
        B.build(sanitize="memory")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    alias = tmp_path / "libhccl_b200_copy.so"
    os.symlink(B.lib_path(), alias)
    code = "import cann_hccl_b200._lib as L; L.lib(); print(L.LIB_PATH)"
    out = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, HCCL_B200_LIB=str(alias)), cwd=root, capture_output=True, text=True, timeout=120)
    assert out.stdout.strip().endswith("libhccl_b200_copy.so"), out.stdout + out.stderr


def test_hccl_test_alltoallv_count_matrix_is_consistent():
    from cann_hccl_b200.utils import hccl_test as T
    for p in (2, 3, 8):
        m = T.a2av_matrix(1000, p)
        sc, sd, rc, rd = T.a2av_rows(m, range(p))
        assert (sc == m).all() and (rc == m.T).all() and (m >= 1).all()
        for r in range(p):
            assert sd[r][0] == 0 and rd[r][0] == 0
            assert all(sd[r][j + 1] == sd[r][j] + sc[r][j] for j in range(p - 1))
            assert all(rd[r][j + 1] == rd[r][j] + rc[r][j] for j in range(p - 1))
