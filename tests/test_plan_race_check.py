"""Static race detection over every lowered plan (algo/racecheck.cc).

On GPUs every channel of every rank is a CTA of its own; the CPU executor runs a rank's channels one after the other and so
never shows a missing dependency between them.  The checker builds the happens-before relation of a plan (program order per
rank and channel, flag signal -> wait) and demands that conflicting accesses are ordered by it."""
import ctypes as C

import pytest

from cann_hccl_b200 import _lib as L

COLLS = {"allreduce": L.ALLREDUCE, "allgather": L.ALLGATHER, "reducescatter": L.REDUCE_SCATTER, "broadcast": L.BROADCAST,
         "reduce": L.REDUCE, "scatter": L.SCATTER, "gather": L.GATHER, "alltoall": L.ALLTOALL}
ROOTED = ("broadcast", "reduce", "scatter", "gather")


def race_check(coll, algo, p, n, nchan, root=0, in_place=0, drop=(-1, -1)):
    msg = C.create_string_buffer(1024)
    rc = L.lib().HcclB200PlanRaceCheck(coll, algo, p, n, L.FP32, nchan, root, in_place, drop[0], drop[1], msg, 1024)
    return rc, msg.value.decode()


@pytest.mark.parametrize("name", sorted(COLLS))
def test_every_plan_orders_its_conflicting_accesses(name):
    """Every (algorithm, rank count, channel count, size, root, in-place form) of the collective: no unordered conflicting
    accesses, no wait without a sender, no cycle of waits."""
    checked = 0
    for algo in range(len(L.ALGO_NAMES)):
        for p in (2, 3, 4, 5, 6, 8):
            for nchan in (1, 2, 3, 5):
                for n in (7, 100_003):
                    for in_place in (0, 1):
                        for root in ((0, p - 1) if name in ROOTED else (0,)):
                            rc, msg = race_check(COLLS[name], algo, p, n, nchan, root, in_place)
                            if rc == L.E_NOT_SUPPORT:
                                continue
                            checked += 1
                            assert rc == L.SUCCESS, "%s p=%d nchan=%d n=%d root=%d in_place=%d: %s" % (L.ALGO_NAMES[algo], p, nchan, n, root, in_place, msg)
    assert checked > 50


@pytest.mark.parametrize("name,coll", [("allgatherv", L.ALLGATHER_V), ("reducescatterv", L.REDUCE_SCATTER_V), ("alltoallv", L.ALLTOALLV),
                                       ("alltoallvc", L.ALLTOALLVC)])
def test_variable_count_plans_order_their_conflicting_accesses(name, coll):
    """Non-uniform layouts (one rank may contribute nothing); AlltoAllV with slots of a third of the largest block, i.e. several
    rounds per ordered pair whose slot reuse hangs on the acknowledgement flags."""
    checked = 0
    for algo in range(len(L.ALGO_NAMES)):
        for p in (2, 3, 4, 5, 8):
            for nchan in (1, 2, 3):
                for n in (5, 7, 1000, 100_003):
                    rc, msg = race_check(coll, algo, p, n, nchan)
                    if rc == L.E_NOT_SUPPORT:
                        continue
                    checked += 1
                    assert rc == L.SUCCESS, "%s p=%d nchan=%d n=%d: %s" % (L.ALGO_NAMES[algo], p, nchan, n, msg)
    assert checked > 50


def test_checker_finds_a_dropped_acknowledgement_wait():
    """AlltoAllV: a sender that does not wait for the acknowledgement of round k - 1 overwrites a slot that is still being read."""
    assert race_check(L.ALLTOALLV, L.ALGO_PAIRWISE, 3, 100_003, 2)[0] == L.SUCCESS
    hits = [race_check(L.ALLTOALLV, L.ALGO_PAIRWISE, 3, 100_003, 2, drop=(0, s)) for s in range(1, 14)]
    assert any(rc == L.E_INTERNAL and "staging" in m for rc, m in hits), hits


def test_checker_finds_a_dropped_wait():
    """Take the wait out of a step that needs it: the checker names the two accesses that are no longer ordered."""
    found = 0
    for coll, algo, p in ((L.ALLREDUCE, L.ALGO_MESH, 4), (L.ALLREDUCE, L.ALGO_RING, 3), (L.ALLGATHER, L.ALGO_RING, 4), (L.ALLREDUCE, L.ALGO_RHD, 4)):
        assert race_check(coll, algo, p, 100_003, 3)[0] == L.SUCCESS
        for step in range(1, 12):
            rc, msg = race_check(coll, algo, p, 100_003, 3, drop=(1, step))
            if rc == L.E_PARA:      # that step has no wait (or the plan is shorter)
                continue
            if rc == L.SUCCESS:     # a wait that other waits of the plan already imply
                continue
            assert rc == L.E_INTERNAL and "unordered" in msg, (L.ALGO_NAMES[algo], step, rc, msg)
            found += 1
    assert found >= 6


def test_checker_reports_halving_steps_without_a_meeting_point():
    """The case that made the check worth writing: recursive halving reduces into ranges that shrink from step to step, so
    the lane of a channel in one step overlaps other channels' lanes of the step before.  Without the meeting point of a rank's
    channels between two halving steps (drop its wait) the accesses to the rank's own staging are unordered."""
    rc, msg = race_check(L.ALLREDUCE, L.ALGO_RHD, 4, 100_003, 3)
    assert rc == L.SUCCESS, msg
    hits = [race_check(L.ALLREDUCE, L.ALGO_RHD, 4, 100_003, 3, drop=(0, s)) for s in range(2, 10)]
    assert any(rc == L.E_INTERNAL and "staging of rank 0" in m and "rank 0 step" in m for rc, m in hits), hits


def test_runtime_knob_checks_every_plan_when_it_is_built():
    """HCCL_PLAN_RACE_CHECK=1: the communicator runs the check (out of place and in place) on every plan it builds."""
    import os
    import subprocess
    import sys
    code = """
import numpy as np
import cann_hccl_b200 as H
from cann_hccl_b200 import _lib as L
p = 4
c = H.Communicator.init_local(p, device=False)
ins = [np.arange(1000, dtype=np.float32) + r for r in range(p)]
for algo in (L.ALGO_MESH, L.ALGO_RING, L.ALGO_RHD, L.ALGO_MESH_ONESHOT):
    outs = [np.zeros(1000, np.float32) for _ in range(p)]
    c.all_reduce(ins, outs, algo=algo)
    assert all(np.allclose(o, sum(ins)) for o in outs)
outs = [np.zeros(250, np.float32) for _ in range(p)]
c.reduce_scatter(ins, outs, algo=L.ALGO_RHD)
assert all(np.allclose(outs[r], sum(ins)[r * 250:(r + 1) * 250]) for r in range(p))
print('RACE CHECK KNOB OK', c.stats()['plans_built'])
c.destroy()
"""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, HCCL_PLAN_RACE_CHECK="1", HCCL_TRANSPORT="host")
    out = subprocess.run([sys.executable, "-c", code], env=env, cwd=root, capture_output=True, text=True, timeout=120)
    assert "RACE CHECK KNOB OK" in out.stdout, out.stdout + out.stderr
