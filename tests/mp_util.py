"""Launch N CPU ranks (one process each, host-memory transport) that rendezvous through a root-info file."""
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))


def run_ranks(nranks, scenario, env=None, timeout=90, expect_fail_ranks=(), args=()):
    """Runs tests/_worker.py <scenario> on `nranks` processes; returns list of (returncode, stdout+stderr)."""
    tmp = tempfile.mkdtemp(prefix="hcclb_")
    root_file = os.path.join(tmp, "root.bin")
    procs = []
    for r in range(nranks):
        e = dict(os.environ)
        e["HCCL_TRANSPORT"] = "host"
        e.setdefault("HCCL_EXEC_TIMEOUT_MS", "20000")
        e["HCCL_CONNECT_TIMEOUT"] = "30"
        if env:
            e.update(env)
        cmd = [sys.executable, os.path.join(HERE, "_worker.py"), scenario, str(nranks), str(r), root_file] + [str(a) for a in args]
        procs.append(subprocess.Popen(cmd, env=e, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, errors="replace"))
    results = []
    for r, p in enumerate(procs):
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[killed by test timeout]"
        results.append((p.returncode, out))
    for r, (code, out) in enumerate(results):
        if r in expect_fail_ranks:
            continue
        assert code == 0, "rank %d failed (%s):\n%s" % (r, code, out)
    return results
