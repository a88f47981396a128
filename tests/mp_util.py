"""Run a test case as N rank processes and collect one JSON result per rank."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_ranks(case, nranks, env=None, timeout=180, per_rank_env=None, expect_exit=None, args=()):
    """Start `nranks` interpreters running tests/rank_worker.py <case>.

    Rank 0 creates the unique id inside its own process and publishes it through a file, so the
    rendezvous service lives in a rank process exactly as it does in real jobs.
    Returns a list of dicts (one per rank, in rank order); a rank that died yields
    {"rank": r, "died": returncode, "stderr": ...}.
    """
    import tempfile

    base_env = dict(os.environ)
    base_env.setdefault("UCCL_BOOTSTRAP_IFNAME", "lo")
    base_env["PYTHONPATH"] = ROOT + os.pathsep + base_env.get("PYTHONPATH", "")
    if env:
        base_env.update(env)
    tmp = tempfile.mkdtemp(prefix="uccl_test_")
    idfile = os.path.join(tmp, "uid")
    procs = []
    for r in range(nranks):
        e = dict(base_env)
        if per_rank_env and r in per_rank_env:
            e.update(per_rank_env[r])
        cmd = [sys.executable, os.path.join(ROOT, "tests", "rank_worker.py"), case, str(r), str(nranks), idfile] + [str(a) for a in args]
        procs.append(subprocess.Popen(cmd, env=e, stdout=subprocess.PIPE, stderr=subprocess.PIPE, cwd=ROOT))
    out = []
    for r, p in enumerate(procs):
        try:
            so, se = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            so, se = p.communicate()
            out.append({"rank": r, "died": "timeout", "stderr": se.decode(errors="replace")[-2000:]})
            continue
        res = None
        for line in so.decode(errors="replace").splitlines():
            if line.startswith("RESULT "):
                res = json.loads(line[7:])
        if res is None:
            res = {"rank": r, "died": p.returncode, "stderr": se.decode(errors="replace")[-2000:]}
        else:
            res["returncode"] = p.returncode
        out.append(res)
    return out


def assert_all_ok(results):
    for r in results:
        assert "died" not in r, r
        assert not r.get("fail"), r
        assert "exc" not in r, r["exc"]
