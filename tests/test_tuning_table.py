"""The measured tuner table shipped with the package parses and drives the tuner."""
import json
import os
import subprocess
import sys
import textwrap

from mp_util import ROOT

SCRIPT = textwrap.dedent("""
    import sys
    sys.path.insert(0, %r)
    import unified_ccl_b200 as u
    c = u.Communicator(0, 1)
    c.load_tuning(u.tuning_table())
    algo, proto, blocks = c.query_tuning("allreduce", 1 << 20, True)
    assert algo in ("ring", "net", "one_shot", "two_shot", "nvls", "copy_engine"), algo
    try:
        c.load_tuning("/nonexistent/table.json")
        raise SystemExit("a missing table was accepted")
    except u._C.UcclError:
        pass
    c.destroy()
    print("table ok")
""") % ROOT


def test_shipped_table_is_well_formed():
    import unified_ccl_b200 as u

    doc = json.load(open(u.tuning_table()))
    assert doc["version"] == 1 and doc["nranks"] == 8
    colls = {e["coll"] for e in doc["entries"]}
    assert {"allreduce", "allgather", "reducescatter"} <= colls
    for e in doc["entries"]:
        assert e["us"] > 0 and e["bytes"] > 0 and e["blocks"] >= 0


def test_shipped_table_loads():
    env = dict(os.environ, UCCL_BACKEND="cpu", UCCL_BOOTSTRAP_IFNAME="lo")
    p = subprocess.run([sys.executable, "-c", SCRIPT], env=env, capture_output=True, text=True, timeout=120)
    assert p.returncode == 0 and "table ok" in p.stdout, p.stdout[-2000:] + p.stderr[-2000:]
