"""ucclCommInitAll: one process creates a communicator per rank (one thread each inside the library)
and drives them from one Python thread per rank (reference: src/init.cc ucclCommInitAll)."""
import os
import subprocess
import sys
import textwrap

from mp_util import ROOT

SCRIPT = textwrap.dedent("""
    import os, sys, threading
    sys.path.insert(0, %r)
    import torch
    from unified_ccl_b200 import _C

    n = 3
    comms = _C.comm_init_all(n, [])
    assert len(comms) == n and all(comms)
    assert [_C.comm_rank(c) for c in comms] == list(range(n))
    assert all(_C.comm_count(c) == n for c in comms)
    bufs = [torch.full((4096,), float(i + 1)) for i in range(n)]
    errs = []

    def work(i):
        try:
            _C.allreduce(comms[i], bufs[i].data_ptr(), bufs[i].data_ptr(), bufs[i].numel(), 2, 0)
        except Exception as e:  # noqa: BLE001
            errs.append(repr(e))

    th = [threading.Thread(target=work, args=(i,)) for i in range(n)]
    [t.start() for t in th]
    [t.join(60) for t in th]
    assert not errs, errs
    assert all(not t.is_alive() for t in th)
    assert all(torch.equal(b, torch.full((4096,), 6.0)) for b in bufs)
    for c in comms:
        _C.comm_destroy(c)
    print("init_all ok")
""") % ROOT


def test_comm_init_all_cpu_ranks():
    env = dict(os.environ, UCCL_BACKEND="cpu", UCCL_BOOTSTRAP_IFNAME="lo")
    p = subprocess.run([sys.executable, "-c", SCRIPT], env=env, capture_output=True, text=True, timeout=120)
    assert p.returncode == 0 and "init_all ok" in p.stdout, p.stdout[-2000:] + p.stderr[-2000:]
