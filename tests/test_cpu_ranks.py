"""CPU-rank integration: real processes, real bootstrap, proxy thread, FIFOs and network plugin."""
import os

import pytest

from mp_util import ROOT, assert_all_ok, run_ranks

CPU = {"UCCL_BACKEND": "cpu"}


def test_allreduce_config1_two_processes():
    """fp32 all-reduce of 1,048,576 elements between 2 host processes, seeds 1234 + r, exact."""
    res = run_ranks("allreduce_config1", 2, env=CPU)
    assert_all_ok(res)
    for r in res:
        assert r["err"] == 0.0
        assert r["proxy_posts"] > 0 and r["net"] == "Socket"


@pytest.mark.parametrize("n", [2, 3, 4])
def test_collective_matrix(n):
    assert_all_ok(run_ranks("collectives_small", n, env=CPU))


def test_sendrecv_groups():
    assert_all_ok(run_ranks("sendrecv", 4, env=CPU))


def test_api_contract_single_rank():
    assert_all_ok(run_ranks("api_contract", 1, env=CPU))


def test_api_contract_two_ranks():
    assert_all_ok(run_ranks("api_contract", 2, env=CPU))


def test_external_plugin_carries_the_ring():
    plugin = os.path.join(ROOT, "plugins", "sample", "libuccl-net-sample.so")
    assert os.path.exists(plugin), "build the sample plugin with `make`"
    env = dict(CPU, UCCL_NET_PLUGIN=plugin)
    res = run_ranks("allreduce_config1", 2, env=env)
    assert_all_ok(res)
    assert all(r["net"] == "UnixSample" for r in res)


def test_ucx_plugin_over_the_stand_in():
    """plugins/ucx/plugin.cc (listener queue, client / server endpoints, tagged posts, polling, forced
    close) built against the in-tree stand-in of the UCP calls it uses: the collective matrix and the
    config-1 all-reduce travel through it between host processes."""
    plugin = os.path.join(ROOT, "plugins", "ucx", "libuccl-net-ucx-fake.so")
    assert os.path.exists(plugin), "build it with `make` (or `make ucx-fake`)"
    env = dict(CPU, UCCL_NET_PLUGIN=plugin, UCCL_SOCKET_IFNAME="lo")
    res = run_ranks("allreduce_config1", 2, env=env)
    assert_all_ok(res)
    assert all(r["net"] == "UCX" and r["err"] == 0.0 for r in res)
    assert_all_ok(run_ranks("collectives_small", 3, env=env))
    assert_all_ok(run_ranks("sendrecv", 4, env=env))


def test_ucx_plugin_without_ucx_reports_it(tmp_path):
    """Built without UCCL_HAS_UCX the plugin loads, and its init() says what is missing."""
    import ctypes
    import subprocess

    so = tmp_path / "libuccl-net-ucx-none.so"
    subprocess.run(["g++", "-std=c++17", "-fPIC", "-shared", "-I" + os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "plugins", "ucx", "plugin.cc"), "-o", str(so)], check=True)
    lib = ctypes.CDLL(str(so))
    assert hasattr(lib, "ucclNetPlugin_v1")
    table = (ctypes.c_void_p * 18).in_dll(lib, "ucclNetPlugin_v1")
    assert b"not compiled in" in ctypes.cast(table[0], ctypes.c_char_p).value
    init = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(ctypes.c_void_p))(table[1])
    handle = ctypes.c_void_p()
    assert init(ctypes.byref(handle)) == 4  # ucclInvalidUsage


def test_c_abi_client_processes():
    """A C++ program drives ucclCommInitRank / ucclAllReduce / group(all-gather + reduce-scatter)
    across three processes (the reference's tests/cpp/test_allreduce.cc, which needs mpirun)."""
    import subprocess
    import tempfile

    exe = os.path.join(ROOT, "tests", "native", "c_api_client")
    idfile = os.path.join(tempfile.mkdtemp(prefix="uccl_capi_"), "uid")
    env = dict(os.environ, UCCL_BACKEND="cpu", UCCL_BOOTSTRAP_IFNAME="lo")
    procs = [subprocess.Popen([exe, "rank", str(r), "3", idfile], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE)
             for r in range(3)]
    for r, p in enumerate(procs):
        out, err = p.communicate(timeout=120)
        assert p.returncode == 0 and b"ok" in out, (r, out[-500:], err[-1500:])


def test_c_abi_client_init_all():
    import subprocess

    exe = os.path.join(ROOT, "tests", "native", "c_api_client")
    env = dict(os.environ, UCCL_BACKEND="cpu", UCCL_BOOTSTRAP_IFNAME="lo")
    p = subprocess.run([exe, "initall", "3"], env=env, capture_output=True, timeout=120)
    assert p.returncode == 0 and p.stdout.count(b"ok") == 3, (p.stdout[-500:], p.stderr[-1500:])


def test_small_slots_and_one_channel():
    """Many sub-chunks per step and FIFO wrap-around."""
    env = dict(CPU, UCCL_NET_CHUNK_BYTES="4096", UCCL_NCHANNELS="1")
    assert_all_ok(run_ranks("collectives_small", 3, env=env))


def test_rank_that_never_joins_times_out():
    env = dict(CPU, UCCL_BOOTSTRAP_TIMEOUT_MS="1500")
    res = run_ranks("never_joins", 3, env=env, timeout=60)
    for r in res[:-1]:
        assert "died" not in r and not r["fail"], r
        assert r["seconds"] < 30
        assert "remote" in r["err"].lower() or "timed out" in r["err"].lower() or "rendezvous" in r["err"].lower()
    assert res[-1].get("absent")


def test_rank_that_exits_between_steps():
    env = dict(CPU, UCCL_WAIT_TIMEOUT_MS="1500")
    res = run_ranks("peer_exits", 3, env=env, timeout=90)
    for r in res[:-1]:
        assert "died" not in r and not r["fail"], r
        assert r["seconds"] < 30
    assert res[-1]["left"]


@pytest.mark.parametrize("jitter_us", [50, 400])
def test_collective_matrix_with_schedule_perturbation(jitter_us):
    """Random pauses between the steps of the proxy threads and of the host transfer loops: the
    results must not depend on the interleaving (UCCL_JITTER_US)."""
    env = dict(CPU, UCCL_JITTER_US=str(jitter_us))
    assert_all_ok(run_ranks("collectives_small", 3, env=env, timeout=300))
    assert_all_ok(run_ranks("sendrecv", 4, env=env, timeout=300))
