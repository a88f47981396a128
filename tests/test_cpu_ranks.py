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
