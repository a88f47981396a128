"""Multi-GPU tests: one process per GPU over NVLink.  Need >= 2 devices."""
import pytest
import torch

from mp_util import assert_all_ok, run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _n():
    n = torch.cuda.device_count()
    return 8 if n >= 8 else (4 if n >= 4 else 2)


def test_allreduce_config1_on_gpus():
    res = run_ranks("allreduce_config1", 2)
    assert_all_ok(res)


def test_collective_matrix():
    assert_all_ok(run_ranks("collectives_small", _n(), timeout=300))


def test_collective_matrix_symmetric_buffers():
    assert_all_ok(run_ranks("collectives_symmetric", _n(), timeout=300))


def test_canaries_stay_intact_under_collectives():
    assert_all_ok(run_ranks("canary", _n(), env={"UCCL_CANARY": "1"}, timeout=200))


def test_allreduce_every_algorithm():
    res = run_ranks("allreduce_algos", _n(), timeout=400)
    assert_all_ok(res)
    hist = res[0]["algo_hist"]
    # ring, one-shot, two-shot and copy-engine all ran (NVLS only where the fabric has it)
    assert hist[1] > 0 and hist[2] > 0 and hist[3] > 0 and hist[5] > 0
    if res[0]["nvls"]:
        assert hist[4] > 0


def test_ring_and_copy_engine_allgather_reduce_scatter():
    """Ring (Simple, LL128) and copy-engine all-gather / reduce-scatter / all-reduce with a staging area so
    small that a chunk needs more pieces than a channel has slots."""
    env = {"UCCL_STAGING_BYTES": "1M", "UCCL_MAX_CTAS": "2", "UCCL_WAIT_TIMEOUT_MS": "5000"}
    res = run_ranks("ring_ce_matrix", _n(), env=env, timeout=300)
    assert_all_ok(res)
    assert res[0]["algo_hist"][1] > 0 and res[0]["algo_hist"][5] > 0


def test_hybrid_exec_mode():
    """UCCL_EXEC_MODE=hybrid: SM kernels below 1 MiB, copy engines from there up."""
    res = run_ranks("collectives_symmetric", _n(), env={"UCCL_EXEC_MODE": "hybrid"}, timeout=300)
    assert_all_ok(res)


def test_cuda_ipc_heap():
    """UCCL_P2P=ipc: the symmetric heap from cudaMalloc + cudaIpc handles (no multicast) instead of VMM."""
    res = run_ranks("collectives_symmetric", 2, env={"UCCL_P2P": "ipc"}, timeout=300)
    assert_all_ok(res)
    assert not res[0]["nvls"]


def test_collectives_with_scale_and_cast():
    """ucclReduceScatterEx / ucclAllReduceEx: sum, scale, other output type (fp32 / bf16 / fp16 / fp8 + scales)."""
    env = {"UCCL_STAGING_BYTES": "4M"}
    assert_all_ok(run_ranks("fused_cast", _n(), env=env, timeout=300))


def test_sendrecv():
    assert_all_ok(run_ranks("sendrecv", _n()))


def test_rma_put_get_signal():
    assert_all_ok(run_ranks("rma", _n()))


def test_rma_device_api():
    """devicePutSignal / deviceWaitSignal* / deviceGetReduce<T> ... called from kernels, 2 or more GPUs."""
    assert_all_ok(run_ranks("rma_device", min(_n(), 4), env={"UCCL_WAIT_TIMEOUT_MS": "800"}))


def test_fused_allreduce_residual_rmsnorm():
    assert_all_ok(run_ranks("fused_norm", _n()))


# all-gather transport / reducer CTAs of the reduce-scatter; each pair runs as rank processes of its own,
# so that one pair's failure or time limit says which pair it was and leaves the others their verdict
@pytest.mark.parametrize("modes", ["ce/0", "kernel/0", "spread/0", "ce/8", "spread/16"])
def test_tensor_parallel_mlp(modes):
    assert_all_ok(run_ranks("tp_mlp", _n(), timeout=120, args=[modes],
                            env={"UCCL_WAIT_TIMEOUT_MS": "5000", "UCCL_TEST_DUMP_AFTER_S": "100"}))


def test_moe_dispatch_combine():
    assert_all_ok(run_ranks("moe", _n(), timeout=300))


def test_network_path_on_gpus():
    """UCCL_FORCE_NET=1: persistent ring kernel <-> mapped FIFO <-> proxy <-> socket plugin."""
    res = run_ranks("collectives_small", 2, env={"UCCL_FORCE_NET": "1"}, timeout=300)
    assert_all_ok(res)
    assert res[0]["algo_hist"][6] > 0


def test_skipped_collective_reports_timeout():
    env = {"UCCL_WAIT_TIMEOUT_MS": "800", "UCCL_NVLS": "0"}
    res = run_ranks("skipped_collective", 2, env=env, timeout=120)
    for r in res:
        assert "died" not in r and not r["fail"], r
    assert res[0]["timeouts"] >= 1 and res[0]["seconds"] < 30
    assert "wait expired" in res[0]["last"] or "remote" in (res[0]["err"] or "").lower()


def test_rank_that_exits_between_steps():
    env = {"UCCL_WAIT_TIMEOUT_MS": "800", "UCCL_NVLS": "0"}
    res = run_ranks("peer_exits", 2, env=env, timeout=120)
    assert "died" not in res[0] and not res[0]["fail"], res[0]
    assert res[0]["seconds"] < 30
