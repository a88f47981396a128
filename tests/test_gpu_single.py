"""Single-GPU tests: API contract on CUDA tensors, symmetric allocation, fused norm with one rank."""
import pytest
import torch

from mp_util import assert_all_ok, run_ranks

gpu = pytest.mark.gpu


@gpu
def test_api_contract_cuda():
    assert_all_ok(run_ranks("api_contract", 1))


@gpu
def test_single_rank_collectives_cuda():
    assert_all_ok(run_ranks("collectives_small", 1))


@gpu
def test_fused_norm_single_rank():
    assert_all_ok(run_ranks("fused_norm", 1))


@gpu
def test_tp_mlp_single_rank():
    assert_all_ok(run_ranks("tp_mlp", 1))


@gpu
def test_moe_single_rank():
    assert_all_ok(run_ranks("moe", 1))


@gpu
def test_canaries_around_symmetric_buffers():
    assert_all_ok(run_ranks("canary", 1, env={"UCCL_CANARY": "1"}))


@gpu
def test_native_library_is_loaded():
    """The CUDA path must come from this repository's shared objects, not from a fallback."""
    import unified_ccl_b200 as u

    loaded = [line.split()[-1] for line in open("/proc/self/maps") if "libuccl.so" in line or "_uccl_bindings" in line]
    assert any("libuccl.so" in p for p in loaded) and any("_uccl_bindings" in p for p in loaded)
    a = torch.randn(256, 128, device="cuda").to(torch.bfloat16)
    b = torch.randn(512, 128, device="cuda").to(torch.bfloat16)
    out = u.ops.gemm_bf16(a, b)
    torch.cuda.synchronize()
    assert torch.allclose(out.float(), a.float() @ b.float().t(), atol=0.5, rtol=2e-2)
