"""tcgen05 GEMM vs an fp32 PyTorch reference of the same op."""
import pytest
import torch

gpu = pytest.mark.gpu


def _run(M, N, K, epilogue=0, seed=0):
    from unified_ccl_b200.ops import gemm_bf16

    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn(M, K, device="cuda", dtype=torch.float32, generator=g).to(torch.bfloat16)
    b = (torch.randn(N, K, device="cuda", dtype=torch.float32, generator=g) * 0.05).to(torch.bfloat16)
    out = gemm_bf16(a, b, swiglu=bool(epilogue))
    torch.cuda.synchronize()
    ref = a.float() @ b.float().t()
    if epilogue:
        gate, up = ref[:, : N // 2], ref[:, N // 2:]
        ref = torch.nn.functional.silu(gate) * up
    return out.float(), ref


@gpu
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (1024, 1024, 1024), (4096, 3584, 4096)])
def test_gemm_plain(M, N, K):
    out, ref = _run(M, N, K)
    err = (out - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 2e-2 * scale + 1e-2, (err, scale)


@gpu
@pytest.mark.parametrize("M,N,K", [(200, 264, 72), (130, 40, 136), (1, 8, 8)])
def test_gemm_ragged(M, N, K):
    out, ref = _run(M, N, K)
    err = (out - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 2e-2 * scale + 1e-2, (err, scale)


@gpu
@pytest.mark.parametrize("M,N,K", [(256, 512, 128), (1024, 3584, 1024), (300, 272, 64)])
def test_gemm_swiglu(M, N, K):
    out, ref = _run(M, N, K, epilogue=1)
    err = (out - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 2e-2 * scale + 1e-2, (err, scale)
