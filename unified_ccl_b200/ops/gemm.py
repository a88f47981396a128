"""bf16 GEMM on tcgen05 tensor cores (TMEM accumulators, TMA-fed)."""
import torch

from .. import _C


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor = None, swiglu: bool = False) -> torch.Tensor:
    """``out = a @ b.T`` with ``a`` [M, K] and ``b`` [N, K] bf16 CUDA tensors (last dim contiguous).

    With ``swiglu=True`` the rows of ``b`` are ``[gate (N/2); up (N/2)]`` and the result is
    ``silu(a @ gate.T) * (a @ up.T)`` of shape [M, N/2], computed in the GEMM epilogue.
    """
    if not (a.is_cuda and b.is_cuda):
        raise ValueError("gemm_bf16 needs CUDA tensors")
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("gemm_bf16 needs bf16 inputs")
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1]:
        raise ValueError("shape mismatch: a [M,K], b [N,K]")
    if a.stride(1) != 1 or b.stride(1) != 1:
        raise ValueError("innermost dimension must be contiguous")
    M, K = a.shape
    N = b.shape[0]
    n_out = N // 2 if swiglu else N
    if out is None:
        out = torch.empty(M, n_out, device=a.device, dtype=torch.bfloat16)
    elif out.shape != (M, n_out) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        raise ValueError("bad out tensor")
    with torch.cuda.device(a.device):
        _C.gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
                     1 if swiglu else 0, torch.cuda.current_stream().cuda_stream)
    return out
