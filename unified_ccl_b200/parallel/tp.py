"""Fused tensor-parallel operators (bf16, CUDA)."""
import torch

from .. import _C
from ..communicator import Communicator


def _bf16(*ts):
    for t in ts:
        if t.dtype != torch.bfloat16 or not t.is_cuda or not t.is_contiguous():
            raise TypeError("fused operators take contiguous bf16 CUDA tensors")


def allreduce_residual_rmsnorm(comm: Communicator, x: torch.Tensor, residual: torch.Tensor, gamma: torch.Tensor,
                               eps: float = 1e-6, out: torch.Tensor = None, residual_out: torch.Tensor = None):
    """``h = allreduce(x) + residual``; returns ``(rmsnorm(h) * gamma, h)`` in one kernel.

    ``x`` holds this rank's partial sums [tokens, hidden].  For zero-copy operation allocate ``x`` and
    ``residual_out`` with ``comm.empty``; other tensors are staged (size limited by UCCL_STAGING_BYTES).
    ``residual_out`` may be ``residual`` itself.
    """
    _bf16(x, residual, gamma)
    tokens, hidden = x.shape
    if out is None:
        out = torch.empty_like(x)
    if residual_out is None:
        residual_out = residual
    _bf16(out, residual_out)
    _C.allreduce_residual_rmsnorm(comm.handle, x.data_ptr(), residual.data_ptr(), gamma.data_ptr(), out.data_ptr(),
                                  residual_out.data_ptr(), tokens, hidden, float(eps), comm._stream())
    return out, residual_out


def autotune_allreduce_residual_rmsnorm(comm: Communicator, x: torch.Tensor, residual: torch.Tensor, gamma: torch.Tensor,
                                        eps: float = 1e-6, out: torch.Tensor = None, iters: int = 10, candidates=(0, 1, 2, 4)):
    """Times :func:`allreduce_residual_rmsnorm` on these tensors under each shape of its switch path (CUDA
    events, summed over the ranks so that every rank takes the same decision), keeps the fastest on this
    communicator and returns ``{rows: microseconds averaged over ranks}``.  The runs update ``residual`` in
    place (as a layer stack does), so its content is not preserved.  Collective; a no-op without an NVSwitch
    multicast alias or on one rank."""
    if comm.world_size == 1 or not comm.info["nvls"]:
        return {}
    if out is None:
        out = torch.empty_like(x)
    stream = torch.cuda.current_stream(x.device)
    times = torch.zeros(len(candidates), device=x.device, dtype=torch.float32)
    tick = torch.zeros(1, device=x.device)
    for i, rows in enumerate(candidates):
        comm.set_fused_norm_rows(rows)
        allreduce_residual_rmsnorm(comm, x, residual, gamma, eps, out=out, residual_out=residual)  # warm-up
        # line the ranks' hosts up, so that the timed launches are not spent waiting for a late peer
        comm.allreduce(tick)
        stream.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(stream)
        for _ in range(iters):
            allreduce_residual_rmsnorm(comm, x, residual, gamma, eps, out=out, residual_out=residual)
        e.record(stream)
        e.synchronize()
        times[i] = s.elapsed_time(e) * 1e3 / iters
    comm.allreduce(times)
    stream.synchronize()
    avg = (times / comm.world_size).tolist()
    best = min(range(len(candidates)), key=lambda i: avg[i])
    comm.set_fused_norm_rows(candidates[best])
    return {candidates[i]: round(avg[i], 1) for i in range(len(candidates))}


def allgather_gemm(comm: Communicator, x_shard: torch.Tensor, x_full: torch.Tensor, w: torch.Tensor,
                   out: torch.Tensor = None, swiglu: bool = False) -> torch.Tensor:
    """``out = allgather(x_shard) @ w.T`` with the gather overlapped tile by tile with the GEMM.

    ``x_shard`` [M / world, K]; ``x_full`` [M, K] symmetric scratch (``comm.empty``) that receives the gathered
    activations; ``w`` [N, K].  With ``swiglu`` the rows of ``w`` are [gate; up] and ``out`` is [M, N/2].
    """
    _bf16(x_shard, x_full, w)
    M, K = x_full.shape
    N = w.shape[0]
    if x_shard.shape[0] * comm.world_size != M or x_shard.shape[1] != K or w.shape[1] != K:
        raise ValueError("shape mismatch")
    n_out = N // 2 if swiglu else N
    if out is None:
        out = torch.empty(M, n_out, device=x_full.device, dtype=torch.bfloat16)
    _bf16(out)
    _C.allgather_gemm(comm.handle, x_shard.data_ptr(), x_full.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K,
                      1 if swiglu else 0, comm._stream())
    return out


def gemm_reduce_scatter(comm: Communicator, a: torch.Tensor, w: torch.Tensor, c_partial: torch.Tensor,
                        out: torch.Tensor = None) -> torch.Tensor:
    """``out = reduce_scatter(a @ w.T)`` over the rows, reduced while later tiles are still being computed.

    ``a`` [M, K]; ``w`` [N, K]; ``c_partial`` [M, N] symmetric scratch (``comm.empty``); ``out`` [M / world, N].
    """
    _bf16(a, w, c_partial)
    M, K = a.shape
    N = w.shape[0]
    if c_partial.shape != (M, N) or w.shape[1] != K:
        raise ValueError("shape mismatch")
    if out is None:
        out = torch.empty(M // comm.world_size, N, device=a.device, dtype=torch.bfloat16)
    _bf16(out)
    _C.gemm_reduce_scatter(comm.handle, a.data_ptr(), w.data_ptr(), c_partial.data_ptr(), out.data_ptr(), M, N, K,
                           comm._stream())
    return out
