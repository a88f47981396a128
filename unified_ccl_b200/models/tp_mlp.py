"""Llama-style SwiGLU MLP block, tensor parallel with sequence-parallel activations.

    x_shard [M / tp, H]  --all-gather-->  x [M, H]
    h = silu(x @ Wg_r.T) * (x @ Wu_r.T)            column-parallel, Wg_r / Wu_r [F / tp, H]
    y_shard = reduce_scatter(h @ Wd_r.T)           row-parallel,    Wd_r [H, F / tp]

Both collectives run inside the GEMM kernels (all-gather -> GEMM with the SwiGLU epilogue, and
GEMM -> reduce-scatter), so one forward pass is two kernel launches plus three tiny barriers.
"""
import torch

from ..communicator import Communicator
from ..ops import gemm_bf16
from ..parallel import allgather_gemm, gemm_reduce_scatter


class TensorParallelMLP:
    def __init__(self, comm: Communicator, hidden: int, ffn: int, tokens: int, seed: int = 0, device=None):
        tp = comm.world_size
        if ffn % tp or tokens % tp:
            raise ValueError("ffn and tokens must be divisible by the tensor-parallel size")
        self.comm, self.hidden, self.ffn, self.tokens, self.tp = comm, hidden, ffn, tokens, tp
        dev = device if device is not None else torch.device("cuda", comm.info["cuda_device"])
        g = torch.Generator(device="cpu").manual_seed(seed)
        # full weights are generated from the seed on every rank and sliced, so that all
        # tensor-parallel sizes compute the same function
        fs = ffn // tp
        r = comm.rank
        wg = (torch.randn(ffn, hidden, generator=g) * 0.02)[r * fs:(r + 1) * fs]
        wu = (torch.randn(ffn, hidden, generator=g) * 0.02)[r * fs:(r + 1) * fs]
        wd = (torch.randn(hidden, ffn, generator=g) * 0.02)[:, r * fs:(r + 1) * fs]
        self.w_gate_up = torch.cat([wg, wu], 0).to(dev, torch.bfloat16).contiguous()  # [2 * F / tp, H]
        self.w_down = wd.to(dev, torch.bfloat16).contiguous()                          # [H, F / tp]
        self.x_full = comm.empty((tokens, hidden), torch.bfloat16) if tp > 1 else None
        self.h = torch.empty(tokens, fs, device=dev, dtype=torch.bfloat16)
        self.c_partial = comm.empty((tokens, hidden), torch.bfloat16) if tp > 1 else None
        self.y = torch.empty(tokens // tp, hidden, device=dev, dtype=torch.bfloat16)

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        if self.tp == 1:
            gemm_bf16(x_shard, self.w_gate_up, out=self.h, swiglu=True)
            gemm_bf16(self.h, self.w_down, out=self.y)
            return self.y
        allgather_gemm(self.comm, x_shard, self.x_full, self.w_gate_up, out=self.h, swiglu=True)
        gemm_reduce_scatter(self.comm, self.h, self.w_down, self.c_partial, out=self.y)
        return self.y

    __call__ = forward

    def reference(self, x_full: torch.Tensor) -> torch.Tensor:
        """fp32 PyTorch restatement of this rank's partial result (before the reduce-scatter)."""
        fs = self.ffn // self.tp
        x = x_full.float()
        g = x @ self.w_gate_up[:fs].float().t()
        u = x @ self.w_gate_up[fs:].float().t()
        h = (torch.nn.functional.silu(g) * u).to(torch.bfloat16).float()
        return h @ self.w_down.float().t()
