"""The library baseline for the fused tensor-parallel MLP: NCCL all-gather, cuBLAS GEMMs, an
elementwise SwiGLU step and NCCL reduce-scatter, each a separate launch on one stream.

Two forms of the SwiGLU step: ``fused_swiglu=False`` is plain eager PyTorch (three elementwise
kernels with fresh allocations), ``fused_swiglu=True`` a one-pass kernel into a preallocated
buffer (baseline/swiglu_kernel.cu), which is the stronger comparator."""
import ctypes
import os

import torch
import torch.distributed as dist

_LIB = None


def _swiglu_lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libbaseline_swiglu.so")
        _LIB = ctypes.CDLL(path)
        _LIB.baselineSwiglu.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_long, ctypes.c_int, ctypes.c_void_p]
    return _LIB


class NcclCublasMLP:
    def __init__(self, w_gate_up: torch.Tensor, w_down: torch.Tensor, tokens: int, tp: int, fused_swiglu: bool = False):
        self.w_gate_up, self.w_down, self.tp = w_gate_up, w_down, tp
        self.fused_swiglu = fused_swiglu
        if fused_swiglu:
            f2 = w_gate_up.shape[0]
            self.gu = torch.empty(tokens, f2, device=w_gate_up.device, dtype=torch.bfloat16)
            self.h = torch.empty(tokens, f2 // 2, device=w_gate_up.device, dtype=torch.bfloat16)
            self.part = torch.empty(tokens, w_down.shape[0], device=w_gate_up.device, dtype=torch.bfloat16)
        hidden = w_gate_up.shape[1]
        dev = w_gate_up.device
        self.x_full = torch.empty(tokens, hidden, device=dev, dtype=torch.bfloat16)
        self.y = torch.empty(tokens // tp, hidden, device=dev, dtype=torch.bfloat16)

    def up(self, x_shard: torch.Tensor) -> torch.Tensor:
        """all-gather, up/gate GEMM, SwiGLU"""
        if self.tp > 1:
            dist.all_gather_into_tensor(self.x_full, x_shard)
            x = self.x_full
        else:
            x = x_shard
        if self.fused_swiglu:
            torch.matmul(x, self.w_gate_up.t(), out=self.gu)
            rc = _swiglu_lib().baselineSwiglu(self.gu.data_ptr(), self.h.data_ptr(), self.gu.shape[0], self.gu.shape[1] // 2,
                                              torch.cuda.current_stream().cuda_stream)
            if rc != 0:
                raise RuntimeError("baseline SwiGLU kernel failed: cudaError %d" % rc)
            return self.h
        gu = torch.matmul(x, self.w_gate_up.t())
        f = gu.shape[1] // 2
        self.h = torch.nn.functional.silu(gu[:, :f]) * gu[:, f:]
        return self.h

    def down(self) -> torch.Tensor:
        """down GEMM, reduce-scatter"""
        part = torch.matmul(self.h, self.w_down.t(), out=self.part) if self.fused_swiglu else torch.matmul(self.h, self.w_down.t())
        if self.tp > 1:
            dist.reduce_scatter_tensor(self.y, part)
            return self.y
        return part

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        self.up(x_shard)
        return self.down()

    __call__ = forward
