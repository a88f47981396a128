"""The library baseline for the fused tensor-parallel MLP: NCCL all-gather, cuBLAS GEMMs, an
elementwise SwiGLU kernel and NCCL reduce-scatter, each a separate launch on one stream."""
import torch
import torch.distributed as dist


class NcclCublasMLP:
    def __init__(self, w_gate_up: torch.Tensor, w_down: torch.Tensor, tokens: int, tp: int):
        self.w_gate_up, self.w_down, self.tp = w_gate_up, w_down, tp
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
        gu = torch.matmul(x, self.w_gate_up.t())
        f = gu.shape[1] // 2
        self.h = torch.nn.functional.silu(gu[:, :f]) * gu[:, f:]
        return self.h

    def down(self) -> torch.Tensor:
        """down GEMM, reduce-scatter"""
        part = torch.matmul(self.h, self.w_down.t())
        if self.tp > 1:
            dist.reduce_scatter_tensor(self.y, part)
            return self.y
        return part

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        self.up(x_shard)
        return self.down()

    __call__ = forward
