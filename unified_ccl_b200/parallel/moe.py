"""Expert-parallel MoE dispatch (bf16 -> fp8 e4m3 with 1x128 fp32 scales) and weighted combine."""
import torch

from .. import _C
from ..communicator import Communicator, _tensor_from_ptr


class MoeDispatcher:
    """Owns the symmetric receive area of one MoE layer.

    ``dispatch(x, topk_idx)`` routes every (token, k) pair to the rank that owns the expert and
    returns views of the receive area; the caller computes one bf16 output row per received row
    into ``expert_out`` (same indexing); ``combine(topk_weight)`` returns, for every local token,
    the weighted sum of its top-k expert outputs.
    """

    def __init__(self, comm: Communicator, max_tokens: int, hidden: int, num_experts: int, topk: int,
                 capacity_factor: float = 0.0):
        if not comm.on_gpu:
            raise ValueError("MoE dispatch needs a communicator on GPUs")
        self.comm, self.max_tokens, self.hidden, self.num_experts, self.topk = comm, max_tokens, hidden, num_experts, topk
        self._ctx = _C.moe_create(comm.handle, max_tokens, hidden, num_experts, topk, float(capacity_factor))
        lay = _C.moe_layout(self._ctx)
        n, rows = lay["nranks"], lay["rows_per_source"]
        dev = comm.info["cuda_device"]
        self.rows_per_source = rows
        self.recv_x = _tensor_from_ptr(lay["recv_x"], n * rows * hidden, torch.float8_e4m3fn, dev).view(n, rows, hidden)
        self.recv_scale = _tensor_from_ptr(lay["recv_scale"], n * rows * (hidden // 128), torch.float32, dev).view(n, rows, hidden // 128)
        self.recv_meta = _tensor_from_ptr(lay["recv_meta"], n * rows * 4, torch.int32, dev).view(n, rows, 4)
        self.recv_counts = _tensor_from_ptr(lay["recv_counts"], n, torch.int32, dev)
        self.expert_out = _tensor_from_ptr(lay["expert_out"], n * rows * hidden, torch.bfloat16, dev).view(n, rows, hidden)
        self._tokens = 0

    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor):
        if x.dtype != torch.bfloat16 or not x.is_contiguous() or x.shape[1] != self.hidden:
            raise TypeError("x must be contiguous bf16 [tokens, hidden]")
        if topk_idx.dtype != torch.int32 or not topk_idx.is_contiguous() or topk_idx.shape != (x.shape[0], self.topk):
            raise TypeError("topk_idx must be contiguous int32 [tokens, topk]")
        self._tokens = x.shape[0]
        _C.moe_dispatch(self._ctx, x.data_ptr(), topk_idx.data_ptr(), self._tokens, self.comm._stream())
        return self.recv_x, self.recv_scale, self.recv_meta, self.recv_counts

    def combine(self, topk_weight: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
        if topk_weight.dtype != torch.float32 or not topk_weight.is_contiguous() or topk_weight.shape != (self._tokens, self.topk):
            raise TypeError("topk_weight must be contiguous fp32 [tokens, topk] of the last dispatch")
        if out is None:
            out = torch.empty(self._tokens, self.hidden, device=topk_weight.device, dtype=torch.bfloat16)
        _C.moe_combine(self._ctx, topk_weight.data_ptr(), self._tokens, out.data_ptr(), self.comm._stream())
        return out

    def overflow(self) -> int:
        return _C.moe_overflow(self._ctx)

    def close(self):
        if self._ctx:
            ctx, self._ctx = self._ctx, 0
            _C.moe_destroy(ctx)


def quantize_fp8_block128(x: torch.Tensor):
    """fp32 PyTorch restatement of the dispatch cast: per 128 elements scale = amax / 448."""
    t, h = x.shape
    xb = x.float().view(t, h // 128, 128)
    scale = xb.abs().amax(-1).clamp_min(1e-10) / 448.0
    q = (xb / scale.unsqueeze(-1)).to(torch.float8_e4m3fn)
    return q.view(t, h), scale
