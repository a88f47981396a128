"""Llama-style SwiGLU MLP block, tensor parallel with sequence-parallel activations.

    x_shard [M / tp, H]  --all-gather-->  x [M, H]
    h = silu(x @ Wg_r.T) * (x @ Wu_r.T)            column-parallel, Wg_r / Wu_r [F / tp, H]
    y_shard = reduce_scatter(h @ Wd_r.T)           row-parallel,    Wd_r [H, F / tp]

Both collectives run inside the GEMM kernels (all-gather -> GEMM with the SwiGLU epilogue, and
GEMM -> reduce-scatter), so one forward pass is two GEMM launches, each behind one small rank-barrier kernel.
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

    # candidates of autotune(): (all-gather mode, communication CTAs or copy-engine lanes, chunks per peer)
    AG_CANDIDATES = (("ce", 0, 2), ("ce", 1, 2), ("ce", 1, 4), ("ce", 2, 2),
                     ("spread", 0, 0), ("kernel", 8, 0), ("kernel", 16, 0))

    def _align(self, stream):
        """Lines the ranks' hosts up before a timed region, so that it is not spent waiting for a late peer."""
        if not hasattr(self, "_tick"):
            self._tick = torch.zeros(1, device=self.h.device)
        self.comm.allreduce(self._tick)
        stream.synchronize()

    def _apply_ag(self, mode, ctas, chunks):
        self.comm.set_fused_options(mode, ctas, chunks)

    def autotune(self, x_shard: torch.Tensor, iters: int = 5, candidates=None):
        """Times the all-gather -> GEMM half of the block under each candidate setting (CUDA events,
        summed over the ranks so that every rank takes the same decision) and keeps the fastest.
        Returns ``{candidate: microseconds averaged over ranks}``; a no-op on one rank."""
        if self.tp == 1:
            return {}
        cands = tuple(candidates or self.AG_CANDIDATES)
        if self.tp <= 2:  # lanes only differ from one stream per peer when there are several peers
            cands = tuple(c for c in cands if not (c[0] == "ce" and c[1] > 0))
        times = torch.zeros(len(cands), device=self.h.device, dtype=torch.float32)
        stream = torch.cuda.current_stream(self.h.device)
        for i, (mode, ctas, chunks) in enumerate(cands):
            try:
                self._apply_ag(mode, ctas, chunks)
                allgather_gemm(self.comm, x_shard, self.x_full, self.w_gate_up, out=self.h, swiglu=True)  # warm-up
                self._align(stream)
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record(stream)
                for _ in range(iters):
                    allgather_gemm(self.comm, x_shard, self.x_full, self.w_gate_up, out=self.h, swiglu=True)
                e.record(stream)
                e.synchronize()
                times[i] = s.elapsed_time(e) * 1e3 / iters
            except (ValueError, RuntimeError):
                # a setting this shape does not allow (refused before anything is launched, on
                # every rank alike): out of the running
                times[i] = 1e9
        self.comm.allreduce(times)
        stream.synchronize()
        avg = (times / self.tp).tolist()
        best = min(range(len(cands)), key=lambda i: avg[i])
        self._apply_ag(*cands[best])
        self.ag_choice = cands[best]
        return {cands[i]: round(avg[i], 1) for i in range(len(cands))}

    # candidates of autotune_rs(): ("kernel", CTAs that only sum)
    RS_CANDIDATES = (("kernel", 0), ("kernel", 8), ("kernel", 16), ("kernel", 24))

    def _apply_rs(self, mode, arg):
        self.comm.set_fused_rs_reducers(arg)

    def autotune_rs(self, iters: int = 5, candidates=None):
        """The same for the GEMM -> reduce-scatter half (``self.h`` must hold activations, e.g. after one
        forward pass)."""
        if self.tp == 1:
            return {}
        cands = tuple(candidates or self.RS_CANDIDATES)
        times = torch.zeros(len(cands), device=self.h.device, dtype=torch.float32)
        stream = torch.cuda.current_stream(self.h.device)
        for i, (mode, chunks) in enumerate(cands):
            try:
                self._apply_rs(mode, chunks)
                gemm_reduce_scatter(self.comm, self.h, self.w_down, self.c_partial, out=self.y)  # warm-up
                self._align(stream)
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record(stream)
                for _ in range(iters):
                    gemm_reduce_scatter(self.comm, self.h, self.w_down, self.c_partial, out=self.y)
                e.record(stream)
                e.synchronize()
                times[i] = s.elapsed_time(e) * 1e3 / iters
            except (ValueError, RuntimeError):
                times[i] = 1e9
        self.comm.allreduce(times)
        stream.synchronize()
        avg = (times / self.tp).tolist()
        best = min(range(len(cands)), key=lambda i: avg[i])
        self._apply_rs(*cands[best])
        self.rs_choice = cands[best]
        return {cands[i]: round(avg[i], 1) for i in range(len(cands))}

    def reference(self, x_full: torch.Tensor) -> torch.Tensor:
        """fp32 PyTorch restatement of this rank's partial result (before the reduce-scatter)."""
        fs = self.ffn // self.tp
        x = x_full.float()
        g = x @ self.w_gate_up[:fs].float().t()
        u = x @ self.w_gate_up[fs:].float().t()
        h = (torch.nn.functional.silu(g) * u).to(torch.bfloat16).float()
        return h @ self.w_down.float().t()
