#!/usr/bin/env python
"""Headline benchmark: the fused tensor-parallel Llama-style MLP block (all-gather -> GEMM with
SwiGLU, GEMM -> reduce-scatter) at TP = number of GPUs, batch 4 x seq 4096, hidden 4096,
ffn 14336, bf16, random-init weights and synthetic activations.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5

Rank 0 prints ONE JSON line.  `value` is the device-timed layer time in microseconds (max over
ranks, CUDA events around exactly `steps` launches, barrier + synchronize on both sides); the
NCCL + cuBLAS comparator is timed the same way in the same process and reported next to it,
together with an all-reduce bus-bandwidth sample against NCCL when N > 1.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# read by CUDA when the context is created: enough hardware queues for the side streams of the
# copy-engine transports (the package sets the same default on import; both arms run under it)
os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")

BATCH, SEQ, HIDDEN, FFN = 4, 4096, 4096, 14336


def reference_arm():
    # The reference is SYCL / Level-Zero code for Intel GPUs with a CMake + icpx build and no
    # setup.py / pyproject.toml: `pip install --target baseline/_ref <reference tree>` answers
    # "Neither 'setup.py' nor 'pyproject.toml' found", and there is no icpx on this image.
    print(json.dumps({"impl": "reference",
                      "unavailable": "reference is Intel SYCL/Level-Zero code built with icpx+CMake: not pip-installable "
                                     "(no setup.py/pyproject.toml) and cannot target NVIDIA GPUs"}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-sweep", action="store_true", help="skip the all-reduce sample against NCCL")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm()
        return 0
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist

    os.environ.setdefault("UCCL_BOOTSTRAP_IFNAME", "lo")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node %d" % args.gpus)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from baseline.nccl_mlp import NcclCublasMLP
    from unified_ccl_b200 import Communicator
    from unified_ccl_b200.models import TensorParallelMLP
    from unified_ccl_b200.utils import ClockSampler

    comm = Communicator(rank, world)
    tokens = BATCH * SEQ
    rows = tokens // world
    mlp = TensorParallelMLP(comm, HIDDEN, FFN, tokens, seed=0)
    base = NcclCublasMLP(mlp.w_gate_up, mlp.w_down, tokens, world)
    base_fused = NcclCublasMLP(mlp.w_gate_up, mlp.w_down, tokens, world, fused_swiglu=True)  # one-pass SwiGLU: the stronger comparator
    autotune = {}
    autotune_rs = {}
    g = torch.Generator(device="cpu").manual_seed(1234 + rank)
    x_host = torch.randn(rows, HIDDEN, generator=g).to(torch.bfloat16).pin_memory()
    x_dev = x_host.to(dev)
    # untimed: pick how the all-gather -> GEMM moves its rows on this box (measured, same on every rank)
    if world > 1 and not os.environ.get("UCCL_FUSED_AG"):
        autotune = {"%s/ctas%d/chunks%d" % k: v for k, v in mlp.autotune(x_dev).items()}
        autotune["chosen"] = "%s/ctas%d/chunks%d" % mlp.ag_choice
    # untimed: the same for the GEMM -> reduce-scatter half (how many CTAs only sum)
    if world > 1 and not os.environ.get("UCCL_FUSED_RS_REDUCERS"):
        mlp(x_dev)  # fills the activations the second half works on
        autotune_rs = {"%s/%d" % k: v for k, v in mlp.autotune_rs().items()}  # kernel/<reducer CTAs>
        autotune_rs["chosen"] = "%s/%d" % mlp.rs_choice

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        s = torch.cuda.Event(enable_timing=True)
        e = torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(steps):
            fn()
        e.record()
        barrier()
        return max_over_ranks(s.elapsed_time(e)) / steps  # ms per step

    # ---- kernel-level number: inputs already on the device
    with ClockSampler(local_rank) as clk:
        ms_ours = timed(lambda: mlp(x_dev), args.steps, args.warmup)
    clocks = clk.summary()
    ms_base = timed(lambda: base(x_dev), args.steps, args.warmup)
    ms_base_fused = timed(lambda: base_fused(x_dev), args.steps, args.warmup)

    # ---- end to end through the public API: H2D of the step's input, D2H of a checksum
    x_in = torch.empty_like(x_dev)
    result_host = torch.empty(1, dtype=torch.float32).pin_memory()

    def e2e_step(model):
        x_in.copy_(x_host, non_blocking=True)
        y = model(x_in)
        result_host.copy_(y[:, :8].float().sum().reshape(1), non_blocking=True)

    ms_e2e = timed(lambda: e2e_step(mlp), args.steps, args.warmup)
    ms_e2e_base = timed(lambda: e2e_step(base), args.steps, args.warmup)
    ms_e2e_base_fused = timed(lambda: e2e_step(base_fused), args.steps, args.warmup)

    # ---- correctness spot check against the fp32 restatement (outside the timed regions)
    y = mlp(x_dev).float()
    yb = base(x_dev).float()
    torch.cuda.synchronize()
    rel = ((y - yb).abs().max() / yb.abs().max().clamp_min(1e-6)).item()

    # ---- the two halves of the block on their own (untimed extra; explains the headline number)
    halves = {}
    if world > 1:
        from unified_ccl_b200.parallel import allgather_gemm, gemm_reduce_scatter
        halves["ag_gemm_us"] = round(1e3 * timed(lambda: allgather_gemm(comm, x_dev, mlp.x_full, mlp.w_gate_up, out=mlp.h, swiglu=True), 10, 3), 1)
        halves["gemm_rs_us"] = round(1e3 * timed(lambda: gemm_reduce_scatter(comm, mlp.h, mlp.w_down, mlp.c_partial, out=mlp.y), 10, 3), 1)
        halves["nccl_ag_cublas_us"] = round(1e3 * timed(lambda: base.up(x_dev), 10, 3), 1)
        halves["cublas_nccl_rs_us"] = round(1e3 * timed(lambda: base.down(), 10, 3), 1)

    # ---- all-reduce sample against NCCL (bus bandwidth, bf16, symmetric buffers)
    sweep = []
    if world > 1 and not args.no_sweep:
        for nbytes in (8 << 10, 1 << 20, 64 << 20, 1 << 30):
            n_el = nbytes // 2
            t_sym = comm.empty(n_el, torch.bfloat16)
            t_sym.fill_(1.0)
            t_nccl = torch.ones(n_el, device=dev, dtype=torch.bfloat16)
            it = 50 if nbytes <= (1 << 20) else 10
            ms_u = timed(lambda: comm.allreduce(t_sym), it, 5)
            ms_n = timed(lambda: dist.all_reduce(t_nccl), it, 5)
            f = 2.0 * (world - 1) / world
            sweep.append({"bytes": nbytes, "ours_us": round(ms_u * 1e3, 2), "nccl_us": round(ms_n * 1e3, 2),
                          "ours_busbw_gbs": round(nbytes * f / (ms_u * 1e-3) / 1e9, 1),
                          "nccl_busbw_gbs": round(nbytes * f / (ms_n * 1e-3) / 1e9, 1)})
            comm.free(t_sym)

    flops = 2.0 * tokens * HIDDEN * (2 * FFN) / world + 2.0 * tokens * (FFN / world) * HIDDEN
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak_tflops = peaks.get("bf16_tflops_sustained", 1400.0)
    link_gbs = 770.0
    ag_bytes = (world - 1) / world * tokens * HIDDEN * 2
    roof_us = max(flops / (peak_tflops * 1e12), 2 * ag_bytes / (link_gbs * 1e9) if world > 1 else 0.0) * 1e6
    launches_per_step = 2 if world == 1 else 4  # two fused GEMM kernels (+ one rank-barrier kernel in front of each)

    if rank == 0:
        out = {
            "metric": "fused_tp_mlp_layer_us",
            "value": round(ms_ours * 1e3, 2),
            "unit": "us",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": round(ms_ours, 5),
            "higher_is_better": False,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic activations N(0,1) seeded per rank, random-init weights N(0,0.02)",
            "config": {"model": "llama-style SwiGLU MLP block", "global_batch": BATCH, "seq_len": SEQ, "hidden": HIDDEN,
                       "ffn": FFN, "parallelism": "tp%d" % world,
                       "l2": "per-rank working set (weights + activations + scratch) exceeds the 126 MB L2; no flush",
                       "cuda_device_max_connections": os.environ.get("CUDA_DEVICE_MAX_CONNECTIONS")},
            "nccl_cublas_us": round(ms_base * 1e3, 2),
            "speedup_vs_nccl_cublas": round(ms_base / ms_ours, 3),
            "nccl_cublas_fused_swiglu_us": round(ms_base_fused * 1e3, 2),
            "speedup_vs_nccl_cublas_fused_swiglu": round(ms_base_fused / ms_ours, 3),
            "tokens_per_s": round(tokens / (ms_ours * 1e-3), 1),
            "roofline_us": round(roof_us, 1),
            "fraction_of_roofline": round(roof_us / (ms_ours * 1e3), 3),
            "roofline_basis": "max(FLOPs / measured sustained cuBLAS bf16, 2 x (N-1)/N x activation bytes / 770 GB/s)",
            "max_rel_diff_vs_nccl_cublas": round(rel, 5),
            "clocks": clocks,
            "e2e": {"value": round(ms_e2e * 1e3, 2), "unit": "us", "h2d_bytes_per_step": x_host.numel() * 2,
                    "d2h_bytes_per_step": 4, "nccl_cublas_value": round(ms_e2e_base * 1e3, 2),
                    "nccl_cublas_fused_swiglu_value": round(ms_e2e_base_fused * 1e3, 2)},
            "gpu_launches": launches_per_step * args.steps,
            "allreduce_vs_nccl": sweep,
            "comm": {k: comm.info[k] for k in ("nvls", "p2p_mode", "net_active")},
            "ag_gemm_autotune_us": autotune,
            "gemm_rs_autotune_us": autotune_rs,
            "halves": halves,
        }
        print(json.dumps(out))
    barrier()
    comm.destroy()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
