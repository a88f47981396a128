#!/usr/bin/env python
"""Where the time of the two fused tensor-parallel GEMM kernels goes, one JSON line on rank 0.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        --master-port 29500 benchmarks/tp_breakdown.py [--tokens 16384 --hidden 4096 --ffn 14336]

Per rank the shapes are those of a Llama-style MLP at TP = N.  Reported (microseconds, CUDA events,
max over ranks): the plain GEMMs, NCCL collectives alone and NCCL + cuBLAS for both halves, the
all-gather -> GEMM under every transport (copy engines with 0..3 lanes and 1..4 chunks, dedicated
communication CTAs, forwarder warps), the GEMM -> reduce-scatter with TMA tile stores and (with
--rs-ce) with copy engines, and the same kernels with one phase left out (no tail, no remote
stores) to see what each phase costs.  Also the maximum absolute error of both fused kernels
against the NCCL + cuBLAS result.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402
import torch.nn.functional as F  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--rs-ce", action="store_true", help="also time the copy-engine reduce-scatter")
    args = ap.parse_args()
    os.environ.setdefault("UCCL_BOOTSTRAP_IFNAME", "lo")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from unified_ccl_b200 import Communicator
    from unified_ccl_b200.ops import gemm_bf16
    from unified_ccl_b200.parallel import allgather_gemm, gemm_reduce_scatter

    comm = Communicator(rank, world)
    M, H = args.tokens, args.hidden
    fs = args.ffn // world
    rows = M // world
    x_shard = torch.randn(rows, H, device=dev).to(torch.bfloat16)
    x_full = comm.empty((M, H), torch.bfloat16)
    x_full.normal_()
    wgu = (torch.randn(2 * fs, H, device=dev) * 0.02).to(torch.bfloat16)
    wd = (torch.randn(H, fs, device=dev) * 0.02).to(torch.bfloat16)
    h = torch.empty(M, fs, device=dev, dtype=torch.bfloat16)
    h.normal_()
    stage = comm.empty((M, H), torch.bfloat16)
    y = torch.empty(rows, H, device=dev, dtype=torch.bfloat16)
    c_plain = torch.empty(M, H, device=dev, dtype=torch.bfloat16)
    xf2 = torch.empty(M, H, device=dev, dtype=torch.bfloat16)

    def timed(fn, it=args.iters, w=5):
        for _ in range(w):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(it):
            fn()
        e.record()
        dist.barrier()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / it], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return round(t.item() * 1e3, 1)

    def nccl_up():
        dist.all_gather_into_tensor(xf2, x_shard)
        gu = xf2 @ wgu.t()
        return F.silu(gu[:, :fs]) * gu[:, fs:]

    def nccl_down():
        dist.reduce_scatter_tensor(y, h @ wd.t())

    def ag():
        allgather_gemm(comm, x_shard, x_full, wgu, out=h, swiglu=True)

    def rs():
        gemm_reduce_scatter(comm, h, wd, stage, out=y)

    res = {"n": world, "tokens": M, "hidden": H, "ffn_per_rank": fs}
    res["gemm_up"] = timed(lambda: gemm_bf16(x_full, wgu, out=h, swiglu=True))
    res["gemm_down"] = timed(lambda: gemm_bf16(h, wd, out=c_plain))
    res["nccl_ag"] = timed(lambda: dist.all_gather_into_tensor(xf2, x_shard))
    res["nccl_rs"] = timed(lambda: dist.reduce_scatter_tensor(y, c_plain))
    res["nccl_ag_cublas"] = timed(nccl_up)
    res["cublas_nccl_rs"] = timed(nccl_down)
    # correctness of the defaults
    ag()
    torch.cuda.synchronize()
    ref = nccl_up()
    res["ag_max_abs_err"] = float((h.float() - ref.float()).abs().max())
    res["x_full_gathered"] = bool(torch.equal(x_full, xf2))
    rs()
    torch.cuda.synchronize()
    y1 = y.clone()
    nccl_down()
    torch.cuda.synchronize()
    res["rs_max_abs_err"] = float((y1.float() - y.float()).abs().max())
    # all-gather -> GEMM by transport
    for lanes in ((0,) if world <= 2 else (0, 1, 2, 3)):
        for chunks in (1, 2, 4):
            comm.set_fused_options("ce", lanes, chunks)
            res["ag_ce_lanes%d_chunks%d" % (lanes, chunks)] = timed(ag)
    for ctas in (8, 16, 24):
        comm.set_fused_options("kernel", ctas, 0)
        res["ag_ctas%d" % ctas] = timed(ag)
    comm.set_fused_options("spread")
    res["ag_spread"] = timed(ag)
    comm.set_fused_options()
    # GEMM -> reduce-scatter, and what its phases cost (debug switches of the kernel)
    res["rs_tma"] = timed(rs)
    for bits, name in ((1, "rs_tma_no_tail"), (2, "rs_tma_no_remote_stores"), (3, "rs_tma_no_tail_no_stores"),
                       (16, "rs_tma_all_local")):
        os.environ["UCCL_FUSED_DEBUG"] = str(bits)
        res[name] = timed(rs)
    os.environ["UCCL_FUSED_DEBUG"] = "0"
    for red in (8, 16):
        comm.set_fused_rs_reducers(red)
        res["rs_tma_reducers%d" % red] = timed(rs)
    comm.set_fused_rs_reducers(0)
    res["async_error"] = comm.async_error()
    if rank == 0:
        print(json.dumps(res), flush=True)
    comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
