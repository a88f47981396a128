#!/usr/bin/env python
"""Run one single-GPU kernel case a few times (for timing with CUDA events, or under ncu).

    python benchmarks/kernel_case.py --case gemm --m 4096 --n 3584 --k 4096 --iters 3
    python benchmarks/kernel_case.py --case gemm_swiglu --m 4096 --n 7168 --k 4096
    python benchmarks/kernel_case.py --case add_norm --tokens 8192 --hidden 8192
    python benchmarks/kernel_case.py --case moe_dispatch --tokens 4096 --hidden 7168
    python benchmarks/kernel_case.py --case moe_combine --tokens 4096 --hidden 7168
    python benchmarks/kernel_case.py --case gemm_rs_self --m 8192 --n 4096 --k 1792

Prints one JSON line with the median device time and the achieved fraction of the measured
peaks in MEASURED_PEAKS.json (copy bandwidth for the memory-bound cases, cuBLAS bf16 burst
throughput for the GEMMs).  Inputs are larger than the L2 or the L2 is flushed between iterations.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True)
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=3584)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--experts", type=int, default=32)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--cublas", action="store_true", help="time torch.matmul (cuBLAS) on the same shape instead")
    args = ap.parse_args()

    os.environ.setdefault("UCCL_BOOTSTRAP_IFNAME", "lo")
    from unified_ccl_b200.ops import gemm_bf16
    from unified_ccl_b200.utils import device_time_ms

    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    basis = "fallback"
    try:
        peaks.update(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))))
        basis = "measured"
    except OSError:
        pass
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    out = {"case": args.case, "peaks": basis}
    if args.case in ("gemm", "gemm_swiglu"):
        a = torch.randn(args.m, args.k, device=dev).to(torch.bfloat16)
        b = (torch.randn(args.n, args.k, device=dev) * 0.02).to(torch.bfloat16)
        sw = args.case == "gemm_swiglu"
        c = torch.empty(args.m, args.n // 2 if sw else args.n, device=dev, dtype=torch.bfloat16)
        fn = (lambda: torch.matmul(a, b.t())) if args.cublas else (lambda: gemm_bf16(a, b, out=c, swiglu=sw))
        t = device_time_ms(fn, args.iters, args.warmup)
        flops = 2.0 * args.m * args.n * args.k
        out.update(m=args.m, n=args.n, k=args.k, ms=round(t["median"], 4), tflops=round(flops / t["median"] / 1e9, 1),
                   frac_of_cublas_peak=round(flops / t["median"] / 1e9 / peaks["bf16_tflops"], 3), impl="cublas" if args.cublas else "uccl")
    elif args.case == "add_norm":
        from unified_ccl_b200 import Communicator
        from unified_ccl_b200.parallel import allreduce_residual_rmsnorm

        comm = Communicator(0, 1)
        x = torch.randn(args.tokens, args.hidden, device=dev).to(torch.bfloat16)
        res = torch.randn(args.tokens, args.hidden, device=dev).to(torch.bfloat16)
        gamma = torch.ones(args.hidden, device=dev, dtype=torch.bfloat16)
        o = torch.empty_like(x)
        ro = torch.empty_like(x)
        t = device_time_ms(lambda: allreduce_residual_rmsnorm(comm, x, res, gamma, 1e-6, out=o, residual_out=ro), args.iters, args.warmup)
        nbytes = 4.0 * x.numel() * 2
        out.update(tokens=args.tokens, hidden=args.hidden, ms=round(t["median"], 4), gbs=round(nbytes / t["median"] / 1e6, 1),
                   frac_of_copy_bw=round(nbytes / t["median"] / 1e6 / peaks["hbm_gbs"], 3))
        comm.destroy()
    elif args.case == "moe_dispatch":
        from unified_ccl_b200 import Communicator
        from unified_ccl_b200.parallel import MoeDispatcher

        comm = Communicator(0, 1)
        disp = MoeDispatcher(comm, args.tokens, args.hidden, args.experts, args.topk)
        x = torch.randn(args.tokens, args.hidden, device=dev).to(torch.bfloat16)
        idx = torch.randn(args.tokens, args.experts, device=dev).topk(args.topk, dim=-1).indices.to(torch.int32).contiguous()
        t = device_time_ms(lambda: disp.dispatch(x, idx), args.iters, args.warmup)
        nbytes = x.numel() * 2 + args.tokens * args.topk * (args.hidden + args.hidden // 32 + 16)
        out.update(tokens=args.tokens, hidden=args.hidden, topk=args.topk, ms=round(t["median"], 4),
                   gbs=round(nbytes / t["median"] / 1e6, 1), frac_of_copy_bw=round(nbytes / t["median"] / 1e6 / peaks["hbm_gbs"], 3))
        disp.close()
        comm.destroy()
    elif args.case == "moe_combine":
        from unified_ccl_b200 import Communicator
        from unified_ccl_b200.parallel import MoeDispatcher

        comm = Communicator(0, 1)
        disp = MoeDispatcher(comm, args.tokens, args.hidden, args.experts, args.topk)
        x = torch.randn(args.tokens, args.hidden, device=dev).to(torch.bfloat16)
        w, idx = torch.softmax(torch.randn(args.tokens, args.experts, device=dev), -1).topk(args.topk, dim=-1)
        disp.dispatch(x, idx.to(torch.int32).contiguous())
        disp.expert_out.normal_()
        y = torch.empty(args.tokens, args.hidden, device=dev, dtype=torch.bfloat16)
        wf = w.float().contiguous()
        t = device_time_ms(lambda: disp.combine(wf, out=y), args.iters, args.warmup)
        nbytes = args.tokens * args.topk * args.hidden * 2 + y.numel() * 2
        out.update(tokens=args.tokens, hidden=args.hidden, topk=args.topk, ms=round(t["median"], 4),
                   gbs=round(nbytes / t["median"] / 1e6, 1), frac_of_copy_bw=round(nbytes / t["median"] / 1e6 / peaks["hbm_gbs"], 3))
        disp.close()
        comm.destroy()
    elif args.case in ("gemm_rs_self", "ag_gemm_self"):
        # the fused tensor-parallel kernels on a one-rank communicator: tiles are staged and
        # summed (reduce-scatter) or flagged (all-gather) exactly as with peers, all on this GPU
        os.environ["UCCL_FUSED_SELF"] = "1"
        from unified_ccl_b200 import Communicator
        from unified_ccl_b200.parallel import allgather_gemm, gemm_reduce_scatter

        comm = Communicator(0, 1)
        a = torch.randn(args.m, args.k, device=dev).to(torch.bfloat16)
        b = (torch.randn(args.n, args.k, device=dev) * 0.02).to(torch.bfloat16)
        if args.case == "gemm_rs_self":
            stage = comm.empty((args.m, args.n), torch.bfloat16)
            y = torch.empty(args.m, args.n, device=dev, dtype=torch.bfloat16)
            fn = lambda: gemm_reduce_scatter(comm, a, b, stage, out=y)  # noqa: E731
        else:
            full = comm.empty((args.m, args.k), torch.bfloat16)
            y = torch.empty(args.m, args.n, device=dev, dtype=torch.bfloat16)
            fn = lambda: allgather_gemm(comm, a, full, b, out=y)  # noqa: E731
        fn()
        torch.cuda.synchronize()
        ref = a.float() @ b.float().t()
        err = float((y.float() - ref).abs().max() / ref.abs().max())
        t = device_time_ms(fn, args.iters, args.warmup)
        flops = 2.0 * args.m * args.n * args.k
        out.update(m=args.m, n=args.n, k=args.k, ms=round(t["median"], 4), tflops=round(flops / t["median"] / 1e9, 1),
                   max_rel_err=round(err, 5), debug=os.environ.get("UCCL_FUSED_DEBUG", "0"))
        comm.destroy()
    else:
        raise SystemExit("unknown case " + args.case)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
