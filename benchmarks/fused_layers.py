#!/usr/bin/env python
"""Device-timed comparison of the fused kernels against their library baselines, one JSON line each:

  * all-reduce + residual + RMSNorm  (tokens x hidden bf16)  vs NCCL all-reduce + a separate norm kernel
  * MoE dispatch (bf16 -> fp8 e4m3, 1x128 scales) and weighted combine vs NCCL all-to-all + cast / sum kernels
  * one-sided put+signal ping-pong latency vs NCCL send/recv ping-pong

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        --master-port 29500 benchmarks/fused_layers.py --what norm,moe,rma   (add norm_breakdown for the phases of the norm kernel)

Times are CUDA-event times on the launching stream, max over ranks, after warm-up.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="norm,moe,rma")
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--moe-tokens", type=int, default=4096)
    ap.add_argument("--moe-hidden", type=int, default=7168)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    os.environ.setdefault("UCCL_BOOTSTRAP_IFNAME", "lo")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from unified_ccl_b200 import Communicator, Window
    from unified_ccl_b200.parallel import MoeDispatcher, allreduce_residual_rmsnorm, autotune_allreduce_residual_rmsnorm

    comm = Communicator(rank, world)
    n = world

    def timed(fn, iters=args.iters, warmup=5):
        for _ in range(warmup):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        dist.barrier()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item() * 1e3

    def emit(d):
        if rank == 0:
            print(json.dumps(d), flush=True)

    what = args.what.split(",")
    if "norm" in what:
        T, H = args.tokens, args.hidden
        g = torch.Generator(device="cpu").manual_seed(100 + rank)
        x = comm.empty((T, H), torch.bfloat16)
        x.copy_(torch.randn(T, H, generator=g).to(torch.bfloat16))
        res = comm.empty((T, H), torch.bfloat16)
        res.copy_(torch.randn(T, H, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16))
        gamma = (1 + 0.02 * torch.randn(H, generator=torch.Generator().manual_seed(8))).to(torch.bfloat16).to(dev)
        out = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
        xn = x.clone()
        rn = res.clone()

        def baseline():
            dist.all_reduce(xn)
            h = xn + rn
            rn.copy_(h)
            return torch.nn.functional.rms_norm(h, (H,), gamma, 1e-6)

        # untimed: pick the shape of the kernel's switch path on this box (same on every rank)
        shapes = autotune_allreduce_residual_rmsnorm(comm, x, res, gamma, 1e-6, out=out)
        us_f = timed(lambda: allreduce_residual_rmsnorm(comm, x, res, gamma, 1e-6, out=out, residual_out=res))
        us_b = timed(baseline)
        msg = T * H * 2
        roof = max((n - 1) / n * msg * 2 / 770e9, 4 * msg / 6549e9) * 1e6 if n > 1 else 4 * msg / 6549e9 * 1e6
        roof_nvls = max(msg / 770e9, 4 * msg / 6549e9) * 1e6
        emit({"bench": "allreduce_residual_rmsnorm", "n": n, "tokens": T, "hidden": H, "fused_us": round(us_f, 1),
              "nccl_plus_norm_us": round(us_b, 1), "speedup": round(us_b / us_f, 3), "roofline_ring_us": round(roof, 1),
              "roofline_switch_us": round(roof_nvls, 1), "frac_of_ring_roofline": round(roof / us_f, 3), "nvls": comm.info["nvls"],
              "autotune_rows_us": {str(k): v for k, v in shapes.items()}})
        if "norm_breakdown" in what and n > 1:
            # the same kernel with a phase left out (UCCL_NORM_DEBUG), and the two data paths
            parts = {}
            for bits, name in ((1, "no_phase_b"), (2, "no_phase_a_stores"), (3, "loads_only"), (4, "phase_b_only")):
                os.environ["UCCL_NORM_DEBUG"] = str(bits)
                parts[name] = round(timed(lambda: allreduce_residual_rmsnorm(comm, x, res, gamma, 1e-6, out=out, residual_out=res)), 1)
            os.environ["UCCL_NORM_DEBUG"] = "0"
            for rows in (0, 1, 2, 4):  # switch path: 0 = own rows normalised from registers; else rows per pass of the all-reduce phase
                os.environ["UCCL_NORM_MC_ROWS"] = str(rows)
                parts["mc_rows_%d" % rows] = round(timed(lambda: allreduce_residual_rmsnorm(comm, x, res, gamma, 1e-6, out=out, residual_out=res)), 1)
            os.environ.pop("UCCL_NORM_MC_ROWS", None)
            for algo in ("nvls", "two_shot"):
                if algo == "nvls" and not comm.info["nvls"]:
                    continue
                comm.set_algo(algo)
                parts["path_" + algo] = round(timed(lambda: allreduce_residual_rmsnorm(comm, x, res, gamma, 1e-6, out=out, residual_out=res)), 1)
            comm.set_algo("auto")
            parts["allreduce_same_bytes"] = round(timed(lambda: comm.allreduce(x)), 1)
            parts["nccl_allreduce_same_bytes"] = round(timed(lambda: dist.all_reduce(xn)), 1)
            emit({"bench": "allreduce_residual_rmsnorm_breakdown", "n": n, "tokens": T, "hidden": H, "us": parts})
        comm.free(x)
        comm.free(res)

    if "moe" in what and n > 1:
        T, H, E, K = args.moe_tokens, args.moe_hidden, args.experts, args.topk
        disp = MoeDispatcher(comm, T, H, E, K)
        g = torch.Generator(device="cpu").manual_seed(500 + rank)
        x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev)
        w, idx = torch.softmax(torch.randn(T, E, generator=g), -1).topk(K, dim=-1)
        idx = idx.to(torch.int32).to(dev).contiguous()
        w = w.float().to(dev).contiguous()
        us_d = timed(lambda: disp.dispatch(x, idx))
        disp.expert_out.normal_()
        outc = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
        us_c = timed(lambda: disp.combine(w, out=outc))
        # library baseline: cast kernel + NCCL all-to-all of equal splits of the same volume, and back
        rows = T * K
        per = (rows // n) * n
        send8 = torch.empty(per, H, device=dev, dtype=torch.uint8)
        recv8 = torch.empty(per, H, device=dev, dtype=torch.uint8)
        sends = torch.empty(per, H // 128, device=dev, dtype=torch.float32)
        recvs = torch.empty(per, H // 128, device=dev, dtype=torch.float32)
        flat = idx.view(-1).long()
        order = torch.argsort(flat)[:per]
        tok = (order // K)

        def base_dispatch():
            xs = x[tok].float().view(per, H // 128, 128)
            sc = xs.abs().amax(-1).clamp_min(1e-10) / 448.0
            q = (xs / sc.unsqueeze(-1)).to(torch.float8_e4m3fn).view(per, H).view(torch.uint8)
            dist.all_to_all_single(recv8, q)
            dist.all_to_all_single(recvs, sc)

        y16 = torch.randn(per, H, device=dev).to(torch.bfloat16)
        back = torch.empty(per, H, device=dev, dtype=torch.bfloat16)
        wflat = w.view(-1)[order].unsqueeze(-1)

        def base_combine():
            dist.all_to_all_single(back, y16)
            o = torch.zeros(T, H, device=dev, dtype=torch.float32)
            o.index_add_(0, tok, back.float() * wflat)
            return o.to(torch.bfloat16)

        us_bd = timed(base_dispatch)
        us_bc = timed(base_combine)
        remote = (n - 1) / n
        bytes_d = rows * remote * (H + H // 128 * 4 + 16)
        bytes_c = rows * remote * H * 2
        emit({"bench": "moe_dispatch", "n": n, "tokens": T, "hidden": H, "experts": E, "topk": K, "fused_us": round(us_d, 1),
              "nccl_a2a_plus_cast_us": round(us_bd, 1), "speedup": round(us_bd / us_d, 3),
              "roofline_us": round(bytes_d / 770e9 * 1e6, 1), "frac_of_roofline": round(bytes_d / 770e9 * 1e6 / us_d, 3)})
        emit({"bench": "moe_combine", "n": n, "tokens": T, "hidden": H, "experts": E, "topk": K, "fused_us": round(us_c, 1),
              "nccl_a2a_plus_sum_us": round(us_bc, 1), "speedup": round(us_bc / us_c, 3),
              "roofline_us": round(bytes_c / 770e9 * 1e6, 1), "frac_of_roofline": round(bytes_c / 770e9 * 1e6 / us_c, 3)})
        disp.close()

    if "rma" in what and n > 1:
        peer = rank ^ 1
        active = peer < n
        buf = comm.empty(1 << 20, torch.uint8)
        buf.zero_()
        torch.cuda.synchronize()
        win = Window(comm, buf)
        count = [0]
        for nbytes in (8, 64, 512, 4096, 32768, 262144, 1048576):
            src = torch.ones(nbytes, dtype=torch.uint8, device=dev)
            rcv = torch.empty(nbytes, dtype=torch.uint8, device=dev)

            def pingpong():
                # even ranks put first, odd ranks answer: one round trip per call
                if not active:
                    return
                count[0] += 1
                if rank % 2 == 0:
                    win.put_signal(src, peer)
                    win.wait_signal(peer, count[0])
                else:
                    win.wait_signal(peer, count[0])
                    win.put_signal(src, peer)

            def nccl_pingpong():
                if not active:
                    return
                if rank % 2 == 0:
                    dist.send(src, peer)
                    dist.recv(rcv, peer)
                else:
                    dist.recv(rcv, peer)
                    dist.send(src, peer)

            us_r = timed(pingpong, iters=50)
            us_n = timed(nccl_pingpong, iters=50)
            emit({"bench": "rma_pingpong", "n": n, "bytes": nbytes, "put_signal_round_trip_us": round(us_r, 2),
                  "nccl_sendrecv_round_trip_us": round(us_n, 2), "one_way_us": round(us_r / 2, 2)})
        win.close()
        comm.free(buf)

    dist.barrier()
    comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
