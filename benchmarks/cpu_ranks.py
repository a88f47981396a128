"""Config 1 timed: all-reduce (sum, fp32) between CPU ranks through the whole host stack
(bootstrap, proxy threads, FIFOs, network plugin), next to gloo on the same box.

    UCCL_BACKEND=cpu python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29530 benchmarks/cpu_ranks.py [--elements 1048576] [--iters 20]

Host code on both sides, so the clock is the host's (perf_counter around `iters` calls after a
barrier, max over ranks); every figure is taken `--repeat` times and the median and the minimum are
reported, because on a small shared host single runs differ by an order of magnitude.  Rank r holds
values seeded with 1234 + r; the result of the first call is checked against the elementwise sum.
Prints one JSON line per message size on rank 0.
"""
import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--elements", default="1024,65536,1048576,16777216", help="comma list of fp32 element counts per rank")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeat", type=int, default=7)
    args = ap.parse_args()
    os.environ.setdefault("UCCL_BACKEND", "cpu")
    os.environ.setdefault("UCCL_BOOTSTRAP_IFNAME", "lo")
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from unified_ccl_b200 import Communicator

    comm = Communicator(rank, world)

    def timed(fn, iters):
        """(median, minimum) over --repeat runs of the per-call time in microseconds, max over ranks."""
        for _ in range(args.warmup):
            fn()
        runs = []
        for _ in range(args.repeat):
            dist.barrier()
            t0 = time.perf_counter()
            for _ in range(iters):
                fn()
            dt = (time.perf_counter() - t0) / iters
            t = torch.tensor([dt], dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            runs.append(t.item() * 1e6)
        runs.sort()
        return runs[len(runs) // 2], runs[0]

    for count in [int(c) for c in args.elements.split(",")]:
        g = torch.Generator().manual_seed(1234 + rank)
        mine = torch.randn(count, generator=g)
        ref = sum(torch.randn(count, generator=torch.Generator().manual_seed(1234 + r)) for r in range(world))
        x = mine.clone()
        comm.allreduce(x)
        err = (x - ref).abs().max().item()
        iters = args.iters if count <= (1 << 20) else max(3, args.iters // 4)
        y = mine.clone()
        us_ours, min_ours = timed(lambda: comm.allreduce(y), iters)
        z = mine.clone()
        us_gloo, min_gloo = timed(lambda: dist.all_reduce(z), iters)
        if rank == 0:
            nbytes = count * 4
            busf = 2.0 * (world - 1) / world
            print(json.dumps({"bench": "cpu_ranks_allreduce", "n": world, "elements": count, "bytes": nbytes,
                              "max_abs_err_first_call": err, "ours_us": round(us_ours, 1), "gloo_us": round(us_gloo, 1),
                              "ours_min_us": round(min_ours, 1), "gloo_min_us": round(min_gloo, 1),
                              "ours_busbw_gbs": round(nbytes * busf / us_ours / 1e3, 3),
                              "gloo_busbw_gbs": round(nbytes * busf / us_gloo / 1e3, 3),
                              "net": comm.info["net_name"], "proxy_posts": comm.counters()["proxy_posts"]}), flush=True)
    comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
