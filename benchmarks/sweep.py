#!/usr/bin/env python
"""Bus-bandwidth sweep of every collective and algorithm against NCCL on the same GPUs.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        --master-port 29500 benchmarks/sweep.py --out sweep_N.jsonl --tune tune_N.json

Every number is device-timed (CUDA events on the launching stream around `iters` back-to-back
calls, after warm-up, barrier + synchronize on both sides) and is the MAX over ranks.  Bus
bandwidth follows the usual convention: all-reduce bytes * 2(n-1)/n / t, all-gather and
reduce-scatter total bytes * (n-1)/n / t, broadcast and send/recv bytes / t.  Messages up to
--max-bytes; buffers larger than the L2 are their own flush, smaller ones are latency numbers.
The tuner table written by --tune holds, per collective / algorithm / protocol / size, the
measured time and CTA count; load it with UCCL_TUNE_FILE or Communicator.load_tuning().
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
    ap.add_argument("--out", default="")
    ap.add_argument("--tune", default="")
    ap.add_argument("--min-bytes", type=int, default=1 << 10)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--factor", type=int, default=4)
    ap.add_argument("--colls", default="allreduce,allgather,reducescatter,broadcast,sendrecv,alltoall")
    ap.add_argument("--dtypes", default="bf16")
    ap.add_argument("--unregistered", action="store_true", help="also time ordinary (non-symmetric) buffers")
    ap.add_argument("--blocks", default="", help="comma list of CTA counts to try besides the tuner's (two-shot / NVLS, from 256 KiB up)")
    ap.add_argument("--auto-only", action="store_true", help="time NCCL and the tuner's own choice only (e.g. with UCCL_TUNE_FILE set to a table just measured)")
    ap.add_argument("--no-table", action="store_true", help="measure with the built-in priors (UCCL_TUNE_AUTO=0)")
    args = ap.parse_args()

    os.environ.setdefault("UCCL_BOOTSTRAP_IFNAME", "lo")
    if args.no_table:
        os.environ["UCCL_TUNE_AUTO"] = "0"
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from unified_ccl_b200 import Communicator

    comm = Communicator(rank, world)
    nvls = bool(comm.info["nvls"])
    n = world

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, iters, warmup=3):
        for _ in range(warmup):
            fn()
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        barrier()
        t = torch.tensor([s.elapsed_time(e) / iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item() * 1e3  # us

    def iters_for(nbytes):
        return 100 if nbytes <= (64 << 10) else (40 if nbytes <= (4 << 20) else (10 if nbytes <= (256 << 20) else 4))

    dts = {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}
    sizes = []
    b = args.min_bytes
    while b <= args.max_bytes:
        sizes.append(b)
        b *= args.factor
    results, tune = [], []
    env_blocks = [int(x) for x in args.blocks.split(",") if x]

    def record(coll, impl, algo, proto, dt, nbytes, us, busf, registered, blocks=0):
        row = {"coll": coll, "impl": impl, "algo": algo, "proto": proto, "dtype": dt, "bytes": nbytes, "us": round(us, 2),
               "busbw_gbs": round(nbytes * busf / (us * 1e-6) / 1e9, 2), "n": n, "registered": registered, "blocks": blocks}
        if impl == "uccl" and algo == "auto" and coll != "sendrecv":
            row["chosen"] = "%s/%s/%d" % comm.query_tuning(coll, nbytes, registered)  # what the tuner ran
        results.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
        if impl == "uccl" and registered and algo != "auto":
            tune.append({"coll": coll, "algo": algo, "proto": proto, "bytes": nbytes, "us": round(us, 3), "blocks": blocks})

    def uccl_algo(coll, qname, algo, proto, dtn, nbytes, fn, it, busf):
        """Time one (algorithm, protocol) at the tuner's CTA count and, from 256 KiB up, at every count of
        --blocks; every result is recorded, the tuner table keeps the best per size."""
        if args.auto_only:
            return
        comm.set_algo(algo, proto)
        comm.set_blocks(0)
        us = timed(fn, it)
        if nbytes <= (1 << 20):
            us = min(us, timed(fn, it))  # latency-sized messages: one delayed rank must not end up in the table
        record(coll, "uccl", algo, proto, dtn, nbytes, us, busf, True, comm.query_tuning(qname, nbytes, True)[2])
        if nbytes >= (256 << 10) and algo in ("two_shot", "nvls") and proto == "simple":
            for nb in env_blocks:
                comm.set_blocks(nb)
                record(coll, "uccl", algo, proto, dtn, nbytes, timed(fn, max(3, it // 2)), busf, True, nb)
            comm.set_blocks(0)

    for dtn in args.dtypes.split(","):
        dt = dts[dtn]
        es = torch.empty((), dtype=dt).element_size()
        for coll in args.colls.split(","):
            for nbytes in sizes:
                it = iters_for(nbytes)
                if coll == "allreduce":
                    cnt = nbytes // es
                    busf = 2.0 * (n - 1) / n
                    sym = comm.empty(cnt, dt); sym.fill_(1)
                    plain = torch.ones(cnt, dtype=dt, device=dev)
                    record(coll, "nccl", "nccl", "-", dtn, nbytes, timed(lambda: dist.all_reduce(plain), it), busf, False)
                    combos = [("one_shot", "ll"), ("one_shot", "simple"), ("two_shot", "simple"), ("ring", "simple"),
                              ("ring", "ll128"), ("copy_engine", "simple")]
                    if nvls:
                        combos.insert(3, ("nvls", "simple"))
                    for algo, proto in combos:
                        if proto == "ll" and nbytes > 65536:
                            continue
                        if proto == "ll128" and nbytes > 65536:
                            continue  # the tuner refuses it above the packet capacity and would time its own choice instead
                        if algo == "one_shot" and proto == "simple" and nbytes > (16 << 20):
                            continue
                        if algo == "copy_engine" and nbytes < (1 << 20):
                            continue
                        uccl_algo(coll, "allreduce", algo, proto, dtn, nbytes, lambda: comm.allreduce(sym), it, busf)
                        if args.unregistered and algo in ("two_shot", "nvls", "one_shot"):
                            record(coll, "uccl", algo, proto, dtn, nbytes, timed(lambda: comm.allreduce(plain), it), busf, False)
                    comm.set_algo("auto", "auto")
                    record(coll, "uccl", "auto", "auto", dtn, nbytes, timed(lambda: comm.allreduce(sym), it), busf, True)
                    comm.free(sym)
                elif coll in ("allgather", "reducescatter"):
                    cnt = max(1, nbytes // es // n)  # per-rank chunk; nbytes is the total
                    busf = (n - 1) / n
                    big_sym = comm.empty(cnt * n, dt); big_sym.fill_(1)
                    small = torch.ones(cnt, dtype=dt, device=dev)
                    big = torch.ones(cnt * n, dtype=dt, device=dev)
                    if coll == "allgather":
                        record(coll, "nccl", "nccl", "-", dtn, nbytes, timed(lambda: dist.all_gather_into_tensor(big, small), it), busf, False)
                        for algo in (["nvls"] if nvls else []) + ["two_shot", "ring", "copy_engine"]:
                            if algo == "copy_engine" and nbytes < (1 << 20):
                                continue
                            uccl_algo(coll, "allgather", algo, "simple", dtn, nbytes, lambda: comm.allgather(small, big_sym), it, busf)
                        if cnt * es <= 65536:  # low-latency packets: up to 64 KiB per rank
                            uccl_algo(coll, "allgather", "one_shot", "ll", dtn, nbytes, lambda: comm.allgather(small, big_sym), it, busf)
                        if args.unregistered:
                            comm.set_algo("auto", "auto")
                            record(coll, "uccl", "auto", "auto", dtn, nbytes, timed(lambda: comm.allgather(small, big), it), busf, False)
                    else:
                        record(coll, "nccl", "nccl", "-", dtn, nbytes, timed(lambda: dist.reduce_scatter_tensor(small, big), it), busf, False)
                        for algo in (["nvls"] if nvls else []) + ["two_shot", "ring", "copy_engine"]:
                            if algo == "copy_engine" and nbytes < (1 << 20):
                                continue
                            uccl_algo(coll, "reducescatter", algo, "simple", dtn, nbytes, lambda: comm.reduce_scatter(big_sym, small), it, busf)
                        if cnt * es <= 65536:
                            uccl_algo(coll, "reducescatter", "one_shot", "ll", dtn, nbytes, lambda: comm.reduce_scatter(big_sym, small), it, busf)
                        if args.unregistered:
                            comm.set_algo("auto", "auto")
                            record(coll, "uccl", "auto", "auto", dtn, nbytes, timed(lambda: comm.reduce_scatter(big, small), it), busf, False)
                    comm.set_algo("auto", "auto")
                    if coll == "allgather":
                        record(coll, "uccl", "auto", "auto", dtn, nbytes, timed(lambda: comm.allgather(small, big_sym), it), busf, True)
                    else:
                        record(coll, "uccl", "auto", "auto", dtn, nbytes, timed(lambda: comm.reduce_scatter(big_sym, small), it), busf, True)
                    comm.free(big_sym)
                elif coll == "broadcast":
                    cnt = nbytes // es
                    sym = comm.empty(cnt, dt); sym.fill_(1)
                    plain = torch.ones(cnt, dtype=dt, device=dev)
                    record(coll, "nccl", "nccl", "-", dtn, nbytes, timed(lambda: dist.broadcast(plain, 0), it), 1.0, False)
                    for algo in (["nvls"] if nvls else []) + ["two_shot"]:
                        uccl_algo(coll, "broadcast", algo, "simple", dtn, nbytes, lambda: comm.broadcast(sym, 0), it, 1.0)
                    comm.set_algo("auto", "auto")
                    record(coll, "uccl", "auto", "auto", dtn, nbytes, timed(lambda: comm.broadcast(sym, 0), it), 1.0, True)
                    comm.free(sym)
                elif coll == "alltoall":
                    cnt = max(1, nbytes // es // n)
                    sym = comm.empty(cnt * n, dt); sym.fill_(1)
                    dst = torch.empty(cnt * n, dtype=dt, device=dev)
                    src = torch.ones(cnt * n, dtype=dt, device=dev)
                    record(coll, "nccl", "nccl", "-", dtn, nbytes, timed(lambda: dist.all_to_all_single(dst, src), it), (n - 1) / n, False)
                    uccl_algo(coll, "alltoall", "two_shot", "simple", dtn, nbytes, lambda: comm.alltoall(sym, dst), it, (n - 1) / n)
                    if cnt * es <= 65536:  # low-latency packets: up to 64 KiB per rank
                        uccl_algo(coll, "alltoall", "one_shot", "ll", dtn, nbytes, lambda: comm.alltoall(sym, dst), it, (n - 1) / n)
                    comm.set_algo("auto", "auto")
                    record(coll, "uccl", "auto", "auto", dtn, nbytes, timed(lambda: comm.alltoall(sym, dst), it), (n - 1) / n, True)
                    comm.free(sym)
                elif coll == "sendrecv":
                    cnt = nbytes // es
                    s_t = torch.ones(cnt, dtype=dt, device=dev)
                    r_t = torch.empty(cnt, dtype=dt, device=dev)
                    nxt, prv = (rank + 1) % n, (rank - 1) % n

                    def nccl_sr():
                        ops = [dist.P2POp(dist.isend, s_t, nxt), dist.P2POp(dist.irecv, r_t, prv)]
                        for w in dist.batch_isend_irecv(ops):
                            w.wait()

                    def uccl_sr():
                        with comm.group():
                            comm.send(s_t, nxt)
                            comm.recv(r_t, prv)

                    record(coll, "nccl", "nccl", "-", dtn, nbytes, timed(nccl_sr, it), 1.0, False)
                    record(coll, "uccl", "auto", "simple", dtn, nbytes, timed(uccl_sr, it), 1.0, False)

    if rank == 0:
        if args.out:
            with open(args.out, "w") as f:
                for r in results:
                    f.write(json.dumps(r) + "\n")
        if args.tune:
            with open(args.tune, "w") as f:
                json.dump({"version": 1, "nranks": n, "gpu": torch.cuda.get_device_name(dev), "nvls": nvls,
                           "note": "symmetric buffers, device-timed max over ranks, benchmarks/sweep.py --tune",
                           "entries": tune}, f, indent=0)
    barrier()
    comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
