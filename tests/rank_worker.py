"""One rank of a multi-process test.  Usage: rank_worker.py <case> <rank> <nranks> <idfile> [args...]

Prints a single line "RESULT <json>".  Cases are functions named case_<name> below; each gets
(comm, rank, nranks, args) and returns a dict.  A non-empty "fail" list marks a failed check.
"""
import json
import os
import sys
import time
import traceback

import torch


def _uid(rank, idfile, create=True):
    from unified_ccl_b200 import get_unique_id

    if rank == 0 and create:
        uid = get_unique_id()
        with open(idfile + ".tmp", "wb") as f:
            f.write(uid)
        os.rename(idfile + ".tmp", idfile)
        return uid
    t0 = time.time()
    while not os.path.exists(idfile):
        if time.time() - t0 > 60:
            raise RuntimeError("unique id file never appeared")
        time.sleep(0.01)
    with open(idfile, "rb") as f:
        return f.read()


def _seeded(count, seed, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.rand(count, generator=g) * 2 - 1).to(dtype)


def _dev(comm, rank):
    return torch.device("cuda", comm.info["cuda_device"]) if comm.on_gpu else torch.device("cpu")


def _sync(comm):
    if comm.on_gpu:
        torch.cuda.synchronize()


# ---------------------------------------------------------------------------- cases
def case_allreduce_config1(comm, rank, n, args):
    """fp32, 1,048,576 elements per rank, rank r seeded with 1234 + r, exact elementwise sum."""
    count = 1048576
    x = _seeded(count, 1234 + rank).to(_dev(comm, rank))
    ref = sum(_seeded(count, 1234 + r) for r in range(n))
    t0 = time.time()
    comm.allreduce(x)
    _sync(comm)
    dt = time.time() - t0
    err = (x.cpu() - ref).abs().max().item()
    tol = 0.0 if n == 2 else 1e-5
    return {"err": err, "seconds": dt, "fail": [] if err <= tol else [("allreduce", err)],
            "proxy_posts": comm.counters()["proxy_posts"], "net": comm.info["net_name"]}


def _collective_matrix(comm, rank, n, counts, dtypes, sym=False, inplace_ag=True):
    dev = _dev(comm, rank)
    fail = []

    def mk(numel, dt):
        return comm.empty(numel, dt) if sym else torch.empty(numel, dtype=dt, device=dev)

    for dt in dtypes:
        tol = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 2e-3}[dt] * n
        for cnt in counts:
            # all-reduce, in place and out of place
            xs = [_seeded(cnt, 1234 + r, dt) for r in range(n)]
            ref = sum(x.float() for x in xs)
            x = mk(cnt, dt)
            x.copy_(xs[rank])
            comm.allreduce(x)
            _sync(comm)
            e = (x.float().cpu() - ref).abs().max().item() if cnt else 0.0
            if e > tol:
                fail.append(("allreduce", str(dt), cnt, e))
            src = xs[rank].to(dev)
            out = mk(cnt, dt)
            comm.allreduce(src, out=out)
            _sync(comm)
            e = (out.float().cpu() - ref).abs().max().item() if cnt else 0.0
            if e > tol or not torch.equal(src.cpu(), xs[rank]):
                fail.append(("allreduce_oop", str(dt), cnt, e))
            # all-gather
            s = torch.full((cnt,), float(rank + 1), dtype=dt, device=dev)
            r = mk(cnt * n, dt)
            comm.allgather(s, r)
            _sync(comm)
            exp = torch.cat([torch.full((cnt,), float(p + 1)) for p in range(n)]) if cnt else torch.empty(0)
            if not torch.equal(r.float().cpu(), exp):
                fail.append(("allgather", str(dt), cnt))
            # reduce-scatter
            full = [_seeded(cnt * n, 99 + p, dt) for p in range(n)]
            s2 = mk(cnt * n, dt)
            s2.copy_(full[rank])
            r2 = torch.empty(cnt, dtype=dt, device=dev)
            comm.reduce_scatter(s2, r2)
            _sync(comm)
            exp2 = sum(f.float() for f in full)[rank * cnt:(rank + 1) * cnt]
            e = (r2.float().cpu() - exp2).abs().max().item() if cnt else 0.0
            if e > tol:
                fail.append(("reduce_scatter", str(dt), cnt, e))
            # broadcast from the last rank
            b = mk(cnt, dt)
            b.fill_(float(rank))
            comm.broadcast(b, root=n - 1)
            _sync(comm)
            if cnt and not (b.float().cpu() == n - 1).all():
                fail.append(("broadcast", str(dt), cnt))
            # reduce to rank 0
            rd = mk(cnt, dt)
            rd.copy_(xs[rank])
            out2 = torch.zeros(cnt, dtype=dt, device=dev)
            comm.reduce(rd, out2, root=0)
            _sync(comm)
            if rank == 0 and cnt:
                e = (out2.float().cpu() - ref).abs().max().item()
                if e > tol:
                    fail.append(("reduce", str(dt), cnt, e))
            # all-to-all
            if cnt:
                a = mk(cnt * n, dt)
                a.copy_((torch.arange(n * cnt) % 251 + rank).to(dt))
                a2 = torch.empty(cnt * n, dtype=dt, device=dev)
                comm.alltoall(a, a2)
                _sync(comm)
                exp3 = torch.cat([(torch.arange(rank * cnt, (rank + 1) * cnt) % 251 + p).to(dt) for p in range(n)])
                if not torch.equal(a2.cpu(), exp3):
                    fail.append(("alltoall", str(dt), cnt))
    return fail


def case_collectives_small(comm, rank, n, args):
    fail = _collective_matrix(comm, rank, n, [0, 1, 3, 257, 70001], [torch.float32, torch.bfloat16, torch.float16])
    return {"fail": fail, "algo_hist": comm.counters()["algo_hist"]}


def case_collectives_symmetric(comm, rank, n, args):
    fail = _collective_matrix(comm, rank, n, [8, 4096, 70001, 1 << 20], [torch.bfloat16, torch.float32], sym=True)
    return {"fail": fail, "nvls": comm.info["nvls"]}


def case_allreduce_algos(comm, rank, n, args):
    dev = _dev(comm, rank)
    fail = []
    combos = [("one_shot", "ll"), ("one_shot", "simple"), ("two_shot", "simple"), ("nvls", "simple"),
              ("ring", "simple"), ("ring", "ll128"), ("copy_engine", "simple")]
    for dt in (torch.bfloat16, torch.float32, torch.float16):
        tol = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 2e-3}[dt] * n
        es = torch.empty((), dtype=dt).element_size()
        for cnt in (1, 7, 1000, 4096, 65536 + 3, 1 << 20):
            xs = [_seeded(cnt, 1234 + r, dt) for r in range(n)]
            ref = sum(x.float() for x in xs)
            for algo, proto in combos:
                if proto == "ll" and cnt * es > 65536:
                    continue
                for sym in (False, True):
                    comm.set_algo(algo, proto)
                    x = comm.empty(cnt, dt) if sym else torch.empty(cnt, dtype=dt, device=dev)
                    x.copy_(xs[rank])
                    comm.allreduce(x)
                    _sync(comm)
                    e = (x.float().cpu() - ref).abs().max().item()
                    if e > tol:
                        fail.append((algo, proto, str(dt), cnt, sym, e))
                    if sym:
                        comm.free(x)
    comm.set_algo("auto", "auto")
    return {"fail": fail, "algo_hist": comm.counters()["algo_hist"], "nvls": comm.info["nvls"]}


def case_ring_ce_matrix(comm, rank, n, args):
    """All-gather, reduce-scatter and all-reduce forced onto the ring (Simple and LL128), onto the
    copy engines and onto the low-latency packets, out of place and in place.  Run with a small UCCL_STAGING_BYTES and few CTAs so that
    one chunk needs more pieces than a channel has slots (several rounds of the reduce-scatter
    schedule, FIFO wrap-around) and the copy-engine path loops over its staging area."""
    dev = _dev(comm, rank)
    fail = []
    # one_shot / ll: the packet form of all three (chunks up to 64 KiB; larger ones take the direct kernels)
    # two_shot / one_shot: the direct kernels, which with this staging area move a few MiB of ordinary
    # (not symmetric) memory in several pieces
    combos = [("ring", "simple"), ("ring", "ll128"), ("copy_engine", "simple"), ("one_shot", "ll"),
              ("two_shot", "simple"), ("one_shot", "simple")]
    for dt in (torch.float32, torch.bfloat16):
        tol = {torch.float32: 1e-5, torch.bfloat16: 2e-2}[dt] * n
        for cnt in (5, 4099, (1 << 20) + 3):
            mine = _seeded(cnt, 300 + rank, dt)
            full = [_seeded(cnt * n, 99 + p, dt) for p in range(n)]
            exp_ag = torch.cat([_seeded(cnt, 300 + p, dt) for p in range(n)])
            exp_rs = sum(f.float() for f in full)[rank * cnt:(rank + 1) * cnt]
            exp_ar = sum(_seeded(cnt, 300 + p, dt).float() for p in range(n))
            for algo, proto in combos:
                if proto == "ll128" and cnt > (1 << 18):
                    continue  # 112 payload bytes per 128-byte line: keep the slow protocol to small messages
                comm.set_algo(algo, proto)
                # all-gather, out of place then in place (my part already sits in the output)
                r = torch.zeros(cnt * n, dtype=dt, device=dev)
                comm.allgather(mine.to(dev), r)
                _sync(comm)
                if not torch.equal(r.cpu(), exp_ag):
                    fail.append(("allgather", algo, proto, str(dt), cnt))
                r2 = torch.zeros(cnt * n, dtype=dt, device=dev)
                r2[rank * cnt:(rank + 1) * cnt] = mine.to(dev)
                comm.allgather(r2[rank * cnt:(rank + 1) * cnt], r2)
                _sync(comm)
                if not torch.equal(r2.cpu(), exp_ag):
                    fail.append(("allgather_inplace", algo, proto, str(dt), cnt))
                # reduce-scatter, out of place then in place (output = my part of the input)
                s2 = full[rank].to(dev)
                o = torch.zeros(cnt, dtype=dt, device=dev)
                comm.reduce_scatter(s2, o)
                _sync(comm)
                e = (o.float().cpu() - exp_rs).abs().max().item()
                if e > tol:
                    fail.append(("reduce_scatter", algo, proto, str(dt), cnt, e))
                s3 = full[rank].to(dev)
                comm.reduce_scatter(s3, s3[rank * cnt:(rank + 1) * cnt])
                _sync(comm)
                e = (s3[rank * cnt:(rank + 1) * cnt].float().cpu() - exp_rs).abs().max().item()
                if e > tol:
                    fail.append(("reduce_scatter_inplace", algo, proto, str(dt), cnt, e))
                x = mine.to(dev)
                comm.allreduce(x)
                _sync(comm)
                e = (x.float().cpu() - exp_ar).abs().max().item()
                if e > tol:
                    fail.append(("allreduce", algo, proto, str(dt), cnt, e))
    comm.set_algo("auto", "auto")
    return {"fail": fail, "algo_hist": comm.counters()["algo_hist"]}


def case_fused_cast(comm, rank, n, args):
    """Reduce-scatter / all-reduce with scale and a different output type against the fp32 restatement:
    bf16 -> fp32, bf16 -> bf16, fp32 -> bf16, fp16 -> fp16, and bf16 / fp32 -> fp8-e4m3 with 1 x 128 scales;
    symmetric and ordinary input buffers (the latter in several staged pieces)."""
    from unified_ccl_b200.parallel import quantize_fp8_block128

    dev = _dev(comm, rank)
    fail = []
    f8 = torch.float8_e4m3fn
    pairs = [(torch.bfloat16, torch.float32), (torch.bfloat16, torch.bfloat16), (torch.float32, torch.bfloat16),
             (torch.float16, torch.float16), (torch.bfloat16, f8), (torch.float32, f8)]
    for per in (128, 5 * 128, 3 * 4096 + 128, 1 << 19):
        for din, dout in pairs:
            for sym in (True, False):
                scale = 0.37
                full = [_seeded(per * n, 700 + p, din) for p in range(n)]
                tot = sum(f.float() for f in full) * scale
                exp = tot[rank * per:(rank + 1) * per]
                s_in = comm.empty(per * n, din) if sym else torch.empty(per * n, dtype=din, device=dev)
                s_in.copy_(full[rank])
                out = torch.empty(per, dtype=dout, device=dev)
                out, scales = comm.reduce_scatter_cast(s_in, out, scale)
                _sync(comm)
                if dout == f8:
                    q, sc = quantize_fp8_block128(exp.view(1, -1))
                    deq = out.float().cpu().view(-1, 128) * scales.cpu().view(-1, 1)
                    ref = q.float().view(-1, 128) * sc.view(-1, 1)
                    # a sum that differs in the last fp32 bit can move an element across one fp8 step
                    amax = exp.view(-1, 128).abs().amax(-1, keepdim=True)
                    bad = ((deq - ref).abs() > 0.0625 * amax + 1e-6).sum().item()
                    if bad or not torch.allclose(scales.cpu(), sc.view(-1), rtol=1e-5, atol=0):
                        fail.append(("rs_fp8", str(din), per, sym, bad))
                else:
                    tol = {torch.float32: 2e-6, torch.bfloat16: 8e-3, torch.float16: 1e-3}[dout] * max(1.0, exp.abs().max().item())
                    e = (out.float().cpu() - exp).abs().max().item()
                    if e > tol:
                        fail.append(("rs_cast", str(din), str(dout), per, sym, e))
                # all-reduce form on the same data
                o2 = torch.empty(per * n, dtype=dout, device=dev)
                o2, sc2 = comm.allreduce_cast(s_in, o2, scale)
                _sync(comm)
                if dout == f8:
                    deq = o2.float().cpu().view(-1, 128) * sc2.cpu().view(-1, 1)
                    amax = tot.view(-1, 128).abs().amax(-1, keepdim=True)
                    bad = ((deq - tot.view(-1, 128)).abs() > 0.07 * amax + 1e-6).sum().item()
                    if bad:
                        fail.append(("ar_fp8", str(din), per, sym, bad))
                else:
                    tol = {torch.float32: 2e-6, torch.bfloat16: 8e-3, torch.float16: 1e-3}[dout] * max(1.0, tot.abs().max().item())
                    e = (o2.float().cpu() - tot).abs().max().item()
                    if e > tol:
                        fail.append(("ar_cast", str(din), str(dout), per, sym, e))
                if sym:
                    comm.free(s_in)
    return {"fail": fail}


def case_sendrecv(comm, rank, n, args):
    dev = _dev(comm, rank)
    fail = []
    for cnt in (5, 1 << 18, (5 << 20) + 77):
        s = torch.full((cnt,), float(rank), device=dev)
        r = torch.empty(cnt, device=dev)
        with comm.group():
            comm.send(s, (rank + 1) % n)
            comm.recv(r, (rank - 1) % n)
        _sync(comm)
        if not (r.cpu() == (rank - 1) % n).all():
            fail.append(("ring_exchange", cnt))
    # ungrouped pair: even ranks send first, odd ranks receive first
    if n % 2 == 0:
        peer = rank ^ 1
        s = torch.arange(1000, dtype=torch.float32, device=dev) + rank
        r = torch.empty(1000, device=dev)
        if rank % 2 == 0:
            comm.send(s, peer)
            comm.recv(r, peer)
        else:
            comm.recv(r, peer)
            comm.send(s, peer)
        _sync(comm)
        if not torch.equal(r.cpu(), torch.arange(1000, dtype=torch.float32) + peer):
            fail.append(("pair",))
    # two sends and two receives with the same peer in one group share a FIFO and keep their order;
    # a long group (more operations per peer than one launch carries) is cut at the same places on both ends
    for reps, cnt in ((2, 3000), (2, (3 << 20) + 5), (5, 70001)):
        nxt, prv = (rank + 1) % n, (rank - 1) % n
        ss = [torch.full((cnt + i,), float(10 * rank + i), device=dev) for i in range(reps)]
        rr = [torch.empty(cnt + i, device=dev) for i in range(reps)]
        with comm.group():
            for i in range(reps):
                comm.send(ss[i], nxt)
            for i in range(reps):
                comm.recv(rr[i], prv)
        _sync(comm)
        for i in range(reps):
            if not (rr[i].cpu() == 10 * prv + i).all():
                fail.append(("same_peer_twice", reps, cnt, i))
    # send to self inside a group
    s = torch.full((64,), 7.0, device=dev)
    r = torch.zeros(64, device=dev)
    with comm.group():
        comm.send(s, rank)
        comm.recv(r, rank)
    _sync(comm)
    if not (r.cpu() == 7).all():
        fail.append(("self",))
    return {"fail": fail}


def case_api_contract(comm, rank, n, args):
    """The reference's Python test contract (tests/python/test_allreduce.py) on this backend."""
    dev = _dev(comm, rank)
    fail = []
    for dt in (torch.float16, torch.bfloat16, torch.float32):
        for size in (1, 16, 256, 1024, 4096, 65536):
            t = torch.ones(size, dtype=dt, device=dev)
            ptr = t.data_ptr()
            out = comm.allreduce(t)
            _sync(comm)
            if out.data_ptr() != ptr:
                fail.append(("not in place", str(dt), size))
            if not torch.allclose(t.float().cpu(), torch.full((size,), float(n))):
                fail.append(("value", str(dt), size))
    try:
        comm.allreduce(torch.ones(4, dtype=torch.int32, device=dev))
        fail.append(("int32 accepted",))
    except TypeError:
        pass
    try:
        wrong = torch.ones(4, device="cpu" if comm.on_gpu else "meta")
        comm.allreduce(wrong)
        fail.append(("wrong device accepted",))
    except (ValueError, NotImplementedError, RuntimeError):
        pass
    try:
        comm.allgather(torch.ones(4, device=dev), torch.ones(5, device=dev))
        fail.append(("bad allgather size accepted",))
    except ValueError:
        pass
    if comm.rank != rank or comm.world_size != n:
        fail.append(("rank/world_size",))
    # tuning knobs: accepted values stick, out-of-range values are refused
    comm.set_fused_options("kernel", 12, 0)
    comm.set_fused_options("ce", 0, 2)
    comm.set_fused_options()
    for bad in (("ce", 65, 0), ("ce", 0, 65), ("kernel", -1, 0)):
        try:
            comm.set_fused_options(*bad)
            fail.append(("bad fused option accepted", bad))
        except Exception:
            pass
    comm.set_fused_options("spread")
    comm.set_fused_options()
    comm.set_fused_rs_reducers(8)
    comm.set_fused_rs_reducers(0)
    for bad in (65, -1):
        try:
            comm.set_fused_rs_reducers(bad)
            fail.append(("bad fused reduce-scatter option accepted", bad))
        except Exception:
            pass
    comm.destroy()
    comm.destroy()  # idempotent
    return {"fail": fail}


def case_fused_norm(comm, rank, n, args):
    from unified_ccl_b200.parallel import allreduce_residual_rmsnorm

    dev = _dev(comm, rank)
    fail = []
    eps = 1e-6
    for tokens, hidden in ((512, 1024), (130, 2048), (7, 8192), (64, 16384)):
        xs = [(torch.randn(tokens, hidden, generator=torch.Generator().manual_seed(100 + r))).to(torch.bfloat16)
              for r in range(n)]
        res = torch.randn(tokens, hidden, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16)
        gamma = (1 + 0.02 * torch.randn(hidden, generator=torch.Generator().manual_seed(8))).to(torch.bfloat16)
        h = (sum(x.float() for x in xs) + res.float()).to(torch.bfloat16).float()
        ref = h * torch.rsqrt((h * h).mean(-1, keepdim=True) + eps) * gamma.float()
        # both data paths (multimem through the switch, plain peer loads / stores) at every size
        algos = ("auto", "nvls", "two_shot") if (n > 1 and comm.info["nvls"]) else ("auto",)
        for sym, algo in [(s_, a_) for s_ in (True, False) for a_ in algos]:
            comm.set_algo(algo)
            x = comm.empty((tokens, hidden), torch.bfloat16) if sym else torch.empty(tokens, hidden, dtype=torch.bfloat16, device=dev)
            x.copy_(xs[rank])
            r_in = res.to(dev)
            r_out = comm.empty((tokens, hidden), torch.bfloat16) if sym else torch.empty_like(r_in)
            out, r_out = allreduce_residual_rmsnorm(comm, x, r_in, gamma.to(dev), eps, residual_out=r_out)
            _sync(comm)
            e1 = (r_out.float().cpu() - h).abs().max().item()
            e2 = (out.float().cpu() - ref).abs().max().item()
            # partial sums are rounded to bf16 once more when the switch reduces them
            if e1 > 0.13 * max(1.0, h.abs().max().item()) / 8 or e2 > 0.06:
                fail.append((tokens, hidden, sym, algo, e1, e2))
            if sym:
                comm.free(x)
                comm.free(r_out)
        comm.set_algo("auto")
    return {"fail": fail}


def case_tp_mlp(comm, rank, n, args):
    from unified_ccl_b200.models import TensorParallelMLP

    dev = _dev(comm, rank)
    fail = []
    # every way of moving the all-gather's rows (copy engines, dedicated CTAs, a forwarder warp per CTA),
    # and the reduce-scatter with and without CTAs that only sum: "all-gather mode/reducer CTAs"
    modes = [("ce", "0"), ("kernel", "0"), ("spread", "0"), ("ce", "8"), ("spread", "16")] if n > 1 else [("ce", "0")]
    if args:  # a subset, "ag/reducers,ag/reducers,..."
        modes = [tuple(m.split("/")) for m in args[0].split(",")]
    for ag_mode, rs_mode in modes:
        os.environ["UCCL_FUSED_AG"] = ag_mode
        os.environ["UCCL_FUSED_RS_REDUCERS"] = rs_mode
        shapes = [(512, 1024, 256 * n), (1024, 3584 * 2, 128 * n), (512, 2048, 1024 * n)]
        for hidden, ffn, tokens in shapes:
            # a run that is cut off by its time limit still says how far it got
            print("tp_mlp rank %d: all-gather %s, reducer CTAs %s, shape %s" % (rank, ag_mode, rs_mode, (hidden, ffn, tokens)),
                  file=sys.stderr, flush=True)
            mlp = TensorParallelMLP(comm, hidden, ffn, tokens, seed=3)
            x_full = torch.randn(tokens, hidden, generator=torch.Generator().manual_seed(11)).to(torch.bfloat16).to(dev)
            rows = tokens // n
            x_shard = x_full[rank * rows:(rank + 1) * rows].contiguous()
            for it in range(3):  # repeated calls reuse flags and scratch buffers
                y = mlp(x_shard)
            _sync(comm)
            gathered = mlp.x_full.clone() if n > 1 else x_full
            part = mlp.reference(x_full).contiguous()
            comm.allreduce(part)
            _sync(comm)
            ref = part[rank * rows:(rank + 1) * rows]
            err = (y.float() - ref).abs().max().item()
            scale = ref.abs().max().item()
            if not err <= 3e-2 * scale + 1e-3:
                fail.append((ag_mode, rs_mode, hidden, ffn, tokens, err, scale))
            if not torch.equal(gathered, x_full):
                fail.append((ag_mode, "x_full not gathered", hidden, tokens))
    os.environ.pop("UCCL_FUSED_AG", None)
    os.environ.pop("UCCL_FUSED_RS_REDUCERS", None)
    return {"fail": fail, "nvls": comm.info["nvls"], "async": comm.async_error(), "last": comm.last_error()}


def case_rma(comm, rank, n, args):
    from unified_ccl_b200 import Window

    dev = _dev(comm, rank)
    fail = []
    peer = (rank + 1) % n
    prev = (rank - 1) % n
    for sym in (True, False):
        cnt = 1 << 16
        buf = comm.empty(cnt, torch.float32) if sym else torch.empty(cnt, dtype=torch.float32, device=dev)
        buf.zero_()
        _sync(comm)
        win = Window(comm, buf)
        # every rank puts a pattern into its successor's window and signals
        for it in range(1, 4):
            src = torch.full((cnt // 2,), float(100 * it + rank), device=dev)
            win.put_signal(src, peer, offset=cnt // 4)
            win.wait_signal(prev, it)
            _sync(comm)
            got = buf[cnt // 4: cnt // 4 + cnt // 2]
            if not (got == 100 * it + prev).all().item():
                fail.append(("put_signal", sym, it))
            # tell the writer its data was consumed before it overwrites it
            win.signal(prev)
            win.wait_signal(peer, 0)  # no-op wait keeps the API exercised
            comm.allreduce(torch.zeros(1, device=dev))  # cheap barrier between rounds
            _sync(comm)
        # plain get from the predecessor's window
        buf.fill_(float(rank))
        _sync(comm)
        comm.allreduce(torch.zeros(1, device=dev))
        dst = torch.empty(128, device=dev)
        win.get(dst, prev, offset=5)
        _sync(comm)
        if not (dst == prev).all().item():
            fail.append(("get", sym))
        comm.allreduce(torch.zeros(1, device=dev))
        _sync(comm)
        win.close()
        if sym:
            comm.free(buf)
    return {"fail": fail}


def case_rma_device(comm, rank, n, args):
    """Kernels that call the device-side one-sided API (include/uccl_device.cuh) between GPUs:
    put + signal, cooperative / multi waits, element put / get, get + signal, fused get + reduce for
    fp32 / bf16 / fp16, both descriptor forms, and a wait that runs out (a signal nobody sends)."""
    import ctypes

    from unified_ccl_b200 import Window

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    lib = ctypes.CDLL(os.path.join(root, "tests", "native", "libuccl_devtest.so"))
    vp, sz, u64, ci = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_ulonglong, ctypes.c_int
    lib.ucclDevTestPutSignal.argtypes = [vp, ci, ci, sz, vp, sz, vp]
    lib.ucclDevTestWaitReduce.argtypes = [vp, ci, ci, u64, ci, vp, vp, sz, sz, vp, vp]
    lib.ucclDevTestWaitMultiGet.argtypes = [vp, vp, vp, ci, sz, vp, sz, vp, vp]
    lib.ucclDevTestPutElements.argtypes = [vp, ci, sz, vp, sz, vp]
    lib.ucclDevTestGetElements.argtypes = [vp, ci, sz, vp, sz, vp]
    lib.ucclDevTestMakeWindow.argtypes = [vp]
    dev = _dev(comm, rank)
    fail = []
    nxt, prv = (rank + 1) % n, (rank - 1) % n
    stream = comm._stream()
    dts = {torch.float32: 2, torch.bfloat16: 1, torch.float16: 0}

    def barrier():
        comm.allreduce(torch.zeros(1, device=dev))
        _sync(comm)

    for dyn in (0, 1):
        cnt = 1 << 14
        buf = comm.empty(cnt, torch.float32)
        buf.zero_()
        buf[: cnt // 4] = float(rank + 1)  # what my successor pulls and reduces
        _sync(comm)
        win = Window(comm, buf)
        if lib.ucclDevTestMakeWindow(win._win) != 0:
            fail.append(("makeDeviceWindow", dyn))
        ok = torch.zeros(1, dtype=torch.int32, device=dev)
        seen = {p: 0 for p in range(n)}  # signals received from each peer so far
        for it in range(1, 4):
            src = torch.full((cnt // 2,), float(100 * it + rank), device=dev)
            rc = lib.ucclDevTestPutSignal(win._win, dyn, nxt, (cnt // 4) * 4, src.data_ptr(), src.numel() * 4, stream)
            seen[prv] += 1
            ones = torch.ones(cnt // 4, device=dev)
            res = torch.empty(cnt // 4, device=dev)
            rc |= lib.ucclDevTestWaitReduce(win._win, dyn, prv, seen[prv], dts[torch.float32], ones.data_ptr(), res.data_ptr(),
                                            cnt // 4, 0, ok.data_ptr(), stream)
            _sync(comm)
            if rc != 0 or ok.item() != 1:
                fail.append(("launch/wait", dyn, it, rc, ok.item()))
                break
            if not (buf[cnt // 4: cnt // 4 + cnt // 2] == 100 * it + prv).all().item():
                fail.append(("put_signal", dyn, it))
            if not (res == prv + 2).all().item():
                fail.append(("get_reduce_f32", dyn, it))
            barrier()
        # 16-bit get + reduce: widened to fp32, rounded once
        for dt in (torch.bfloat16, torch.float16):
            w16 = comm.empty(4096, dt)
            w16.copy_(_seeded(4096, 40 + rank, dt))
            _sync(comm)
            win16 = Window(comm, w16)
            barrier()
            loc = _seeded(4096, 80 + rank, dt).to(dev)
            out = torch.empty_like(loc)
            rc = lib.ucclDevTestWaitReduce(win16._win, dyn, prv, 0, dts[dt], loc.data_ptr(), out.data_ptr(), 4096, 0,
                                           ok.data_ptr(), stream)
            _sync(comm)
            exp = (loc.float().cpu() + _seeded(4096, 40 + prv, dt).float()).to(dt)
            if rc != 0 or ok.item() != 1 or not torch.equal(out.cpu(), exp):
                fail.append(("get_reduce", str(dt), dyn, rc))
            barrier()
            win16.close()
            comm.free(w16)
        if dyn == 0:
            # element put in both directions, one multi wait for both neighbours, then get + signal
            buf.zero_()
            barrier()
            a = torch.full((64,), float(1000 + rank), device=dev)
            rc = lib.ucclDevTestPutElements(win._win, nxt, 0, a.data_ptr(), 64, stream)
            rc |= lib.ucclDevTestPutElements(win._win, prv, 64, a.data_ptr(), 64, stream)
            seen[prv] += 1
            seen[nxt] += 1
            peers = sorted({prv, nxt})
            pd = torch.tensor(peers, dtype=torch.int32, device=dev)
            ed = torch.tensor([seen[p] for p in peers], dtype=torch.int64, device=dev)
            got = torch.zeros(128, device=dev)
            barrier()  # every window is filled before anybody pulls from one
            rc |= lib.ucclDevTestWaitMultiGet(win._win, pd.data_ptr(), ed.data_ptr(), len(peers), 0, got.data_ptr(), 128 * 4,
                                              ok.data_ptr(), stream)
            seen[peers[0]] += 1  # deviceGetSignal counts the pull on the local counter of that peer
            _sync(comm)
            if rc != 0 or ok.item() != 1:
                fail.append(("multi", rc, ok.item()))
            if not ((buf[:64] == 1000 + prv).all().item() and (buf[64:128] == 1000 + nxt).all().item()):
                fail.append(("put_elements",))
            # what peers[0] holds in its first 128 floats: [1000 + its prv] * 64 + [1000 + its nxt] * 64
            q = peers[0]
            expq = torch.cat([torch.full((64,), 1000.0 + (q - 1) % n), torch.full((64,), 1000.0 + (q + 1) % n)])
            if not torch.equal(got.cpu(), expq):
                fail.append(("get_signal",))
            g2 = torch.zeros(64, device=dev)
            rc = lib.ucclDevTestGetElements(win._win, nxt, 64, g2.data_ptr(), 64, stream)
            _sync(comm)
            if rc != 0 or not (g2 == 1000 + (nxt + 1) % n).all().item():
                fail.append(("get_elements", rc))
            # a wait that runs out: nobody sends this signal; the kernel reports it and returns
            t0 = time.time()
            rc = lib.ucclDevTestWaitReduce(win._win, dyn, prv, 10 ** 9, dts[torch.float32], 0, 0, 0, 0, ok.data_ptr(), stream)
            _sync(comm)
            took = time.time() - t0
            if rc != 0 or ok.item() != 0 or took > 20:
                fail.append(("timeout path", rc, ok.item(), took))
            z = torch.ones(8, device=dev) * 2
            if z.sum().item() != 16:
                fail.append(("context unusable",))
            # checked mode of the header: a put that would run 56 bytes past the window is left out and
            # recorded; nothing in the run so far was refused
            rec = (ctypes.c_ulonglong * 4)()
            lib.ucclDevTestCheckRead.argtypes = [vp]
            if lib.ucclDevTestCheckRead(ctypes.cast(rec, vp)) != 0 or rec[0] != 0:
                fail.append(("check record not clean", list(rec)))
            barrier()
            before = buf.clone()
            src = torch.full((16,), 7.0, device=dev)
            rc = lib.ucclDevTestPutSignal(win._win, 0, nxt, cnt * 4 - 8, src.data_ptr(), 64, stream)
            _sync(comm)
            barrier()
            lib.ucclDevTestCheckRead(ctypes.cast(rec, vp))
            if rc != 0 or rec[0] != 1 or rec[1] != ((1 << 32) | nxt) or rec[2] != cnt * 4 - 8 or rec[3] != 64:
                fail.append(("out-of-window put not refused", rc, list(rec)))
            if not torch.equal(before, buf):
                fail.append(("out-of-window put touched the window",))
        barrier()
        win.close()
        comm.free(buf)
    return {"fail": fail}


def case_moe(comm, rank, n, args):
    from unified_ccl_b200.parallel import MoeDispatcher, quantize_fp8_block128

    dev = _dev(comm, rank)
    fail = []
    for hidden, experts, topk, max_tokens in ((1024, 8 * n, 4, 192), (7168, 32 * n, 8, 96)):
        eloc = experts // n
        disp = MoeDispatcher(comm, max_tokens, hidden, experts, topk)

        def inputs(r):
            g = torch.Generator().manual_seed(500 + r)
            t = max_tokens - 3 * r
            x = torch.randn(t, hidden, generator=g).to(torch.bfloat16)
            logits = torch.randn(t, experts, generator=g)
            w, idx = torch.softmax(logits, -1).topk(topk, dim=-1)
            return x, idx.to(torch.int32), w.float().contiguous()

        everyone = [inputs(r) for r in range(n)]
        x, idx, w = everyone[rank]
        for rnd in range(2):  # the second round reuses every buffer and counter
            rx, rs, rm, rc = disp.dispatch(x.to(dev), idx.to(dev).contiguous())
            _sync(comm)
            counts = rc.cpu().tolist()
            for s in range(n):
                xs, idxs, _ = everyone[s]
                want = {(t, int(idxs[t, k]) - rank * eloc, k) for t in range(xs.shape[0]) for k in range(topk)
                        if int(idxs[t, k]) // eloc == rank}
                meta = rm[s, :counts[s]].cpu()
                got = {(int(m[0]), int(m[1]), int(m[2])) for m in meta}
                if counts[s] != len(want) or got != want or (counts[s] and not (meta[:, 3] == 1).all()):
                    fail.append(("routing", hidden, rnd, s, counts[s], len(want)))
                    continue
                if counts[s] == 0:
                    continue
                src_rows = xs[meta[:, 0].long()].float()
                deq = rx[s, :counts[s]].float().cpu().view(counts[s], hidden // 128, 128) * rs[s, :counts[s]].cpu().unsqueeze(-1)
                amax = src_rows.view(counts[s], hidden // 128, 128).abs().amax(-1, keepdim=True)
                bad = ((deq - src_rows.view_as(deq)).abs() > 0.0625 * amax + 1e-6).sum().item()
                qref, sref = quantize_fp8_block128(src_rows)
                if bad or not torch.allclose(rs[s, :counts[s]].cpu(), sref, rtol=1e-6, atol=0):
                    fail.append(("payload", hidden, rnd, s, bad))
                # the "expert": scale the dequantised row by (global expert id + 1)
                gid = (meta[:, 1] + rank * eloc + 1).float().unsqueeze(-1)
                disp.expert_out[s, :counts[s]] = (deq.view(counts[s], hidden) * gid).to(torch.bfloat16).to(dev)
            out = disp.combine(w.to(dev))
            _sync(comm)
            q, sc = quantize_fp8_block128(x.float())
            deq_x = (q.float().view(x.shape[0], hidden // 128, 128) * sc.unsqueeze(-1)).view(x.shape[0], hidden)
            ref = torch.zeros(x.shape[0], hidden)
            for k in range(topk):
                ref += w[:, k:k + 1] * (deq_x * (idx[:, k:k + 1].float() + 1)).to(torch.bfloat16).float()
            err = (out.float().cpu() - ref).abs().max().item()
            if err > 2e-2 * ref.abs().max().item() + 1e-3:
                fail.append(("combine", hidden, rnd, err, ref.abs().max().item()))
        if disp.overflow() != 0:
            fail.append(("overflow", hidden))
        disp.close()
    return {"fail": fail}


def case_canary(comm, rank, n, args):
    """UCCL_CANARY=1: collectives on odd-sized symmetric buffers leave the guard regions intact; a store
    just past a buffer's end (inside this rank's own mapping, so nothing faults) is found and located."""
    from unified_ccl_b200.communicator import _tensor_from_ptr
    dev = _dev(comm, rank)
    fail = []
    numel = 70001  # not a multiple of a 16-byte vector
    x = comm.empty((numel,), torch.bfloat16)
    g = comm.empty((numel * n,), torch.bfloat16)
    for it in range(2):
        x.copy_(torch.full((numel,), float(rank + 1), device=dev, dtype=torch.bfloat16))
        comm.allreduce(x)
        comm.allgather(x, g)
        comm.reduce_scatter(g, x)
        _sync(comm)
    try:
        comm.check_memory()
    except Exception as e:  # noqa: BLE001
        fail.append(("clean run flagged", str(e)))
    # overrun: eight elements behind the end of x, written by this rank through its own mapping
    over = _tensor_from_ptr(x.data_ptr(), numel + 8, torch.bfloat16, dev.index)
    over[numel + 3 :].fill_(1.0)
    _sync(comm)
    msg = None
    try:
        comm.check_memory()
    except Exception as e:  # noqa: BLE001
        msg = str(e)
    if msg is None or ("offset %d" % ((numel + 3) * 2)) not in (comm.last_error() + msg):
        fail.append(("overrun not located", msg, comm.last_error()))
    freed_err = None
    try:
        comm.free(x)
    except Exception as e:  # noqa: BLE001
        freed_err = str(e)
    if freed_err is None:
        fail.append(("free did not report the overrun",))
    comm.free(g)
    return {"fail": fail, "msg": msg}


def case_skipped_collective(comm, rank, n, args):
    """The last rank skips one all-reduce: the others' device-side waits run out and report it."""
    dev = _dev(comm, rank)
    x = torch.ones(4096, device=dev)
    comm.allreduce(x)
    _sync(comm)
    res = {"fail": [], "_abort": True}
    if rank == n - 1:
        time.sleep(float(args[0]) if args else 3.0)
        res["skipped"] = True
        return res
    t0 = time.time()
    err = None
    try:
        y = torch.ones(1 << 16, device=dev)
        comm.allreduce(y)
        _sync(comm)
        comm.finalize()
    except Exception as e:  # noqa: BLE001
        err = str(e)
    res["seconds"] = time.time() - t0
    res["err"] = err
    res["async"] = comm.async_error()
    res["last"] = comm.last_error()
    res["timeouts"] = comm.counters()["wait_timeouts"]
    if err is None:
        res["fail"].append(("no error",))
    # the CUDA context must still be usable after the timed-out kernel
    z = torch.ones(8, device=dev) * 2
    _sync(comm)
    if z.sum().item() != 16:
        res["fail"].append(("context unusable",))
    return res


def case_peer_exits(comm, rank, n, args):
    """Rank n-1 leaves between steps; the others get an error on their next collective."""
    dev = _dev(comm, rank)
    x = torch.ones(1024, device=dev)
    comm.allreduce(x)
    _sync(comm)
    ok_first = bool((x.cpu() == n).all())
    if rank == n - 1:
        return {"fail": [] if ok_first else [("first",)], "left": True, "_exit_now": True}
    time.sleep(0.5)
    t0 = time.time()
    err = None
    try:
        y = torch.ones(1 << 20, device=dev)
        comm.allreduce(y)
        _sync(comm)
        if comm.on_gpu:
            comm.finalize()
    except Exception as e:  # noqa: BLE001
        err = str(e)
    took = time.time() - t0
    fail = []
    if not ok_first:
        fail.append(("first",))
    if err is None and comm.async_error() == 0:
        fail.append(("no error surfaced",))
    return {"fail": fail, "err": err, "seconds": took, "async": comm.async_error(), "last": comm.last_error(),
            "timeouts": comm.counters()["wait_timeouts"], "_abort": True}


def main():
    case, rank, n, idfile = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
    if os.environ.get("UCCL_TEST_DUMP_AFTER_S"):
        # a rank that is still running after this many seconds prints where it is and exits
        import faulthandler

        faulthandler.dump_traceback_later(float(os.environ["UCCL_TEST_DUMP_AFTER_S"]), exit=True)
    args = sys.argv[5:]
    res = {"rank": rank}
    comm = None
    try:
        if torch.cuda.is_available() and os.environ.get("UCCL_BACKEND", "") != "cpu":
            torch.cuda.set_device(rank % torch.cuda.device_count())
        if case == "never_joins" and rank == n - 1:
            _uid(rank, idfile)  # learn the id, then walk away without joining
            print("RESULT " + json.dumps({"rank": rank, "absent": True}), flush=True)
            return
        from unified_ccl_b200 import Communicator

        uid = _uid(rank, idfile)
        if case == "never_joins":
            t0 = time.time()
            try:
                Communicator(rank, n, unique_id=uid)
                res["fail"] = [("init succeeded",)]
            except Exception as e:  # noqa: BLE001
                res["err"] = str(e)
                res["seconds"] = time.time() - t0
                res["fail"] = []
            print("RESULT " + json.dumps(res), flush=True)
            return
        comm = Communicator(rank, n, unique_id=uid)
        res.update(globals()["case_" + case](comm, rank, n, args))
    except Exception:  # noqa: BLE001
        res["exc"] = traceback.format_exc()
    print("RESULT " + json.dumps(res, default=str), flush=True)
    if res.get("_exit_now"):
        os._exit(0)  # leave without tearing the communicator down, like a crashed rank
    try:
        if comm is not None:
            if res.get("_abort"):
                comm.abort()
            else:
                comm.destroy()
    except Exception:  # noqa: BLE001
        pass


if __name__ == "__main__":
    main()
