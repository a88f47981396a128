"""The allocation-free MoE dispatch entry point, called through its exported C symbol.

Some callers of this library cannot allocate device memory at all (they live inside another
component's memory pool, or in a loop that must never touch the CUDA allocator), so they cannot
create the context object that the regular dispatch needs.  For them the library exports
ucclMoeDispatchLocalNoAlloc, whose bookkeeping sits in a fixed array inside the library.  This
test checks that it produces what the regular dispatch (one rank) produces, twice in a row: the
second call must not be confused by what the first one left in the shared array.

Collected last on purpose (file name), so a run that stops at the first failure has already run
everything else.
"""
import ctypes
import os

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _lib():
    lib = ctypes.CDLL(os.path.join(ROOT, "unified_ccl_b200", "libuccl.so"))
    fn = lib.ucclMoeDispatchLocalNoAlloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    lib.ucclNoAllocLastError.restype = ctypes.c_char_p
    return lib


def _sorted_rows(recv_x, recv_scale, recv_meta, count):
    """Rows ordered by (token, k) so that two runs with different atomic orders can be compared."""
    meta = recv_meta[:count].cpu()
    key = meta[:, 0].long() * 64 + meta[:, 2].long()
    order = torch.argsort(key)
    x = recv_x[:count].view(torch.uint8).cpu()[order]
    return x, recv_scale[:count].cpu()[order], meta[order]


def test_rejects_sizes_beyond_the_built_in_scratch():
    """Argument checks run before any CUDA call, so this part needs no GPU."""
    lib = _lib()
    one = ctypes.c_void_p(16)
    rc = lib.ucclMoeDispatchLocalNoAlloc(one, one, 4097, 1024, 8, 4, one, one, one, one, 1 << 20, None)
    assert rc == 3 and b"tokens" in lib.ucclNoAllocLastError()
    rc = lib.ucclMoeDispatchLocalNoAlloc(one, one, 16, 1024, 8, 17, one, one, one, one, 1 << 20, None)
    assert rc == 3 and b"topk" in lib.ucclNoAllocLastError()
    rc = lib.ucclMoeDispatchLocalNoAlloc(one, one, 16, 1000, 8, 4, one, one, one, one, 1 << 20, None)
    assert rc == 3 and b"hidden" in lib.ucclNoAllocLastError()
    rc = lib.ucclMoeDispatchLocalNoAlloc(one, one, 16, 1024, 8, 4, one, one, one, one, 63, None)
    assert rc == 3 and b"rowsCapacity" in lib.ucclNoAllocLastError()
    odd = ctypes.c_void_p(18)  # a scale pointer that a float store cannot use
    rc = lib.ucclMoeDispatchLocalNoAlloc(one, one, 16, 1024, 8, 4, one, odd, one, one, 64, None)
    assert rc == 3 and b"4-byte aligned" in lib.ucclNoAllocLastError()


@pytest.mark.gpu
def test_matches_the_regular_dispatch_twice_in_a_row():
    os.environ.setdefault("UCCL_BOOTSTRAP_IFNAME", "lo")
    from unified_ccl_b200 import Communicator
    from unified_ccl_b200.parallel import MoeDispatcher, quantize_fp8_block128

    lib = _lib()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    comm = Communicator(0, 1)
    hidden, experts, topk, max_tokens = 2048, 16, 4, 300
    disp = MoeDispatcher(comm, max_tokens, hidden, experts, topk)
    cap = max_tokens * topk
    # the caller owns the outputs; nothing below allocates inside the entry point
    out_x = torch.empty(cap, hidden, dtype=torch.uint8, device=dev)
    out_s = torch.empty(cap, hidden // 128, dtype=torch.float32, device=dev)
    out_m = torch.empty(cap, 4, dtype=torch.int32, device=dev)
    out_c = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    for call, tokens in enumerate((300, 77)):
        g = torch.Generator().manual_seed(900 + call)
        x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16).to(dev)
        idx = torch.randn(tokens, experts, generator=g).topk(topk, dim=-1).indices.to(torch.int32).to(dev).contiguous()
        if call == 1:
            idx[5, 2] = -1  # an unused slot
        rx, rs, rm, rc = disp.dispatch(x, idx)
        torch.cuda.synchronize()
        want = _sorted_rows(rx[0], rs[0], rm[0], int(rc[0].item()))
        ret = lib.ucclMoeDispatchLocalNoAlloc(x.data_ptr(), idx.data_ptr(), tokens, hidden, experts, topk, out_x.data_ptr(),
                                              out_s.data_ptr(), out_m.data_ptr(), out_c.data_ptr(), cap, stream)
        assert ret == 0, lib.ucclNoAllocLastError()
        torch.cuda.synchronize()
        count = int(out_c.item())
        assert count == int(rc[0].item()) == int((idx >= 0).sum().item())
        got = _sorted_rows(out_x, out_s, out_m, count)
        assert torch.equal(got[2], want[2])                      # same (token, expert, k, 1) descriptors
        assert torch.equal(got[0], want[0])                      # same fp8 payload, bit for bit
        assert torch.allclose(got[1], want[1], rtol=1e-6, atol=0)  # same scales
        # and both equal the fp32 restatement of the cast (amax / 448 per 128 elements, e4m3 rounding)
        src_rows = x.float().cpu()[got[2][:, 0].long()]
        q_ref, s_ref = quantize_fp8_block128(src_rows)
        assert torch.allclose(got[1], s_ref, rtol=1e-6, atol=0)
        deq = got[0].view(torch.float8_e4m3fn).float().view(count, hidden // 128, 128) * got[1].unsqueeze(-1)
        ref = q_ref.float().view(count, hidden // 128, 128) * s_ref.unsqueeze(-1)
        amax = src_rows.view(count, hidden // 128, 128).abs().amax(-1, keepdim=True)
        assert ((deq - ref).abs() <= 0.0625 * amax + 1e-6).all()  # at most one fp8 step apart, never more
        assert (got[0] != q_ref.view(torch.uint8)).float().mean().item() < 1e-3  # and bit-identical almost everywhere
    disp.close()
    comm.destroy()
