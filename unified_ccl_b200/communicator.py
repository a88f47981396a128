"""``Communicator``: the user-facing object, one per rank.

Keeps the contract of the reference's Python class (bindings/python/uccl/uccl.py:7-150:
``Communicator(rank, world_size)``, in-place ``allreduce``, ``allgather(send, recv)``,
``reduce_scatter(send, recv)``, idempotent ``destroy``, ``rank`` / ``world_size`` properties)
and adds the rest of the library: broadcast, reduce, all-to-all, send/recv, groups, symmetric
tensors, fused kernels, tuning and counters.  Tensors are ``torch`` CUDA tensors for a
communicator on GPUs (the kernels run on the current torch stream) and CPU tensors for a
communicator created with ``UCCL_BACKEND=cpu`` or on a machine without GPUs.
"""
import contextlib
import os
import threading

import torch

from . import _C

_DTYPES = {
    torch.float16: 0,
    torch.bfloat16: 1,
    torch.float32: 2,
    torch.uint8: 4,
}
if hasattr(torch, "float8_e4m3fn"):
    _DTYPES[torch.float8_e4m3fn] = 3
_REDUCIBLE = (torch.float16, torch.bfloat16, torch.float32)

ALGOS = {"auto": 0, "ring": 1, "one_shot": 2, "two_shot": 3, "nvls": 4, "copy_engine": 5, "net": 6}
PROTOS = {"auto": 0, "simple": 1, "ll": 2, "ll128": 3}
COLLS = {"allreduce": 0, "allgather": 1, "reducescatter": 2, "broadcast": 3, "reduce": 4, "alltoall": 5,
         "sendrecv": 6, "rma": 7}

_instance_counter = 0
_instance_lock = threading.Lock()


def get_unique_id() -> bytes:
    """Start the rendezvous service in this process and return the 128-byte id naming it."""
    return _C.get_unique_id()


def _derive_unique_id(rank: int, world_size: int) -> bytes:
    """Agree on a unique id without the caller passing one."""
    global _instance_counter
    if world_size == 1:
        return _C.get_unique_id()
    try:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized() and dist.get_world_size() == world_size:
            box = [_C.get_unique_id() if rank == 0 else None]
            dist.broadcast_object_list(box, src=0)
            return box[0]
    except Exception:
        pass
    with _instance_lock:
        inst = _instance_counter
        _instance_counter += 1
    spec = os.environ.get("UCCL_COMM_ID")
    if spec:
        host, port = spec.rsplit(":", 1)
        port = int(port) + inst
    elif "MASTER_ADDR" in os.environ and "MASTER_PORT" in os.environ:
        host = os.environ["MASTER_ADDR"]
        port = int(os.environ["MASTER_PORT"]) + 29 + inst
    else:
        raise RuntimeError(
            "Communicator(world_size>1) needs a unique id: pass unique_id=..., initialise torch.distributed, "
            "or set UCCL_COMM_ID=ip:port (or MASTER_ADDR/MASTER_PORT)")
    if host == "localhost":
        host = "127.0.0.1"
    uid = _C.unique_id_from_address(host, port, 0x5eed + inst)
    if rank == 0:
        _C.serve_unique_id(uid)
    return uid


class Communicator:
    def __init__(self, rank: int, world_size: int, unique_id: bytes = None):
        if world_size < 1 or world_size > _C.MAX_RANKS:
            raise ValueError(f"world_size must be in [1, {_C.MAX_RANKS}], got {world_size}")
        if rank < 0 or rank >= world_size:
            raise ValueError(f"rank must be in [0, {world_size}), got {rank}")
        self._comm = 0
        self._rank = rank
        self._world_size = world_size
        self._sym = {}  # data_ptr -> bytes, symmetric allocations to free
        if unique_id is None:
            unique_id = _derive_unique_id(rank, world_size)
        self._comm = _C.comm_init_rank(world_size, unique_id, rank)
        self._info = _C.comm_info(self._comm)

    # ------------------------------------------------------------------ properties
    @property
    def rank(self) -> int:
        return self._rank

    @property
    def world_size(self) -> int:
        return self._world_size

    @property
    def info(self) -> dict:
        return dict(self._info)

    @property
    def on_gpu(self) -> bool:
        return self._info["cuda_device"] >= 0

    @property
    def handle(self) -> int:
        return self._comm

    # ------------------------------------------------------------------ helpers
    def _check(self, t: torch.Tensor, reducible=False):
        if self._comm == 0:
            raise RuntimeError("communicator was destroyed")
        if not isinstance(t, torch.Tensor):
            raise TypeError("expected a torch.Tensor")
        if t.dtype not in _DTYPES:
            raise TypeError(f"unsupported dtype {t.dtype}")
        if reducible and t.dtype not in _REDUCIBLE:
            raise TypeError(f"dtype {t.dtype} cannot be reduced; use float16, bfloat16 or float32")
        if self.on_gpu and not t.is_cuda:
            raise ValueError("this communicator runs on GPUs: tensors must be CUDA tensors")
        if not self.on_gpu and t.is_cuda:
            raise ValueError("this communicator runs on the CPU backend: tensors must be CPU tensors")
        if t.is_cuda and t.device.index != self._info["cuda_device"]:
            raise ValueError(f"tensor is on cuda:{t.device.index}, communicator on cuda:{self._info['cuda_device']}")
        if not t.is_contiguous():
            raise ValueError("tensor must be contiguous")

    def _stream(self) -> int:
        if not self.on_gpu:
            return 0
        return torch.cuda.current_stream(self._info["cuda_device"]).cuda_stream

    # ------------------------------------------------------------------ collectives
    def allreduce(self, tensor: torch.Tensor, op: str = "sum", out: torch.Tensor = None) -> torch.Tensor:
        """Sum ``tensor`` over all ranks, in place (or into ``out``)."""
        if op != "sum":
            raise ValueError("only op='sum' is supported")
        self._check(tensor, reducible=True)
        dst = tensor if out is None else out
        if out is not None:
            self._check(out, reducible=True)
            if out.dtype != tensor.dtype or out.numel() != tensor.numel():
                raise ValueError("out must match tensor in dtype and size")
        _C.allreduce(self._comm, tensor.data_ptr(), dst.data_ptr(), tensor.numel(), _DTYPES[tensor.dtype], self._stream())
        return dst

    def allgather(self, send_tensor: torch.Tensor, recv_tensor: torch.Tensor) -> torch.Tensor:
        self._check(send_tensor)
        self._check(recv_tensor)
        if recv_tensor.dtype != send_tensor.dtype:
            raise ValueError("send and recv dtypes differ")
        if recv_tensor.numel() != send_tensor.numel() * self._world_size:
            raise ValueError("recv_tensor must hold world_size * send_tensor.numel() elements")
        _C.allgather(self._comm, send_tensor.data_ptr(), recv_tensor.data_ptr(), send_tensor.numel(),
                     _DTYPES[send_tensor.dtype], self._stream())
        return recv_tensor

    def reduce_scatter(self, send_tensor: torch.Tensor, recv_tensor: torch.Tensor, op: str = "sum") -> torch.Tensor:
        if op != "sum":
            raise ValueError("only op='sum' is supported")
        self._check(send_tensor, reducible=True)
        self._check(recv_tensor, reducible=True)
        if recv_tensor.dtype != send_tensor.dtype:
            raise ValueError("send and recv dtypes differ")
        if send_tensor.numel() != recv_tensor.numel() * self._world_size:
            raise ValueError("send_tensor must hold world_size * recv_tensor.numel() elements")
        _C.reduce_scatter(self._comm, send_tensor.data_ptr(), recv_tensor.data_ptr(), recv_tensor.numel(),
                          _DTYPES[send_tensor.dtype], self._stream())
        return recv_tensor

    def _ex_args(self, send_tensor, out_tensor, scales, per_rank):
        self._check(send_tensor, reducible=True)
        self._check(out_tensor)
        if out_tensor.dtype not in _REDUCIBLE and _DTYPES[out_tensor.dtype] != 3:
            raise TypeError("output must be float16, bfloat16, float32 or float8_e4m3fn")
        if _DTYPES[out_tensor.dtype] == 3:
            if scales is None:
                scales = torch.empty(out_tensor.numel() // 128, dtype=torch.float32, device=out_tensor.device)
            if scales.dtype != torch.float32 or scales.numel() * 128 != out_tensor.numel() or per_rank % 128:
                raise ValueError("fp8 output takes one float32 scale per 128 elements")
        else:
            scales = None
        return scales

    def reduce_scatter_cast(self, send_tensor: torch.Tensor, recv_tensor: torch.Tensor, scale: float = 1.0,
                            scales: torch.Tensor = None):
        """``recv = cast(scale * reduce_scatter(send))`` in one kernel: the sum stays in fp32 until the
        store.  ``recv_tensor`` may be float16 / bfloat16 / float32, or float8_e4m3fn with one float32
        scale per 128 elements (returned as the second value)."""
        if send_tensor.numel() != recv_tensor.numel() * self._world_size:
            raise ValueError("send_tensor must hold world_size * recv_tensor.numel() elements")
        scales = self._ex_args(send_tensor, recv_tensor, scales, recv_tensor.numel())
        _C.reduce_scatter_ex(self._comm, send_tensor.data_ptr(), recv_tensor.data_ptr(), recv_tensor.numel(),
                             _DTYPES[send_tensor.dtype], _DTYPES[recv_tensor.dtype], float(scale),
                             scales.data_ptr() if scales is not None else 0, self._stream())
        return recv_tensor, scales

    def allreduce_cast(self, send_tensor: torch.Tensor, out: torch.Tensor, scale: float = 1.0, scales: torch.Tensor = None):
        """``out = cast(scale * allreduce(send))``; the gather half moves elements of the output type."""
        if send_tensor.numel() != out.numel():
            raise ValueError("out must hold as many elements as send_tensor")
        scales = self._ex_args(send_tensor, out, scales, out.numel() // self._world_size)
        _C.allreduce_ex(self._comm, send_tensor.data_ptr(), out.data_ptr(), send_tensor.numel(), _DTYPES[send_tensor.dtype],
                        _DTYPES[out.dtype], float(scale), scales.data_ptr() if scales is not None else 0, self._stream())
        return out, scales

    def broadcast(self, tensor: torch.Tensor, root: int = 0) -> torch.Tensor:
        self._check(tensor)
        if not 0 <= root < self._world_size:
            raise ValueError("root out of range")
        _C.broadcast(self._comm, tensor.data_ptr(), tensor.data_ptr(), tensor.numel(), _DTYPES[tensor.dtype], root,
                     self._stream())
        return tensor

    def reduce(self, send_tensor: torch.Tensor, recv_tensor: torch.Tensor = None, root: int = 0) -> torch.Tensor:
        self._check(send_tensor, reducible=True)
        if not 0 <= root < self._world_size:
            raise ValueError("root out of range")
        if recv_tensor is None:
            recv_tensor = send_tensor
        else:
            self._check(recv_tensor, reducible=True)
            if recv_tensor.numel() != send_tensor.numel() or recv_tensor.dtype != send_tensor.dtype:
                raise ValueError("recv_tensor must match send_tensor")
        _C.reduce(self._comm, send_tensor.data_ptr(), recv_tensor.data_ptr(), send_tensor.numel(),
                  _DTYPES[send_tensor.dtype], root, self._stream())
        return recv_tensor

    def alltoall(self, send_tensor: torch.Tensor, recv_tensor: torch.Tensor) -> torch.Tensor:
        self._check(send_tensor)
        self._check(recv_tensor)
        if send_tensor.numel() != recv_tensor.numel() or send_tensor.dtype != recv_tensor.dtype:
            raise ValueError("send and recv must match in size and dtype")
        if send_tensor.numel() % self._world_size:
            raise ValueError("numel must be a multiple of world_size")
        if send_tensor.data_ptr() == recv_tensor.data_ptr():
            raise ValueError("all-to-all cannot run in place")
        _C.alltoall(self._comm, send_tensor.data_ptr(), recv_tensor.data_ptr(), send_tensor.numel() // self._world_size,
                    _DTYPES[send_tensor.dtype], self._stream())
        return recv_tensor

    def send(self, tensor: torch.Tensor, peer: int):
        self._check(tensor)
        _C.send(self._comm, tensor.data_ptr(), tensor.numel(), _DTYPES[tensor.dtype], peer, self._stream())

    def recv(self, tensor: torch.Tensor, peer: int):
        self._check(tensor)
        _C.recv(self._comm, tensor.data_ptr(), tensor.numel(), _DTYPES[tensor.dtype], peer, self._stream())
        return tensor

    @contextlib.contextmanager
    def group(self):
        """Operations issued inside the block are launched together when it exits."""
        _C.group_start()
        try:
            yield self
        except BaseException:
            try:
                _C.group_end()
            finally:
                raise
        else:
            _C.group_end()

    # ------------------------------------------------------------------ symmetric memory
    def empty(self, shape, dtype=torch.bfloat16) -> torch.Tensor:
        """Collective: a tensor backed by symmetric (peer-mapped, multicast-bound) memory.

        Every rank must call with the same shape and dtype, in the same order.  Collectives on
        such tensors run zero-copy.  The memory is released by :meth:`free` or :meth:`destroy`.
        """
        if not self.on_gpu:
            return torch.empty(shape, dtype=dtype)
        if isinstance(shape, int):
            shape = (shape,)
        numel = 1
        for s in shape:
            numel *= int(s)
        itemsize = torch.empty((), dtype=dtype).element_size()
        nbytes = max(numel * itemsize, 16)
        ptr = _C.mem_alloc(self._comm, nbytes)
        self._sym[ptr] = nbytes
        return _tensor_from_ptr(ptr, numel, dtype, self._info["cuda_device"]).view(*shape)

    def free(self, tensor: torch.Tensor):
        ptr = tensor.data_ptr()
        if ptr in self._sym:
            _C.mem_free(self._comm, ptr)
            del self._sym[ptr]

    def check_memory(self):
        """Collective: verify the guard regions around every symmetric buffer (needs ``UCCL_CANARY=1`` in
        the environment when the communicator is created; a no-op otherwise).  Raises when a store
        landed outside a buffer; the message names the buffer and the byte offset."""
        if self.on_gpu:
            _C.mem_check(self._comm)

    def is_symmetric(self, tensor: torch.Tensor) -> bool:
        return _C.mem_peer_pointer(self._comm, tensor.data_ptr(), self._rank) != 0 if self.on_gpu else False

    # ------------------------------------------------------------------ tuning / introspection
    def set_algo(self, algo: str = "auto", proto: str = "auto"):
        _C.set_algo(self._comm, ALGOS[algo], PROTOS[proto])

    def set_blocks(self, blocks: int = 0):
        """Force the CTA count of collective kernels (0 = let the tuner decide)."""
        _C.set_blocks(self._comm, int(blocks))

    def set_fused_options(self, ag_mode: str = "auto", comm_ctas: int = 0, ce_chunks: int = 0):
        """How the all-gather -> GEMM fusion moves its rows: ``"ce"`` (copy engines, ``ce_chunks`` copies per
        peer; ``comm_ctas`` then is the number of copy-engine lanes, 0 = one stream per peer, k = k streams
        that serve the peers one after the other), ``"kernel"`` (``comm_ctas`` communication CTAs inside the
        GEMM launch) or ``"spread"`` (a forwarder warp in every GEMM CTA); 0 keeps a default."""
        _C.set_fused_options(self._comm, {"auto": 0, "ce": 1, "kernel": 2, "spread": 3}[ag_mode], int(comm_ctas), int(ce_chunks))

    def set_fused_norm_rows(self, rows: int = -1):
        """Shape of the fused all-reduce + residual + RMSNorm on the switch path: 1..4 = all-reduce phase with
        that many rows per CTA and pass, then a local normalise phase; 0 = one phase; -1 = default."""
        _C.set_fused_norm_rows(self._comm, int(rows))

    def set_fused_rs_reducers(self, reducer_ctas: int = 0):
        """CTAs of the fused GEMM -> reduce-scatter launch that only sum the staged partial tiles (0 = none)."""
        _C.set_fused_rs_reducers(self._comm, int(reducer_ctas))

    def load_tuning(self, path: str):
        _C.load_tuning(self._comm, path)

    def query_tuning(self, coll: str, nbytes: int, symmetric: bool = False):
        a, p, n = _C.query_tuning(self._comm, COLLS[coll], nbytes, symmetric)
        inv_a = {v: k for k, v in ALGOS.items()}
        inv_p = {v: k for k, v in PROTOS.items()}
        return inv_a[a], inv_p[p], n

    def counters(self) -> dict:
        return _C.comm_counters(self._comm)

    def async_error(self) -> int:
        return _C.get_async_error(self._comm)

    def last_error(self) -> str:
        return _C.get_last_error(self._comm)

    def finalize(self):
        _C.comm_finalize(self._comm)

    # ------------------------------------------------------------------ lifecycle
    def destroy(self):
        if self._comm:
            comm, self._comm = self._comm, 0
            try:
                _C.comm_finalize(comm)
            except Exception:
                pass
            self._sym.clear()
            _C.comm_destroy(comm)

    def abort(self):
        if self._comm:
            comm, self._comm = self._comm, 0
            _C.comm_abort(comm)

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass

    def __repr__(self) -> str:
        return f"Communicator(rank={self._rank}, world_size={self._world_size}, backend={'cuda' if self.on_gpu else 'cpu'})"


class _CudaArray:
    """Minimal ``__cuda_array_interface__`` carrier so torch can wrap a raw device pointer."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,),
            "typestr": "|u1",
            "data": (ptr, False),
            "version": 3,
            "strides": None,
        }


def _tensor_from_ptr(ptr: int, numel: int, dtype, device_index: int) -> torch.Tensor:
    itemsize = torch.empty((), dtype=dtype).element_size()
    raw = torch.as_tensor(_CudaArray(ptr, max(numel * itemsize, 1)), device=torch.device("cuda", device_index))
    return raw[: numel * itemsize].view(dtype)


class Window:
    """A registered buffer that peers can put into / get from, with per-peer signal counters.

    Collective: every rank registers a tensor of the same size.  Signal counters are monotonic;
    ``wait_signal`` takes the absolute number of signals expected from a peer so far (the
    semantics of the reference's ucclWaitSignal, src/rma/rma.cc:474-570).
    """

    def __init__(self, comm: Communicator, tensor: torch.Tensor):
        comm._check(tensor)
        self._comm = comm
        self.tensor = tensor
        self._win = _C.window_register(comm.handle, tensor.data_ptr(), tensor.numel() * tensor.element_size())

    def _args(self, local: torch.Tensor, peer: int, offset_elems: int):
        self._comm._check(local)
        if local.dtype != self.tensor.dtype:
            raise TypeError("dtype differs from the window's")
        return (self._comm.handle, local.data_ptr(), local.numel(), _DTYPES[local.dtype], peer, self._win,
                offset_elems * local.element_size(), self._comm._stream())

    def put(self, local, peer, offset=0):
        _C.put(*self._args(local, peer, offset))

    def get(self, local, peer, offset=0):
        _C.get(*self._args(local, peer, offset))

    def put_signal(self, local, peer, offset=0):
        _C.put_signal(*self._args(local, peer, offset))

    def get_signal(self, local, peer, offset=0):
        _C.get_signal(*self._args(local, peer, offset))

    def signal(self, peer):
        _C.signal(self._comm.handle, peer, self._comm._stream())

    def wait_signal(self, peers, counts):
        if isinstance(peers, int):
            peers, counts = [peers], [counts]
        _C.wait_signal(self._comm.handle, self._win, list(peers), list(counts), self._comm._stream())

    def close(self):
        if self._win:
            win, self._win = self._win, 0
            _C.window_deregister(win)
