"""Peer-mapped output buffers for the multi-GPU path (one process per GPU, one node).

Every rank owns an *arena* of device memory that every other rank maps into its own address space (CUDA IPC;
the 64-byte handles travel through the process group).  A column-sharded projection then writes its shard
straight into the right columns of the full-width matrix in EVERY arena from the kernel's epilogue
(``PeerMatrix.out_for``), and one :meth:`PeerArena.barrier` per exchange point orders the readers after
the writers.  No collective and no re-layout kernel runs on the data path.

torch is used for the process group only; the arenas are allocated and mapped by the C library, and the
tensors handed out are views of arena memory (``__cuda_array_interface__``).
"""

from __future__ import annotations

import ctypes

import torch

from . import _native


def exchange_handles(handle: bytes, group=None) -> list:
    """All-gather of the ranks' 64-byte IPC handles (host side, any backend).  Raises ValueError on EVERY rank when
    some rank contributed something that is not a 64-byte handle, so that no rank goes on to map garbage."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    handles = [None] * world
    dist.all_gather_object(handles, handle, group=group)
    bad = [r for r, h in enumerate(handles) if not isinstance(h, (bytes, bytearray)) or len(h) != 64]
    if bad:
        raise ValueError(f"ranks {bad} did not contribute a 64-byte IPC handle")
    return [bytes(h) for h in handles]


def agree(what: str, value, group=None) -> None:
    """Every rank must pass the same ``value`` (arena size, carving order ...); raises ValueError on every rank
    otherwise.  A mismatch would make ranks store into each other's arenas at different offsets."""
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    values = [None] * dist.get_world_size(group)
    dist.all_gather_object(values, value, group=group)
    if any(v != values[0] for v in values):
        raise ValueError(f"ranks disagree on {what}: {values}")


class _Span:
    """Minimal ``__cuda_array_interface__`` carrier for a raw device pointer."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


class PeerMatrix:
    """A [rows, cols] matrix that exists at the same offset of every rank's arena."""

    def __init__(self, arena: "PeerArena", offset: int, rows: int, cols: int, dtype: torch.dtype):
        self.arena, self.offset, self.rows, self.cols, self.dtype = arena, offset, rows, cols, dtype
        self.local = arena.view(offset, (rows, cols), dtype)  # this rank's copy, a torch tensor

    def out_for(self, col0: int) -> _native.PeerOutStruct:
        """Descriptor for a kernel on this rank that produces columns [col0, col0 + n) of the matrix."""
        out = _native.PeerOutStruct()
        order = self.arena.store_order
        for i, p in enumerate(order):
            out.ptr[i] = self.arena.bases[p] + self.offset
        out.world = len(order)
        out.ld = self.cols
        out.col0 = col0
        return out


class PeerArena:
    """``nbytes`` of payload per rank (plus the flag block the barrier uses), mapped on every rank."""

    def __init__(self, nbytes: int, group=None, device=None):
        import torch.distributed as dist

        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        if self.world > _native.XDK_MAX_PEERS:
            raise ValueError(f"at most {_native.XDK_MAX_PEERS} ranks")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.nbytes = _native.XDK_PEER_FLAG_BYTES + ((nbytes + 255) // 256) * 256
        lib = _native.lib()
        with torch.cuda.device(self.device):
            base = ctypes.c_void_p()
            _native.check(lib.xdk_peer_alloc(self.nbytes, ctypes.byref(base)), "xdk_peer_alloc")
            self.bases = [0] * self.world
            self.bases[self.rank] = base.value
            self._opened = []
            if self.world > 1:
                agree("the arena size", self.nbytes, group)
                handle = (ctypes.c_ubyte * 64)()
                _native.check(lib.xdk_peer_export(base, handle), "xdk_peer_export")
                handles = exchange_handles(bytes(handle), group)
                for p, h in enumerate(handles):
                    if p == self.rank:
                        continue
                    mapped = ctypes.c_void_p()
                    buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                    _native.check(lib.xdk_peer_open(buf, ctypes.byref(mapped)), "xdk_peer_open")
                    self.bases[p] = mapped.value
                    self._opened.append(mapped.value)
        # local copy first, then the peers starting with the next rank: ranks do not all hit the same link at once
        self.store_order = [(self.rank + i) % self.world for i in range(self.world)]
        self._arena_ptrs = (ctypes.c_void_p * _native.XDK_MAX_PEERS)(*self.bases)
        self._cursor = _native.XDK_PEER_FLAG_BYTES
        self._sites = 0
        self._closed = False

    # ---- carving
    def view(self, offset: int, shape, dtype: torch.dtype) -> torch.Tensor:
        count = 1
        for s in shape:
            count *= s
        nbytes = count * torch.empty(0, dtype=dtype).element_size()
        raw = torch.as_tensor(_Span(self.bases[self.rank] + offset, nbytes), device=self.device)
        return raw.view(dtype).view(*shape)

    def matrix(self, rows: int, cols: int, dtype: torch.dtype) -> PeerMatrix:
        """The next free [rows, cols] block (256-byte aligned); every rank must carve in the same order."""
        nbytes = rows * cols * torch.empty(0, dtype=dtype).element_size()
        offset = self._cursor
        if offset + nbytes > self.nbytes:
            raise ValueError("arena exhausted")
        self._cursor = offset + ((nbytes + 255) // 256) * 256
        agree("the carving of the arena", (offset, rows, cols, str(dtype)), self.group)
        return PeerMatrix(self, offset, rows, cols, dtype)

    def new_site(self) -> int:
        """A barrier site id (one per exchange point of a step); every rank must ask in the same order."""
        site = self._sites
        if site >= 64:
            raise ValueError("at most 64 barrier sites per arena")
        self._sites += 1
        return site

    # ---- synchronisation
    def barrier(self, site: int, *, timeout_us: int = 0, dependent_launch: bool = False) -> None:
        """Launched by every rank on its current stream after the kernels that stored into the arenas: returns
        (on the device) once every rank has reached the same barrier of ``site``; bounded by ``timeout_us``
        (default one second), after which :func:`fault_flags` reports the late ranks."""
        with torch.cuda.device(self.device):
            status = _native.lib().xdk_peer_barrier(self._arena_ptrs, self.rank, self.world, site, timeout_us,
                                                    _native.XDK_DEPENDENT_LAUNCH if dependent_launch else 0,
                                                    _native.stream_ptr(self.device))
        _native.check(status, "xdk_peer_barrier")

    @staticmethod
    def fault_flags() -> int:
        """Bit p set: a barrier wait on rank p ran out of time on the current device (synchronises)."""
        return int(_native.lib().xdk_peer_fault_flags())

    def close(self) -> None:
        """Unmap the peers' arenas and free the local one (call after the last kernel has completed, and after a
        host-side barrier: a peer may still be storing into this arena until then)."""
        if self._closed:
            return
        self._closed = True
        lib = _native.lib()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            for ptr in self._opened:
                lib.xdk_peer_close(ctypes.c_void_p(ptr))
            lib.xdk_peer_free(ctypes.c_void_p(self.bases[self.rank]))
