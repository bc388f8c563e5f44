"""Peer-mapped device memory for one process per GPU on a single NVSwitch node.

Every rank allocates its buffers with ``cudaMalloc`` (through the kernel library, outside the
PyTorch caching allocator so the allocation can be exported), publishes the CUDA IPC handle
through one ``all_gather_object`` at set-up, and maps every peer's allocation.  Kernels then
receive a small device table of base pointers (one per rank) and address remote memory with
ordinary loads / stores / reductions: the clip-weighted weight-gradient kernel reduces its
output tiles into the owner's gradient shard, and the shard step stores updated bf16
parameters into every rank's parameter buffer.  No TMA load ever targets a peer mapping.

With a single rank the same objects are plain local tensors and the tables hold one pointer.

Rank-to-rank ordering uses :meth:`PeerGroup.barrier`: a one-warp kernel that publishes an epoch
number into every peer's flag array with a system-scope release store and waits, for a bounded
time, until all flags of its own array reach the epoch.  On expiry it records a status code
instead of spinning forever; the host raises :class:`opaque_b200.ops.DeviceWaitTimeout`.

Reference counterpart: none (packages/opaque-engine/src/opaque/api/engine/distributed uses NCCL
all-reduce only; see distributed/gradients.py:183-193 for the path this replaces).
"""
from __future__ import annotations

import ctypes
from typing import Sequence

import torch
import torch.distributed as dist

from ..ops import lib

_DTYPE_SIZE = {torch.float32: 4, torch.bfloat16: 2, torch.int32: 4, torch.int64: 8, torch.float16: 2}


def _tensor_from_ptr(ptr: int, numel: int, dtype: torch.dtype, device: torch.device, owner=None) -> torch.Tensor:
    """Wrap raw device memory as a tensor through the ``__cuda_array_interface__`` protocol."""
    typestr = {torch.float32: "<f4", torch.bfloat16: "<u2", torch.int32: "<i4", torch.int64: "<i8",
               torch.float16: "<f2"}[dtype]

    class _Holder:
        pass
    h = _Holder()
    h.__cuda_array_interface__ = {"shape": (numel,), "typestr": typestr, "data": (ptr, False), "version": 3,
                                  "strides": None}
    h.owner = owner
    t = torch.as_tensor(h, device=device)
    if dtype == torch.bfloat16:
        t = t.view(torch.bfloat16)
    return t


class PeerBuffer:
    """One logical buffer that exists on every rank; rank r's copy is mapped into every process."""

    def __init__(self, group: "PeerGroup", numel: int, dtype: torch.dtype):
        self.group, self.numel, self.dtype = group, numel, dtype
        nbytes = max(numel * _DTYPE_SIZE[dtype], 256)
        dev = group.device
        self._raw_ptrs: list[int] = []
        self._owned: int | None = None
        self._opened: list[int] = []
        if group.world == 1 or not group.use_ipc:
            self.local = torch.zeros(numel, dtype=dtype, device=dev)
            self._raw_ptrs = [self.local.data_ptr()]
        else:
            L = lib.load()
            p = ctypes.c_void_p()
            lib.check(L.ob_ipc_alloc(ctypes.byref(p), nbytes), "peer buffer allocation")
            self._owned = p.value
            handle = ctypes.create_string_buffer(64)
            lib.check(L.ob_ipc_get_handle(p, handle), "cudaIpcGetMemHandle")
            handles: list = [None] * group.world
            dist.all_gather_object(handles, bytes(handle.raw), group=group.pg)
            for r, h in enumerate(handles):
                if r == group.rank:
                    self._raw_ptrs.append(p.value)
                    continue
                q = ctypes.c_void_p()
                buf = ctypes.create_string_buffer(h, 64)
                lib.check(L.ob_ipc_open_handle(buf, ctypes.byref(q)), "cudaIpcOpenMemHandle")
                self._raw_ptrs.append(q.value)
                self._opened.append(q.value)
            self.local = _tensor_from_ptr(p.value, numel, dtype, dev, owner=self)
        self.table = torch.tensor(self._raw_ptrs, dtype=torch.int64, device=dev)

    def peer_ptr(self, rank: int) -> int:
        return self._raw_ptrs[rank]

    def peer_view(self, rank: int) -> torch.Tensor:
        """Tensor view of rank ``rank``'s copy (for tests and checkpoint gathers)."""
        if rank == self.group.rank or len(self._raw_ptrs) == 1:
            return self.local
        return _tensor_from_ptr(self._raw_ptrs[rank], self.numel, self.dtype, self.group.device, owner=self)

    def close(self) -> None:
        if self._owned is None:
            return
        L = lib.load()
        torch.cuda.synchronize(self.group.device)
        for q in self._opened:
            L.ob_ipc_close_handle(ctypes.c_void_p(q))
        self._opened = []
        if self.group.pg is not None:
            dist.barrier(group=self.group.pg)
        L.ob_ipc_free(ctypes.c_void_p(self._owned))
        self._owned = None


class PeerGroup:
    """The ranks of one node that share peer memory, plus their flag barrier."""

    def __init__(self, device: torch.device | None = None, pg=None, *, use_ipc: bool | None = None,
                 wait_budget_s: float | None = None):
        """``wait_budget_s``: how long a rank waits at the device barrier for its peers before it gives up with a
        status code (default 30 s, or the environment variable ``OPAQUE_B200_PEER_WAIT_S``).  It has to exceed the
        worst host-side skew between ranks inside one step — a first CUDA-graph capture, an out-of-memory retry, a
        checkpoint write on one rank — and stays far below a collective-library timeout."""
        if wait_budget_s is None:
            import os
            wait_budget_s = float(os.environ.get("OPAQUE_B200_PEER_WAIT_S", "30"))
        self.pg = pg if pg is not None else (dist.group.WORLD if dist.is_initialized() else None)
        self.world = dist.get_world_size(self.pg) if self.pg is not None else 1
        self.rank = dist.get_rank(self.pg) if self.pg is not None else 0
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.use_ipc = (self.world > 1) if use_ipc is None else use_ipc
        self.wait_budget_s = wait_budget_s
        self.status = lib.StatusWord(self.device)
        self._epoch = 0
        self.flags = PeerBuffer(self, 64, torch.int32) if self.world > 1 else None
        self.buffers: list[PeerBuffer] = []
        if self.flags is not None:
            self.buffers.append(self.flags)

    def buffer(self, numel: int, dtype: torch.dtype) -> PeerBuffer:
        b = PeerBuffer(self, numel, dtype)
        self.buffers.append(b)
        return b

    def barrier(self) -> None:
        """Device-side barrier on the current stream (ordering of peer writes between steps)."""
        if self.world == 1:
            return
        self._epoch += 1
        rc = lib.load().ob_peer_barrier(self.flags.table.data_ptr(), self.flags.local.data_ptr(), self.rank,
                                        self.world, self._epoch, self.status.ptr(), self.wait_budget_s, lib.stream())
        lib.check(rc, "peer_barrier")

    def check(self, what: str = "peer step") -> None:
        """Raise :class:`DeviceWaitTimeout` if a bounded wait expired since the last check (one D2H read)."""
        self.status.raise_if_set(what)

    def close(self) -> None:
        for b in self.buffers:
            b.close()
        self.buffers = []


class PeerLeftError(RuntimeError):
    """A rank announced that it leaves the job; raised on the others BEFORE they launch their next device barrier."""


class Liveness:
    """Host-side leave notices through the rendezvous key-value store.

    A rank that stops (preemption, an exception it handles, end of its data) calls :meth:`announce_leave` between
    steps, after its last kernel has completed; every other rank calls :meth:`check` before a step and gets a
    :class:`PeerLeftError` instead of waiting for that rank's flag on the device until the bounded wait runs out.
    Only ``set`` / ``check`` on the store are used, so a rank that vanished without a notice costs nothing here — it is
    caught by the bounded device wait (``DeviceWaitTimeout``) or the process-group timeout instead.
    """

    def __init__(self, rank: int, world: int, store=None, prefix: str = "opaque_b200/left"):
        if store is None:
            from torch.distributed.distributed_c10d import _get_default_store
            store = _get_default_store()
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def announce_leave(self, reason: str = "") -> None:
        self.store.set(self._key(self.rank), reason or "left")

    def left(self) -> list[int]:
        return [r for r in range(self.world) if r != self.rank and self.store.check([self._key(r)])]

    def check(self) -> None:
        gone = self.left()
        if gone:
            why = {r: self.store.get(self._key(r)).decode(errors="replace") for r in gone}
            raise PeerLeftError(f"rank(s) {gone} left the job: {why}")
