"""Symmetric (peer-mapped) device memory, flags and the bounded flag barrier.

``SymmetricPool`` hands out buffers that every rank of the group allocates in the same order
with the same size; each rank can then address every peer's copy directly over NVLink.  The
mapping itself comes from ``torch.distributed._symmetric_memory`` (CUDA VMM handles exchanged
through the process group); what travels through the mapped pointers is decided by the kernels
of this package.  ``peer_pointers(t)`` returns the table of peer base addresses of ``t`` as a
CPU ``int64`` tensor (kernels take it by value).

Synchronisation between ranks is built from one small symmetric ``int32`` flag array:

* slot ``BARRIER_BASE + r`` of every rank's array is written only by rank ``r``.  ``barrier()``
  launches one tiny kernel that stores the next epoch into this rank's slot on every peer
  (``st.release.sys``) and then polls its own array until every peer's slot has reached the
  epoch (``ld.acquire.sys``).  The poll is bounded by wall-clock time: when a peer never
  arrives the kernel records the fact in the pool's status word and returns, the stream keeps
  running, and the next :meth:`check` on the host raises :class:`CollectiveTimeout`.  Nothing
  in this file can spin without limit, and nothing traps.
* ``signal`` / ``wait`` expose the two halves separately for pipelined protocols (gradient
  buckets, weight versions): the slot ranges are handed out by :meth:`reserve_slots`.

The library's own symmetric-memory barrier is not used: its wait either never gives up
(``timeout_ms=0``) or traps the context when it does.  NVLink multicast bindings are switched
off for the mapping (``TORCH_SYMM_MEM_DISABLE_MULTICAST``) because every kernel here uses plain
peer loads and stores, and a rank that exits while bound to a multicast object can raise
faults on its peers.
"""

from __future__ import annotations

import os
from typing import Any

import torch
import torch.distributed as dist

os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")


class CollectiveTimeout(RuntimeError):
    """A bounded device-side wait expired (a peer did not arrive in time)."""


def default_timeout_s() -> float:
    """Bound of every flag wait; ``VRL_COLLECTIVE_TIMEOUT_S`` overrides the 60 s default."""
    try:
        return float(os.environ.get("VRL_COLLECTIVE_TIMEOUT_S", "60"))
    except ValueError:
        return 60.0


class SymmetricPool:
    FLAG_SLOTS = 1024
    BARRIER_BASE = 0            # slots [0, 16): one arrival word per rank
    FIRST_FREE_SLOT = 64        # [16, 64) is kept for fixed uses (weight versions start at 16)

    def __init__(self, mesh: Any, group: Any = None, timeout_s: float | None = None) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        self._symm_mem = symm_mem
        self.mesh = mesh
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        if self.world > 16:
            raise ValueError("SymmetricPool supports at most 16 ranks per group")
        self.timeout_s = float(timeout_s) if timeout_s is not None else default_timeout_s()
        self._handles: dict[int, Any] = {}
        self._tables: dict[int, torch.Tensor] = {}
        self._keep: list[torch.Tensor] = []
        self._next_slot = self.FIRST_FREE_SLOT
        self._epoch = 0
        self.bytes_allocated = 0
        self.barriers = 0
        device = torch.device("cuda", torch.cuda.current_device())
        self.device = device
        self.flags = self.allocate(self.FLAG_SLOTS, torch.int32, device, "flags").zero_()
        # {code, slot, last value seen, value expected}; written by a wait that gave up
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        torch.cuda.synchronize()
        # every rank's flags are zero before anybody signals: the one place that needs a
        # host-side rendezvous (the flag barrier itself is only valid afterwards)
        dist.barrier(group=self.group)
        self.barrier()
        self.check("symmetric pool set-up")

    # -- allocation ------------------------------------------------------------------------
    def allocate(self, numel: int, dtype: torch.dtype, device: Any, tag: str = "") -> torch.Tensor:
        """Collective: every rank must call with identical arguments in identical order."""
        del tag
        t = self._symm_mem.empty(int(numel), dtype=dtype, device=device)
        handle = self._symm_mem.rendezvous(t, self.group)
        self._handles[t.data_ptr()] = handle
        self._keep.append(t)
        self.bytes_allocated += t.numel() * t.element_size()
        return t

    def reserve_slots(self, count: int) -> int:
        """First of ``count`` consecutive flag slots (same answer on every rank when every rank
        reserves in the same order)."""
        first = self._next_slot
        if first + count > self.FLAG_SLOTS:
            raise RuntimeError("out of flag slots")
        self._next_slot += int(count)
        return first

    def handle_of(self, tensor: torch.Tensor) -> Any:
        handle = self._handles.get(tensor.data_ptr())
        if handle is None:
            raise KeyError("tensor was not allocated from this SymmetricPool")
        return handle

    def peer_pointers(self, tensor: torch.Tensor) -> torch.Tensor:
        key = tensor.data_ptr()
        table = self._tables.get(key)
        if table is None:
            handle = self.handle_of(tensor)
            table = torch.tensor([int(p) for p in handle.buffer_ptrs], dtype=torch.int64)
            self._tables[key] = table
        return table

    def peer_pointers_at(self, tensor: torch.Tensor, offset_elems: int) -> torch.Tensor:
        """Peer addresses of element ``offset_elems`` of a pool allocation."""
        return self.peer_pointers(tensor) + int(offset_elems) * tensor.element_size()

    # -- synchronisation -----------------------------------------------------------------------
    def barrier(self, timeout_s: float | None = None) -> None:
        """Every peer's work enqueued before its matching ``barrier()`` is complete and visible
        to work this rank enqueues afterwards (on the current stream).  Bounded; see
        :meth:`check`."""
        from visionrl_b200.ops import _ext

        self._epoch += 1
        self.barriers += 1
        _ext.load().flag_barrier(self.peer_pointers(self.flags), self.flags, self.BARRIER_BASE,
                                 self.world, self.rank, self._epoch,
                                 self.timeout_s if timeout_s is None else float(timeout_s),
                                 self.status)

    def signal(self, slot: int, value: int) -> None:
        """Store ``value`` into ``slot`` of every rank's flag array, ordered after this rank's
        earlier work on the current stream."""
        from visionrl_b200.ops import _ext

        _ext.load().flag_signal(self.peer_pointers(self.flags), self.flags, int(slot), self.world,
                                int(value))

    def wait(self, slot0: int, count: int, value: int, timeout_s: float | None = None) -> None:
        """Hold the current stream until local slots ``slot0 … slot0+count-1`` reached ``value``
        (bounded; an expiry is reported by the next :meth:`check`)."""
        from visionrl_b200.ops import _ext

        _ext.load().flag_wait(self.flags, int(slot0), int(count), int(value),
                              self.timeout_s if timeout_s is None else float(timeout_s), self.status)

    def check(self, what: str = "collective") -> None:
        """Read the status word (one small device-to-host copy, synchronises the stream) and raise
        :class:`CollectiveTimeout` if any bounded wait since the last check gave up."""
        code, slot, seen, expected = self.status.tolist()
        if code != 0:
            self.status.zero_()
            raise CollectiveTimeout(
                f"{what}: bounded wait expired on rank {self.rank} (flag slot {slot}: last value "
                f"seen {seen}, expected {expected}); a peer did not arrive within the time limit")

    def check_wait(self, status: torch.Tensor, what: str) -> None:
        """Raise :class:`CollectiveTimeout` if a ``wait_flag`` status word reports expiry."""
        code, seen = status.tolist()[:2]
        if code != 0:
            raise CollectiveTimeout(f"{what}: bounded wait expired on rank {self.rank} "
                                    f"(last value seen {seen})")
