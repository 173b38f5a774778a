"""Symmetric (peer-mapped) device memory.

``SymmetricPool`` hands out buffers that every rank of the group allocates in the same order
with the same size; each rank can then address every peer's copy directly over NVLink.  The
mapping itself comes from ``torch.distributed._symmetric_memory`` (CUDA VMM handles exchanged
through the process group); what travels through the mapped pointers is decided by the kernels
of this package.  ``peer_pointers(t)`` returns the table of peer base addresses of ``t`` as a
CPU ``int64`` tensor (kernels take it by value), and ``flags`` is a small symmetric ``int32``
array used for version / ready words with ``st.release.sys`` / ``ld.acquire.sys``.
"""

from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist


class CollectiveTimeout(RuntimeError):
    """A bounded device-side wait expired (a peer did not arrive in time)."""


class SymmetricPool:
    FLAG_SLOTS = 1024

    def __init__(self, mesh: Any, group: Any = None) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        self._symm_mem = symm_mem
        self.mesh = mesh
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self._handles: dict[int, Any] = {}
        self._tables: dict[int, torch.Tensor] = {}
        self._keep: list[torch.Tensor] = []
        self.bytes_allocated = 0
        self.flags = self.allocate(self.FLAG_SLOTS, torch.int32, torch.device("cuda", torch.cuda.current_device()),
                                   "flags").zero_()
        torch.cuda.synchronize()
        self.barrier()

    def allocate(self, numel: int, dtype: torch.dtype, device: Any, tag: str = "") -> torch.Tensor:
        """Collective: every rank must call with identical arguments in identical order."""
        del tag
        t = self._symm_mem.empty(int(numel), dtype=dtype, device=device)
        handle = self._symm_mem.rendezvous(t, self.group)
        self._handles[t.data_ptr()] = handle
        self._keep.append(t)
        self.bytes_allocated += t.numel() * t.element_size()
        return t

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

    def supports_multicast(self, tensor: torch.Tensor) -> bool:
        return bool(getattr(self.handle_of(tensor), "has_multicast_support", lambda: False)())

    def barrier(self) -> None:
        """All peers' previously enqueued work on the current stream is complete afterwards."""
        self.handle_of(self.flags).barrier(channel=0)

    def check_wait(self, status: torch.Tensor, what: str) -> None:
        """Raise :class:`CollectiveTimeout` if a ``wait_flag`` status word reports expiry."""
        code, seen = status.tolist()
        if code != 0:
            raise CollectiveTimeout(f"{what}: bounded wait expired on rank {self.rank} "
                                    f"(last value seen {seen})")
