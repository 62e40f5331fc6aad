"""Symmetric memory for the fused collective kernels: where the allocations come from.

Both providers give the same three things for a group of GPUs on one machine: `empty()` - a tensor over
this rank's piece of an allocation every rank made at the same call; `peer_ptrs(t)` - every rank's
address of that allocation as seen from this rank (peer loads and stores over NVLink); and
`multicast_ptr(t)` - the address of the NVSwitch multicast mapping for `multimem.*` (0 when the group
has none).

* `TorchSymmetricMemory` (default) - `torch.distributed._symmetric_memory`.
* `NativeSymmetricMemory` (`NT_SYMM_HEAP=native`) - this library's own heap in C++
  (csrc/runtime/symmetric_heap.h): `cuMemCreate` pieces exported as file descriptors, passed between
  the ranks over unix sockets, mapped side by side, and bound to a `cuMulticastCreate` object.  Every
  wait in its rendezvous has a time limit (`NT_SYMM_TIMEOUT_MS`, default 60 s).

The reference has no counterpart: it reaches other GPUs through NCCL only (src/parallel/ep.py:97-130,
src/parallel/dp.py:182-187).
"""
from __future__ import annotations

import os
import uuid

import torch
import torch.distributed as dist


class TorchSymmetricMemory:
    name = "torch"

    def __init__(self, group, device: torch.device):
        import torch.distributed._symmetric_memory as symm_mem

        self._symm_mem, self.group, self.device = symm_mem, group, device
        self._handles: dict[int, object] = {}

    def empty(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        t = self._symm_mem.empty(numel, dtype=dtype, device=self.device)
        self._handles[t.data_ptr()] = self._symm_mem.rendezvous(t, self.group)
        return t

    def peer_ptrs(self, t: torch.Tensor) -> list[int]:
        return list(self._handles[t.data_ptr()].buffer_ptrs)

    def multicast_ptr(self, t: torch.Tensor) -> int:
        return int(getattr(self._handles[t.data_ptr()], "multicast_ptr", 0) or 0)


class NativeSymmetricMemory:
    name = "native"

    def __init__(self, group, device: torch.device, ext=None):
        if ext is None:
            from nanotitan_b200.ops.ext import get_ext

            ext = get_ext()
        self._ext, self.group, self.device = ext, group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        # one socket name space per heap: the group's first rank picks it, the others learn it from there
        job = [f"{os.getpid()}-{uuid.uuid4().hex[:12]}" if self.rank == 0 else None]
        dist.broadcast_object_list(job, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        timeout_ms = int(float(os.environ.get("NT_SYMM_TIMEOUT_MS", "60000")))
        self._heap = ext.symm_heap_open(job[0], self.rank, self.world, device.index or 0, timeout_ms)
        self._records: dict[int, tuple[list[int], int, int, torch.Tensor]] = {}

    def empty(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        raw, peers, mc, alloc_id = self._ext.symm_heap_alloc(self._heap, nbytes, True)
        t = raw.view(dtype)
        self._records[t.data_ptr()] = (list(peers), int(mc), int(alloc_id), raw)
        return t

    def peer_ptrs(self, t: torch.Tensor) -> list[int]:
        return self._records[t.data_ptr()][0]

    def multicast_ptr(self, t: torch.Tensor) -> int:
        return self._records[t.data_ptr()][1]

    def free(self, t: torch.Tensor) -> None:
        """Collective; no kernel on any rank may still use the allocation."""
        _, _, alloc_id, _ = self._records.pop(t.data_ptr())
        self._ext.symm_heap_free(self._heap, alloc_id)

    def close(self) -> None:
        for ptr in list(self._records):
            _, _, alloc_id, _ = self._records.pop(ptr)
            self._ext.symm_heap_free(self._heap, alloc_id)
        self._ext.symm_heap_close(self._heap)


def make_provider(group, device: torch.device):
    kind = os.environ.get("NT_SYMM_HEAP", "torch")
    if kind == "native":
        return NativeSymmetricMemory(group, device)
    if kind != "torch":
        raise ValueError(f"NT_SYMM_HEAP={kind!r}: expected 'torch' or 'native'")
    return TorchSymmetricMemory(group, device)
