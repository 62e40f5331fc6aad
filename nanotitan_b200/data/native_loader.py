"""Training batches from a packed token file through the extension's `TokenWindowLoader`.

Same batches as `DataLoader(PackedTokenDataset, sampler=DistributedSampler, drop_last=True)` - the
reference's loader (src/parallel/dp.py:84-100 over src/data/dataset.py:8-27) - in the same order: the
sampler still decides which samples this rank visits, and `loader.sampler.set_epoch()` works as before.
What differs is who builds a batch: C++ threads widen the uint16 windows straight into a ring of pinned
int64 buffers, so a step's input is ready for its host-to-device copy without a Python call per sample
and without worker processes.

On a GPU the yielded tensors are views of the ring (pinned): a batch stays valid until two more have been
asked for.  Before a slot is refilled the loader waits on a CUDA event recorded when the following batch
was requested, i.e. after the consumer enqueued the copies that read the slot.  On CPU every batch is a
private copy.
"""
from __future__ import annotations

from collections import deque

import torch


class NativeTokenLoader:
    def __init__(self, path: str, seq_len: int, batch_size: int, sampler, device: torch.device, depth: int = 4,
                 threads: int = 2, timeout_s: float = 120.0, ext=None, views: bool | None = None):
        if ext is None:
            from nanotitan_b200.ops.ext import get_ext

            ext = get_ext()
        assert depth >= 3, "two batches stay with the consumer while the next one is filled"
        self.sampler, self.batch_size, self.seq_len, self.depth = sampler, batch_size, seq_len, depth
        self.on_gpu = device.type == "cuda"
        self.views = self.on_gpu if views is None else views  # hand out ring slots themselves, not copies
        self.timeout_ms = int(timeout_s * 1000)
        self._loader = ext.TokenWindowLoader(str(path), seq_len, batch_size, depth, threads)
        self.num_sequences = int(self._loader.num_sequences)
        self._ring = torch.empty(depth * int(self._loader.slot_elements), dtype=torch.int64, pin_memory=self.on_gpu)
        self._loader.set_ring(self._ring, depth)
        self._slots = self._ring.view(depth, 2, batch_size, seq_len)
        self.skip_batches = 0  # the next epoch starts this many batches in (a resumed run); then back to 0

    def __len__(self) -> int:
        return len(self.sampler) // self.batch_size

    def __iter__(self):
        order = torch.tensor(list(iter(self.sampler)), dtype=torch.int64)
        order, self.skip_batches = order[self.skip_batches * self.batch_size :].contiguous(), 0
        self._loader.start(order)
        held: deque[tuple[int, object]] = deque()  # (slot, event that covers the consumer's use of it)
        try:
            while True:
                if held and self.on_gpu and held[-1][1] is None:
                    # everything the consumer enqueued for the previous batch lies before this event
                    event = torch.cuda.Event()
                    event.record()
                    held[-1] = (held[-1][0], event)
                while len(held) > (1 if self.views else 0):
                    slot, event = held.popleft()
                    if event is not None:
                        event.synchronize()
                    self._loader.release(slot)
                slot = self._loader.next(self.timeout_ms)
                if slot < 0:
                    return
                held.append((slot, None))
                x, y = self._slots[slot, 0], self._slots[slot, 1]
                yield (x, y) if self.views else (x.clone(), y.clone())
        finally:
            self._loader.stop()


def skip_batches(loader, n: int):
    """Iterator over `loader`'s next epoch without its first `n` batches.  The native loader never builds
    them; a torch DataLoader has to produce and drop them."""
    if n and isinstance(loader, NativeTokenLoader):
        loader.skip_batches = n
        return iter(loader)
    it = iter(loader)
    for _ in range(n):
        if next(it, None) is None:
            break
    return it


def make_train_loader(dataset, sampler, batch_size: int, device: torch.device, num_workers: int):
    """The native loader for packed token files when the extension is built (and `NT_NATIVE_LOADER` is not 0),
    else a torch DataLoader."""
    import os

    from torch.utils.data import DataLoader

    from nanotitan_b200.data.dataset import PackedTokenDataset
    from nanotitan_b200.ops.ext import have_ext

    if isinstance(dataset, PackedTokenDataset) and have_ext() and os.environ.get("NT_NATIVE_LOADER", "1") != "0":
        return NativeTokenLoader(dataset.path, dataset.seq_len, batch_size, sampler, device, threads=max(1, min(num_workers, 4)))
    return DataLoader(dataset, batch_size=batch_size, shuffle=False, sampler=sampler, num_workers=num_workers,
                      pin_memory=device.type == "cuda", drop_last=True)
