"""Fused gradient-bucket engine: all-reduce + 1/N scale (+ AdamW) in one sm_100a kernel.

`BucketEngine` owns, for one data-parallel group, the symmetric (peer-mapped, and NVLS
multicast-bound when the hardware offers it) memory the buckets live in, a flag pad for
the in-kernel barriers, and a side stream.  `ReducerV1` calls `launch` from the autograd
hook that completes a bucket - the kernel then overlaps the rest of backward - and
`finish` before the optimizer step.  When a `FusedAdamW` is bound, the same kernel updates
the owner's slice of the fp32 master weights and broadcasts the new bf16 parameters, so
`optimizer.step()` has nothing left to do for those buckets.

Symmetric memory comes from a provider in `parallel/symm_memory.py` (torch's, or this library's own heap)
(plumbing); every byte that crosses NVLink is moved by `bucket_allreduce_kernel`.
Set `NT_FUSED_ALLREDUCE=0` to keep the NCCL all-reduce (the measured baseline).  The reference copies every
gradient into a bucket, all-reduces it with NCCL, divides and copies back (src/parallel/reducer.py:103-145),
then runs a separate optimizer pass.
"""
from __future__ import annotations

import logging
import os

import torch
import torch.distributed as dist

logger = logging.getLogger(__name__)

MAX_SLOTS = 256
MAX_RANKS = 16
FLAG_WORDS = MAX_SLOTS * 2 * MAX_RANKS


def owned_slice(numel: int, world: int, rank: int) -> tuple[int, int]:
    """[lo, hi) of a `numel`-element bucket that rank `rank` of `world` reduces and updates: whole
    16-byte vectors (8 16-bit elements), ceil-divided over the ranks - the split
    `bucket_allreduce_kernel` computes on the device."""
    per = ((numel // 8 + world - 1) // world) * 8
    lo = min(numel, per * rank)
    return lo, min(numel, lo + per)


class BucketEngine:
    def __init__(self, group, device: torch.device):
        from nanotitan_b200.parallel.symm_memory import make_provider

        self.symm = make_provider(group, device)
        self.group = group
        self.device = device
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.use_multicast = os.environ.get("NT_MULTIMEM", "1") != "0"
        self.wait_ms = float(os.environ.get("NT_COMM_WAIT_MS", "60000"))
        self.blocks = int(os.environ.get("NT_ALLREDUCE_BLOCKS", "64"))
        self.stream = torch.cuda.Stream(device=device)
        self.flags = self.alloc(FLAG_WORDS, torch.int32, device)
        self.flags.zero_()
        self.flag_peers = self._peer_table(self.flags)
        self.block_counter = torch.zeros(MAX_SLOTS, dtype=torch.int32, device=device)
        # per-slot launch counts, advanced by the kernel itself: a launch has the same arguments every step
        self.epoch_counters = torch.zeros(MAX_SLOTS, dtype=torch.int32, device=device)
        self.slots: dict[int, int] = {}
        self.optim: dict[int, tuple] = {}
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    # ------------------------------------------------------------------ memory
    def alloc(self, numel: int, dtype: torch.dtype, device) -> torch.Tensor:
        """Symmetric allocation; every rank of the group must call in the same order."""
        return self.symm.empty(numel, dtype)

    def _peer_table(self, t: torch.Tensor) -> torch.Tensor:
        return torch.tensor(self.symm.peer_ptrs(t), dtype=torch.int64)

    def _multicast(self, t: torch.Tensor) -> int:
        if not self.use_multicast:
            return 0
        return self.symm.multicast_ptr(t)

    def owned_slice(self, numel: int) -> tuple[int, int]:
        return owned_slice(numel, self.world, self.rank)

    # ------------------------------------------------------------------ reducer interface
    def register(self, bucket) -> None:
        key = id(bucket)
        if key not in self.slots:
            self.slots[key] = len(self.slots)
            assert self.slots[key] < MAX_SLOTS, "too many buckets for the flag pad"
            bucket._peers = self._peer_table(bucket.buffer)
            bucket._mc = self._multicast(bucket.buffer)

    def bind_optimizer(self, bucket, flat_param, master, exp_avg, exp_avg_sq, optimizer) -> None:
        self.register(bucket)
        self.optim[id(bucket)] = (flat_param, self._peer_table(flat_param), self._multicast(flat_param),
                                  master, exp_avg, exp_avg_sq, optimizer)

    def launch(self, reducer, bucket):
        from nanotitan_b200.ops.ext import get_ext

        self.register(bucket)
        key = id(bucket)
        ready = torch.cuda.Event()
        ready.record()
        self.stream.wait_event(ready)
        bound = self.optim.get(key)
        with torch.cuda.stream(self.stream):
            if bound is not None:
                flat_param, param_peers, param_mc, master, m, v, opt = bound
                hyper = opt.param_groups[0]
                get_ext().bucket_allreduce(
                    bucket.buffer, bucket._mc, bucket._peers, param_mc, param_peers, master, m, v, self.flags,
                    self.flag_peers, self.block_counter, self.rank, self.world, self.slots[key], self.epoch_counters,
                    opt.next_step(), opt.device_constants(), hyper["lr"], hyper["betas"][0], hyper["betas"][1], hyper["eps"],
                    hyper["weight_decay"], self.blocks, self.wait_ms)
            else:
                get_ext().bucket_allreduce(
                    bucket.buffer, bucket._mc, bucket._peers, 0, bucket._peers, None, None, None, self.flags,
                    self.flag_peers, self.block_counter, self.rank, self.world, self.slots[key], self.epoch_counters,
                    1, None, 0.0, 0.9, 0.999, 1e-8, 0.0, self.blocks, self.wait_ms)
            done = torch.cuda.Event()
            done.record()
        return done

    def finish(self, reducer, bucket) -> None:
        if bucket.work is not None:
            torch.cuda.current_stream().wait_event(bucket.work)

    def owns_update(self, bucket) -> bool:
        return id(bucket) in self.optim


def attach_if_possible(reducer) -> bool:
    """Give `reducer` a `BucketEngine` when its group spans several GPUs with peer access.
    Must run before the reducer allocates its buckets (see `make_engine`)."""
    return reducer.bucket_engine is not None


def make_engine(group, group_size: int, device: torch.device):
    """-> BucketEngine, or None for a single rank or when switched off (`NT_FUSED_ALLREDUCE=0`).
    A set-up failure raises: the NCCL path is never taken silently."""
    if group is None or group_size < 2 or device.type != "cuda" or group_size > MAX_RANKS:
        return None
    if os.environ.get("NT_FUSED_ALLREDUCE", "1") == "0":
        return None
    try:
        return BucketEngine(group, device)
    except Exception as exc:
        raise RuntimeError(
            f"the fused all-reduce engine could not be set up ({type(exc).__name__}: {exc}); "
            "set NT_FUSED_ALLREDUCE=0 to run the NCCL all-reduce on purpose") from exc
