"""Bucketed gradient reducer driven by autograd hooks.

Contract of the reference's `ReducerV1` (src/parallel/reducer.py:7-145): parameters
are walked in reverse registration order into per-dtype buckets of at most
`bucket_size` MiB; a post-accumulate-grad hook marks a parameter ready; a full bucket
starts its all-reduce at once, overlapping the rest of backward; parameters whose hook
never fired (unused experts) are zero-filled by `prepare_missing_grad`;
`finalize_backward` waits and leaves the group mean in every `param.grad`.

What differs: every `param.grad` *is* a view into its bucket's flat buffer, so there
is no copy-in before and no copy-back after the collective (the reference makes three
extra passes over all gradients per step).  On GPUs the collective of a bucket is the
fused kernel of `nanotitan_b200.parallel.fused_allreduce` (in-switch `multimem`
reduction or peer loads over NVLink, with the 1/N scale and optionally the AdamW
update in the same kernel) when a `bucket_engine` is attached; otherwise it is
`dist.all_reduce` (NCCL on GPUs, gloo on CPU) followed by one in-place scale.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.distributed as dist
import torch.nn as nn


@dataclass
class Bucket:
    index: int
    dtype: torch.dtype
    device: torch.device
    params: list[nn.Parameter] = field(default_factory=list)
    spans: list[tuple[int, int]] = field(default_factory=list)
    size_bytes: int = 0
    numel: int = 0
    ready_count: int = 0
    work: object | None = None
    buffer: torch.Tensor | None = None  # flat gradients; every param.grad views into it
    launched: bool = False
    launched_this_step: bool = False  # consumed by a bound optimizer


def plan_buckets(params, bucket_bytes: int) -> list[Bucket]:
    """Reverse-order, per-dtype, size-capped bucket assignment (pure function, no allocation)."""
    buckets: list[Bucket] = []
    open_by_dtype: dict[torch.dtype, Bucket] = {}
    for p in reversed(list(params)):
        nbytes = p.numel() * p.element_size()
        cur = open_by_dtype.get(p.dtype)
        if cur is None or cur.size_bytes + nbytes > bucket_bytes:
            cur = Bucket(index=len(buckets), dtype=p.dtype, device=p.device)
            buckets.append(cur)
            open_by_dtype[p.dtype] = cur
        # keep every span 16-byte aligned so vector / bulk kernels can address it
        align = max(1, 16 // p.element_size())
        start = (cur.numel + align - 1) // align * align
        cur.spans.append((start, start + p.numel()))
        cur.params.append(p)
        cur.numel = start + p.numel()
        cur.size_bytes += nbytes
    return buckets


class ReducerV1:
    def __init__(self, params, group_size: int, process_group, bucket_size: int, allocator=None, engine=None):
        self.group_size = group_size
        self.process_group = process_group
        self.params = [p for p in params if p.requires_grad]
        self.bucket_size = bucket_size * 1024 * 1024
        self.backward_grad_sync = False
        self.ready_for_sync: set[nn.Parameter] = set()
        self.bucket_engine = engine  # fused all-reduce (+ AdamW) kernels; None = dist.all_reduce
        self._allocator = allocator if engine is None else engine.alloc
        self.initialize_buckets()
        self.hook_handles = [
            p.register_post_accumulate_grad_hook(self.reduce_grad) for p in self.params
        ]

    # ------------------------------------------------------------------ layout
    def initialize_buckets(self) -> None:
        self.buckets = plan_buckets(self.params, self.bucket_size)
        self.param_to_bucket: dict[nn.Parameter, int] = {}
        self.param_to_offset: dict[nn.Parameter, tuple[int, int]] = {}
        for b in self.buckets:
            padded = (b.numel + 127) // 128 * 128
            if self._allocator is not None:
                b.buffer = self._allocator(padded, b.dtype, b.device)
                b.buffer.zero_()
            else:
                b.buffer = torch.zeros(padded, dtype=b.dtype, device=b.device)
            for p, span in zip(b.params, b.spans):
                self.param_to_bucket[p] = b.index
                self.param_to_offset[p] = span
        self.attach_grad_views()

    def grad_view(self, p: nn.Parameter) -> torch.Tensor:
        lo, hi = self.param_to_offset[p]
        return self.buckets[self.param_to_bucket[p]].buffer[lo:hi].view_as(p)

    def attach_grad_views(self) -> None:
        for p in self.params:
            p.grad = self.grad_view(p)
            # Kernels that produce this parameter's gradient may ask for its bucket slot and write
            # there directly (see `zero_grad(lazy=True)`).
            p._nt_grad_sink = (lambda q=p: self.grad_view(q))

    def zero_grad(self, lazy: bool = False) -> None:
        """Eager (default): one memset per bucket, every `param.grad` is its zeroed bucket view.

        Lazy: gradients are dropped (`param.grad = None`) and nothing is written.  The first
        gradient of a step is then *produced in place*: weight-gradient kernels write into the
        parameter's bucket slot (`_nt_grad_sink`) and autograd adopts that tensor as `.grad`, so the
        step has neither a zero-fill nor an add pass for those parameters; gradients that arrive as
        ordinary tensors are copied into their slot by the hook, and parameters that never get one
        are zero-filled by `prepare_missing_grad`."""
        if lazy:
            for p in self.params:
                p.grad = None
            return
        for b in self.buckets:
            b.buffer.zero_()
        for p in self.params:
            if p.grad is None or p.grad.data_ptr() != self.grad_view(p).data_ptr():
                p.grad = self.grad_view(p)

    # ------------------------------------------------------------------ hooks
    def reduce_grad(self, param: nn.Parameter) -> None:
        if not self.backward_grad_sync:
            return
        self.ready_for_sync.add(param)
        bucket = self.buckets[self.param_to_bucket[param]]
        view = self.grad_view(param)
        if param.grad is not None and param.grad.data_ptr() != view.data_ptr():
            view.copy_(param.grad)  # somebody replaced .grad; fold it back into the bucket
            param.grad = view
        bucket.ready_count += 1
        if bucket.ready_count == len(bucket.params):
            self._launch(bucket)

    def _launch(self, bucket: Bucket) -> None:
        bucket.launched = True
        bucket.launched_this_step = True
        if self._engine_for(bucket) is not None:
            bucket.work = self.bucket_engine.launch(self, bucket)
        elif self.group_size > 1:
            bucket.work = dist.all_reduce(
                bucket.buffer, op=dist.ReduceOp.SUM, group=self.process_group, async_op=True
            )
        else:
            bucket.work = None

    def _engine_for(self, bucket: Bucket):
        """The fused kernels take 16-bit buckets; anything else stays on dist.all_reduce."""
        if self.bucket_engine is not None and bucket.dtype in (torch.bfloat16, torch.float16):
            return self.bucket_engine
        return None

    def prepare_missing_grad(self) -> None:
        """Fire the hook of parameters autograd never reached (their grad view is already zero)."""
        for p in self.params:
            if p not in self.ready_for_sync:
                if p.grad is None:
                    p.grad = self.grad_view(p)
                    p.grad.zero_()  # the slot may hold last step's values (lazy zero_grad)
                self.reduce_grad(p)

    def finalize_backward(self) -> None:
        for bucket in self.buckets:
            if not bucket.launched:
                continue
            if self._engine_for(bucket) is not None:
                self.bucket_engine.finish(self, bucket)
            else:
                if bucket.work is not None:
                    bucket.work.wait()
                if self.group_size > 1:
                    bucket.buffer.div_(self.group_size)
            bucket.ready_count = 0
            bucket.work = None
            bucket.launched = False
        self.backward_grad_sync = False
        self.ready_for_sync.clear()

    def remove_hooks(self) -> None:
        for h in self.hook_handles:
            h.remove()
        self.hook_handles = []
