"""Expert-parallel dispatch / return with kernels that write straight into peer memory.

`FusedExchange` holds, for one expert-parallel group, symmetric buffers (mapped into every peer),
the count matrix and a flag pad.  One layer's forward is

    x, routing --ep_dispatch--> expert ranks' staging X_in     (count exchange + pack + push, one kernel)
    ... grouped expert GEMMs read X_in in place ...
    expert outputs --ep_push_rows(1)--> home ranks' staging Y  (already in packed order there)
    ... combine gathers from Y in place ...

and backward runs two pushes the other way round (combine-backward rows to the expert ranks,
dispatch-backward rows home).  Compared with the NCCL path (`parallel/ep.py::_nccl_exchange`) there
is no count collective, no split-size read-back, no packed copy on the home rank, no send / receive
buffers and no regrouping gather / scatter; the host never waits inside a step.  The reference's
expert-parallel path is its torch backend: a count all-to-all with a `.tolist()` read-back, two
`all_to_all_single` per direction and a per-row Python loop that regroups the received rows
(src/model/torch_backend.py:72-147, src/model/moe_ops.py:128-160).

Memory.  X_in and Y of a layer stay alive until that layer's backward (they are what the weight
gradient and the combine backward read), so they come from a pool of symmetric buffers: `acquire`
hands out a free buffer (allocating - a collective over the group - when none fits), `release`
returns it when the layer's backward has used it, `reset` returns everything at the start of a
step.  Every rank runs the same layers in the same order, so the pools evolve identically and a
buffer is the same symmetric allocation on every rank.

Capacity.  Nothing on the host knows how many rows a rank will receive (the counts stay on the
device), so expert-side buffers are sized for the worst case, ep x this rank's own assignment
count, and no row is ever dropped - the reference's semantics.  That is not a formality: with
random-initialised weights the deeper layers of the 16-layer benchmark model route 60-70 % of all
tokens to two experts, so one rank of an ep = 4 group receives 2.7 x its fair share.
`NT_EP_CAPACITY_FACTOR=f` bounds the buffers at f x the fair share for runs whose routing is
known to be balanced (a trained router with the load-balancing loss); rows beyond the bound are
then dropped by the kernel, which records it in the device status word, and the step fails with
a message naming the variable.

Ordering.  Only the dispatch kernel opens with a cross-rank barrier (it carries the counts).  The
other three transfers start without one: each writes a buffer whose last readers on the peers were
enqueued before a kernel that ended with a cross-rank barrier this rank has already passed (the
dispatch of the same layer, or the previous transfer of the same backward), so those reads are over.
All transfers end with a barrier: every rank's rows have landed when the kernel completes.

Symmetric memory comes from a provider in `parallel/symm_memory.py` (torch's, or this library's own heap).
"""
from __future__ import annotations

import math
import os

import torch
import torch.distributed as dist

from nanotitan_b200.ops.ext import get_ext

FLAG_WORDS = 64


class _SymmBuffer:
    """One symmetric allocation viewed as [rows, d], with every rank's address of it."""

    __slots__ = ("flat", "peers", "numel", "dtype")

    def __init__(self, flat, peers):
        self.flat, self.peers, self.numel, self.dtype = flat, peers, flat.numel(), flat.dtype

    def view(self, rows: int, d: int) -> torch.Tensor:
        return self.flat[: rows * d].view(rows, d)


class FusedExchange:
    def __init__(self, group, num_experts: int, device: torch.device):
        from nanotitan_b200.parallel.symm_memory import make_provider

        self.symm, self.group, self.device = make_provider(group, device), group, device
        self.ep = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.E = num_experts
        self.E_loc = num_experts // self.ep
        self.wait_ms = float(os.environ.get("NT_COMM_WAIT_MS", "60000"))
        self.blocks = int(os.environ.get("NT_EP_BLOCKS", "128"))
        self.capacity_factor = float(os.environ.get("NT_EP_CAPACITY_FACTOR", "0"))  # 0 = worst case (ep x)
        self.flags = self._alloc(FLAG_WORDS, torch.int32)
        self.flags.zero_()
        self.flag_peers = self._peers(self.flags)
        self.cmat = self._alloc(self.ep * self.E, torch.int32).view(self.ep, self.E)
        self.cmat.zero_()
        self.cmat_peers = self._peers(self.cmat)
        self.block_counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.epoch_counter = torch.zeros(1, dtype=torch.int32, device=device)  # advanced by the kernels themselves
        self._free: list[_SymmBuffer] = []
        self._used: list[_SymmBuffer] = []
        self._fixed: dict[str, _SymmBuffer] = {}
        self.allocated_bytes = 0
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    # ------------------------------------------------------------------ symmetric memory
    def _alloc(self, numel, dtype):
        return self.symm.empty(numel, dtype)

    def _peers(self, t):
        return torch.tensor(self.symm.peer_ptrs(t), dtype=torch.int64)

    def _new_buffer(self, numel: int, dtype) -> _SymmBuffer:
        flat = self._alloc(numel, dtype)
        self.allocated_bytes += numel * flat.element_size()
        return _SymmBuffer(flat, self._peers(flat))

    def acquire(self, rows: int, d: int, dtype) -> _SymmBuffer:
        """A free pooled buffer of at least rows x d elements (first fit in pool order, else a new
        allocation, which every rank makes at the same call)."""
        need = rows * d
        for i, buf in enumerate(self._free):
            if buf.numel >= need and buf.dtype == dtype:
                self._used.append(self._free.pop(i))
                return buf
        buf = self._new_buffer(need, dtype)
        self._used.append(buf)
        return buf

    def release(self, buf: _SymmBuffer) -> None:
        for i, other in enumerate(self._used):
            if other is buf:
                self._free.append(self._used.pop(i))
                return

    def reset(self) -> None:
        """Start of a step: buffers whose layer never ran backward go back to the pool."""
        self._free.extend(self._used)
        self._used = []

    def fixed(self, name: str, rows: int, d: int, dtype) -> _SymmBuffer:
        """A named buffer that is reused by every layer (the two backward transfers)."""
        buf = self._fixed.get(name)
        if buf is None or buf.numel < rows * d or buf.dtype != dtype:
            buf = self._new_buffer(rows * d, dtype)
            self._fixed[name] = buf
        return buf

    def capacity_rows(self, assignments: int) -> int:
        """Rows an expert rank's buffers hold for a layer in which every rank routes `assignments` rows."""
        worst = max(128, self.ep * assignments)
        if self.capacity_factor <= 0:
            return worst
        bounded = int(math.ceil(self.capacity_factor * assignments / 128.0)) * 128
        return max(128, min(worst, bounded))

    # ------------------------------------------------------------------ primitives
    def allgather_counts(self, counts: torch.Tensor) -> torch.Tensor:
        get_ext().ep_allgather_counts(counts.to(torch.int32).contiguous(), self.cmat_peers, self.flags, self.flag_peers,
                                      self.rank, self.ep, self.epoch_counter, 0, self.wait_ms)
        return self.cmat.clone()

    def push(self, rows: torch.Tensor, cmat: torch.Tensor, direction: int, dst: _SymmBuffer, dst_rows: int,
             entry_barrier: bool = False) -> torch.Tensor:
        """Move `rows` into the peers' `dst` buffers (layout change of `direction`); returns this
        rank's view [dst_rows, d] of `dst`, complete when the kernel has finished."""
        get_ext().ep_push_rows(rows.contiguous(), dst.peers, dst_rows, cmat, self.E_loc, direction, entry_barrier,
                               self.block_counter, self.flags, self.flag_peers, self.rank, self.ep, self.epoch_counter, 0,
                               self.wait_ms, self.blocks)
        return dst.view(dst_rows, rows.shape[1])

    # ------------------------------------------------------------------ layer interface (see parallel/ep.py)
    def dispatch(self, x: torch.Tensor, gates: torch.Tensor, idx: torch.Tensor, counts: torch.Tensor):
        """-> (expert_in [capacity, d] view of this rank's staging, local_offsets [E_loc + 1],
        packed_gate [A], packed_token [A], slot_of [T, k], context for `gather_back`)."""
        return _Dispatch.apply(x, gates, self, idx, counts)

    def gather_back(self, expert_out: torch.Tensor, ctx) -> torch.Tensor:
        return _Return.apply(expert_out, self, ctx)


class _LayerContext:
    """What the transfers of one layer share: its count matrix and buffers."""

    __slots__ = ("cmat", "assignments", "capacity", "x_in", "y_home", "d", "dtype")


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gates, exchange, idx, counts):
        ext = get_ext()
        offsets, slot_of = ext.assign_slots(idx, counts)
        tokens, d = x.shape
        layer = _LayerContext()
        layer.assignments = tokens * idx.shape[1]
        layer.capacity = exchange.capacity_rows(layer.assignments)
        layer.d, layer.dtype = d, x.dtype
        # both forward buffers are taken before the dispatch kernel is enqueued: its barriers then
        # order every peer's earlier reads of them before the first store into them
        layer.x_in = exchange.acquire(layer.capacity, d, x.dtype)
        layer.y_home = exchange.acquire(layer.assignments, d, x.dtype)
        cmat, local_offsets, packed_token, packed_gate = ext.ep_dispatch(
            x.contiguous(), gates.contiguous(), idx, slot_of, counts, offsets, exchange.cmat, exchange.cmat_peers,
            layer.x_in.peers, layer.capacity, exchange.E_loc, exchange.block_counter, exchange.flags, exchange.flag_peers,
            exchange.rank, exchange.ep, exchange.epoch_counter, exchange.wait_ms, exchange.blocks)
        layer.cmat = cmat
        ctx.exchange, ctx.layer, ctx.tokens = exchange, layer, tokens
        ctx.save_for_backward(slot_of)
        expert_in = layer.x_in.view(layer.capacity, d)
        ctx.mark_non_differentiable(local_offsets, packed_token, slot_of)
        ctx.set_materialize_grads(False)
        return expert_in, local_offsets, packed_gate, packed_token, slot_of, _Opaque(layer)

    @staticmethod
    def backward(ctx, d_expert_in, _doff, d_packed_gate, _dtok, _dslot, _dctx):
        (slot_of,) = ctx.saved_tensors
        exchange, layer = ctx.exchange, ctx.layer
        dx = None
        if d_expert_in is not None:
            home = exchange.fixed("dx_home", layer.assignments, layer.d, layer.dtype)
            landed = exchange.push(d_expert_in, layer.cmat, 1, home, layer.assignments)
            dx = get_ext().pack_bwd(landed, slot_of.view(-1), None, ctx.tokens)
        dgates = d_packed_gate[slot_of.long()] if d_packed_gate is not None else None
        exchange.release(layer.x_in)  # the weight-gradient GEMMs that read it are already enqueued
        return dx, dgates, None, None, None


class _Opaque:
    """Carries a Python object through an autograd Function's outputs."""

    def __init__(self, value):
        self.value = value


class _Return(torch.autograd.Function):
    @staticmethod
    def forward(ctx, expert_out, exchange, opaque):
        layer = opaque.value
        ctx.exchange, ctx.layer = exchange, layer
        return exchange.push(expert_out, layer.cmat, 1, layer.y_home, layer.assignments)

    @staticmethod
    def backward(ctx, d_returned):
        exchange, layer = ctx.exchange, ctx.layer
        dst = exchange.fixed("dy_expert", layer.capacity, layer.d, layer.dtype)
        d_expert_out = exchange.push(d_returned, layer.cmat, 0, dst, layer.capacity)
        exchange.release(layer.y_home)  # combine-backward, its last reader, ran before this node
        return d_expert_out, None, None


_EXCHANGES: dict = {}


def get_exchange(group, num_experts: int, device: torch.device):
    """One `FusedExchange` per expert-parallel group (shared by all layers).  None only when the
    fused path is switched off (`NT_FUSED_EP=0`); a set-up failure raises instead of silently
    falling back to the NCCL path."""
    if os.environ.get("NT_FUSED_EP", "1") == "0" or group is None:
        return None
    key = id(group)
    if key not in _EXCHANGES:
        try:
            _EXCHANGES[key] = FusedExchange(group, num_experts, device)
        except Exception as exc:
            raise RuntimeError(
                f"the fused expert-parallel exchange could not be set up ({type(exc).__name__}: {exc}); "
                "set NT_FUSED_EP=0 to run the NCCL all-to-all path on purpose") from exc
    return _EXCHANGES[key]


def reset_pools() -> None:
    """Return every pooled buffer (called at the start of a training step)."""
    for exchange in _EXCHANGES.values():
        if exchange is not None:
            exchange.reset()
