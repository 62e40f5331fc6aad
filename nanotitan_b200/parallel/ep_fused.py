"""Expert-parallel dispatch / return with kernels that write straight into peer memory.

`FusedExchange` holds, for one expert-parallel group, symmetric staging buffers (mapped into
every peer), the all-gathered count matrix and a flag pad.  A layer's forward does:

    counts --ep_allgather_counts--> C[src][expert]           (peer stores + flag barrier)
    packed rows --ep_push_rows(0)--> expert ranks' staging    (already expert-major there)
    ... grouped expert GEMMs ...
    expert outputs --ep_push_rows(1)--> home ranks' staging   (already in packed order there)

and backward runs the two pushes the other way round.  Compared with the NCCL path
(`parallel/ep.py::_nccl_exchange`) there is no count collective, no split-size read-back for the
collective, no send/receive buffers and no regrouping gather/scatter.  One 4-byte host read per
layer remains: the number of rows this rank received, needed to size the activation tensors.
Symmetric memory and its rendezvous come from `torch.distributed._symmetric_memory`.
"""
from __future__ import annotations

import logging
import os

import torch
import torch.distributed as dist

from nanotitan_b200.ops.ext import get_ext

logger = logging.getLogger(__name__)

FLAG_WORDS = 64


class FusedExchange:
    def __init__(self, group, num_experts: int, device: torch.device):
        import torch.distributed._symmetric_memory as symm_mem

        self.symm_mem, self.group, self.device = symm_mem, group, device
        self.ep = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.E = num_experts
        self.E_loc = num_experts // self.ep
        self.wait_ms = float(os.environ.get("NT_COMM_WAIT_MS", "60000"))
        self.blocks = int(os.environ.get("NT_EP_BLOCKS", "96"))
        # NT_EP_HOST_COUNTS=1: read the received row count back per layer (exact-size buffers, one
        # host sync per layer).  Default: size the expert-side buffers for the worst case and keep
        # the count on the device, so the host never waits inside a step.
        self.host_counts = os.environ.get("NT_EP_HOST_COUNTS", "0") == "1"
        self._handles = {}
        self.flags = self._alloc(FLAG_WORDS, torch.int32)
        self.flags.zero_()
        self.flag_peers = self._peers(self.flags)
        self.cmat = self._alloc(self.ep * self.E, torch.int32).view(self.ep, self.E)
        self.cmat.zero_()
        self.cmat_peers = self._peers(self.cmat)
        self.block_counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.epoch = 0
        self.staging: dict[int, torch.Tensor] = {}       # direction -> [capacity, d]
        self.staging_peers: dict[int, torch.Tensor] = {}
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def _alloc(self, numel, dtype):
        t = self.symm_mem.empty(numel, dtype=dtype, device=self.device)
        self._handles[t.data_ptr()] = self.symm_mem.rendezvous(t, self.group)
        return t

    def _peers(self, t):
        return torch.tensor(list(self._handles[t.data_ptr()].buffer_ptrs), dtype=torch.int64)

    def _staging_for(self, direction: int, rows: int, d: int, dtype) -> torch.Tensor:
        """Staging buffer rows land in: direction 0 -> expert side (worst case ep * A rows),
        direction 1 -> home side (A rows).  Every rank sees the same shapes, so (re)allocation
        happens on all ranks at the same call."""
        buf = self.staging.get(direction)
        if buf is None or buf.shape[0] < rows or buf.shape[1] != d or buf.dtype != dtype:
            flat = self._alloc(rows * d, dtype)
            buf = flat.view(rows, d)
            self.staging[direction] = buf
            self.staging_peers[direction] = self._peers(flat)
        return buf

    def _next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    # ------------------------------------------------------------------ primitives
    def allgather_counts(self, counts: torch.Tensor) -> torch.Tensor:
        get_ext().ep_allgather_counts(counts.to(torch.int32).contiguous(), self.cmat_peers, self.flags, self.flag_peers,
                                      self.rank, self.ep, self._next_epoch(), 0, self.wait_ms)
        return self.cmat.clone()

    def push(self, rows: torch.Tensor, cmat: torch.Tensor, direction: int, assignments: int, out_rows: int,
             landed: torch.Tensor | None = None) -> torch.Tensor:
        """`landed` (int32 [1] on the device): how many rows arrive here, when `out_rows` is only the
        worst case; the rows past it in the result are uninitialised and nobody reads them."""
        cap = self.ep * assignments if direction == 0 else assignments
        staging = self._staging_for(direction, cap, rows.shape[1], rows.dtype)
        get_ext().ep_push_rows(rows.contiguous(), self.staging_peers[direction], staging.shape[0], cmat, self.E_loc, direction,
                               self.block_counter, self.flags, self.flag_peers, self.rank, self.ep, self._next_epoch(), 0,
                               self.wait_ms, self.blocks)
        if landed is None:
            return staging[:out_rows].clone()
        out = torch.empty(out_rows, rows.shape[1], dtype=rows.dtype, device=rows.device)
        get_ext().copy_rows_prefix(staging, out, landed)
        return out

    # ------------------------------------------------------------------ layer interface (see parallel/ep.py)
    def dispatch(self, packed_x: torch.Tensor, counts: torch.Tensor):
        cmat = self.allgather_counts(counts)
        mine = cmat[:, self.rank * self.E_loc : (self.rank + 1) * self.E_loc]
        per_expert = mine.sum(dim=0)
        local_offsets = torch.zeros(self.E_loc + 1, dtype=torch.int32, device=packed_x.device)
        local_offsets[1:] = torch.cumsum(per_expert, dim=0)
        assignments = packed_x.shape[0]
        if self.host_counts:
            received = int(local_offsets[-1].item())  # the layer's one host read
            if not 0 <= received <= self.ep * assignments:
                raise RuntimeError(
                    f"expert-parallel count exchange returned {received} rows for rank {self.rank}; at most "
                    f"{self.ep * assignments} can arrive (count matrix: {cmat.tolist()})"
                )
            landed = None
        else:
            # Worst case: every rank sends all its assignments here.  The grouped GEMMs walk the
            # tiles that `local_offsets` describes, so the unused tail costs memory, not time.
            received = self.ep * assignments
            landed = local_offsets[-1:]
        expert_in = _Push.apply(packed_x, self, cmat, 0, assignments, received, landed, None)
        return expert_in, local_offsets, (cmat, assignments, landed)

    def gather_back(self, expert_out: torch.Tensor, ctx) -> torch.Tensor:
        cmat, assignments, landed = ctx
        return _Push.apply(expert_out, self, cmat, 1, assignments, assignments, None, landed)


class _Push(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rows, exchange, cmat, direction, assignments, out_rows, landed, landed_back):
        """`landed` / `landed_back`: device-side row counts of the result / of the gradient that
        travels the other way, when their host-side sizes are worst-case bounds (else None)."""
        ctx.exchange, ctx.cmat, ctx.direction, ctx.assignments, ctx.in_rows = exchange, cmat, direction, assignments, rows.shape[0]
        ctx.landed_back = landed_back
        return exchange.push(rows, cmat, direction, assignments, out_rows, landed)

    @staticmethod
    def backward(ctx, grad):
        back = ctx.exchange.push(grad, ctx.cmat, 1 - ctx.direction, ctx.assignments, ctx.in_rows, ctx.landed_back)
        return back, None, None, None, None, None, None, None


_EXCHANGES: dict = {}


def get_exchange(group, num_experts: int, device: torch.device):
    """One `FusedExchange` per expert-parallel group (shared by all layers); None when disabled or
    when symmetric memory cannot be set up (the NCCL path is used then)."""
    if os.environ.get("NT_FUSED_EP", "1") == "0" or group is None:
        return None
    key = id(group)
    if key not in _EXCHANGES:
        try:
            _EXCHANGES[key] = FusedExchange(group, num_experts, device)
        except Exception as exc:  # noqa: BLE001
            logger.warning("fused expert-parallel exchange unavailable (%s: %s); using NCCL", type(exc).__name__, exc)
            _EXCHANGES[key] = None
    return _EXCHANGES[key]
