"""GPipe pipeline step: all microbatch forwards, then all backwards in reverse order.

Contract of the reference's `PipelineParallel` (src/parallel/pp.py:17-210): it wraps
every run (pp_size 1 included) and owns loss computation, `zero_grad`, the reducers'
finalisation, `optimizer.step()` and the step metrics.  Losses are scaled as in the
reference: cross-entropy and the per-stage mean load-balancing loss (divided by
pp_size) are both divided by the number of microbatches; each stage back-propagates
its own auxiliary loss locally; gradient sync fires only on the last backward.

What differs: stage-boundary activations travel with non-blocking NCCL `isend` /
`irecv` whose receives are all posted before the first forward (and before the first
backward), so transfers of microbatch i+1 overlap the compute of microbatch i; the
last stage computes the loss with the fused unembed + cross-entropy op; times are
CUDA-event device times; and there is one device sync per step, at its end.

CUDA graph.  A step launches several thousand kernels, many of them a few microseconds
long, so the host, not the GPU, sets the pace of small models (and with expert parallelism
every cross-rank barrier then waits for the slowest host).  On GPUs with `pp_size == 1`
the step - zero-grad, forward, loss, backward with the bucket kernels on their side
stream, optimizer update - is therefore captured into one CUDA graph after two ordinary
steps and replayed from then on: one launch per step.  Everything that changes from step
to step lives in device memory (token ids in static input buffers, AdamW bias corrections
in a two-float tensor staged before each replay, the epochs of the cross-rank barriers in
counters the kernels advance themselves), so the captured launches never need new
arguments.  `runtime.cuda_graph = false` or `NT_CUDA_GRAPH=0` keeps the step eager.
"""
from __future__ import annotations

import logging
import os
import time

import torch
import torch.distributed as dist

from nanotitan_b200.dist_env import local_device
from nanotitan_b200.metrics import HistogramMetric, ScalarMetric
from nanotitan_b200.profiler import nvtx_range
from nanotitan_b200.utils import resolve_dtype

logger = logging.getLogger(__name__)


class _Clock:
    """Device time (CUDA events) on GPUs, host time on CPU."""

    def __init__(self, device: torch.device):
        self.cuda = device.type == "cuda"
        self.marks: dict[str, object] = {}

    def mark(self, name: str) -> None:
        if self.cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.marks[name] = ev
        else:
            self.marks[name] = time.perf_counter()

    def seconds(self, start: str, end: str) -> float:
        a, b = self.marks[start], self.marks[end]
        if a is None or b is None:
            return 0.0
        if self.cuda:
            return a.elapsed_time(b) / 1e3
        return b - a


class PendingMetrics:
    """Metrics of a step whose device-to-host copies are still in flight (see `train_step`)."""

    def __init__(self, owner, model, host_f, status, done, clock, host_start, n_mb, n_local):
        self.owner, self.model, self.host_f, self.status, self.done = owner, model, host_f, status, done
        self.clock, self.host_start, self.n_mb, self.n_local = clock, host_start, n_mb, n_local
        self.recv_waits = list(owner._recv_waits)
        self.recv_wait_s = 0.0
        self._metrics = None

    def result(self) -> dict:
        if self._metrics is None:
            self._metrics = self.owner._finish_metrics(self)
        return self._metrics


class _StepGraph:
    """A captured step: static inputs, the graph, and its static metric outputs."""

    def __init__(self):
        self.graph = None
        self.x = self.y = None
        self.floats = None      # [ce_sum, aux_sum, routing counts...] written by every replay
        self.n_local = 0
        self.key = None
        self.launches = 0       # kernels of this library recorded in the graph
        self.launches_by_kernel: dict = {}
        self.inner_marks: dict = {}


EAGER_STEPS_BEFORE_CAPTURE = 2


class PipelineParallel:
    def __init__(self, cfg, dim, reducers: dict):
        self.cfg = cfg
        self.dim = dim
        self.device = local_device()
        self.reducers = reducers
        self.stage_inputs: list[torch.Tensor] = []
        self.stage_outputs: list[torch.Tensor] = []
        self._pending: list = []
        self.use_fused_loss = True
        env = os.environ.get("NT_CUDA_GRAPH")
        want = getattr(cfg.runtime, "cuda_graph", True) if env is None else env != "0"
        self.graph_enabled = bool(want) and self.device.type == "cuda" and dim.pp_size == 1
        self._graph: _StepGraph | None = None
        self._eager_steps = 0
        self.graph_replays = 0
        self._recv_waits: list = []

    # ------------------------------------------------------------------ helpers
    def synchronize_device(self) -> None:
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    def _raise_on_device_failure(self) -> None:
        """Bounded device-side waits record a status word instead of hanging; surface it here."""
        if self.device.type != "cuda":
            return
        from nanotitan_b200.ops import ext

        if not ext.have_ext():
            return
        code, kernel, detail, count = ext.get_ext().read_status(True)
        if code == 2 and kernel == 5 and detail >= 100000:
            raise RuntimeError(
                f"expert-parallel dispatch: expert {detail % 100000} received more rows than the staging buffers hold "
                f"({count} rows dropped on this rank); NT_EP_CAPACITY_FACTOR bounds those buffers - unset it (worst-case "
                "buffers, no drops) or raise it")
        if code != 0:
            raise RuntimeError(
                f"a device-side wait or check failed during this step (code={code}, kernel={kernel}, "
                f"detail={detail}, events={count}); a peer rank is probably gone or stalled"
            )

    def prepare_microbatch(self, x, y):
        n = self.cfg.runtime.num_microbatches
        assert x.shape[0] % n == 0
        return x.chunk(chunks=n), y.chunk(chunks=n)

    def _boundary_buffer(self) -> torch.Tensor:
        return torch.empty(
            (self.microbatch_size, self.cfg.model.max_seq_len, self.cfg.model.d_model),
            device=self.device,
            dtype=resolve_dtype(self.cfg.model.dtype),
        )

    def _post_recvs(self, src: int, count: int):
        """Pre-post `count` receives from `src`; returns [(buffer, work)] in arrival order.
        With `NT_PP_PREPOST=0` nothing is posted ahead: `_recv` then posts each receive when its
        microbatch needs it (the reference's blocking order, src/parallel/pp.py:58,183), which is
        what the stage-idle metric `time/pp_recv_wait` is compared against."""
        if os.environ.get("NT_PP_PREPOST", "1") == "0":
            return [None] * count
        posted = []
        for _ in range(count):
            buf = self._boundary_buffer()
            posted.append((buf, dist.irecv(buf, src=src, group=self.dim.pp_group)))
        return posted

    def _recv(self, posted, src: int) -> torch.Tensor:
        """Wait for one boundary tensor.  The compute stream's idle time across the wait is recorded
        between two events (`time/pp_recv_wait` sums them per step)."""
        if posted is None:
            buf = self._boundary_buffer()
            posted = (buf, dist.irecv(buf, src=src, group=self.dim.pp_group))
        buf, work = posted
        timed = self.device.type == "cuda" and not torch.cuda.is_current_stream_capturing()
        if timed:
            before = torch.cuda.Event(enable_timing=True)
            before.record()
        work.wait()
        if timed:
            after = torch.cuda.Event(enable_timing=True)
            after.record()
            self._recv_waits.append((before, after))
        return buf

    def _send(self, tensor: torch.Tensor, dst: int) -> None:
        self._pending.append((tensor, dist.isend(tensor.contiguous(), dst=dst, group=self.dim.pp_group)))

    def _zero_grad(self, optimizer) -> None:
        if self.device.type == "cuda" and self.dim.ep_size > 1:
            from nanotitan_b200.parallel import ep_fused

            ep_fused.reset_pools()  # staging buffers of layers whose backward never ran
        owned = {id(p) for r in self.reducers.values() for p in r.params}
        lazy = self.device.type == "cuda"  # native kernels write first gradients into their bucket slots
        for r in self.reducers.values():
            r.zero_grad(lazy=lazy)
        for group in optimizer.param_groups:
            for p in group["params"]:
                if id(p) not in owned:
                    p.grad = None

    # ------------------------------------------------------------------ step
    def train_step(self, model, batch, optimizer, collect_metrics: bool = True):
        """One optimizer step.  `collect_metrics=True` returns the metrics dict (one device sync).
        `collect_metrics=False` skips the host read and the sync (the step is still complete on the
        stream) and returns None.  `collect_metrics="deferred"` returns a `PendingMetrics` at once:
        the losses, routing counts and kernel status travel to pinned host memory behind the step,
        and `.result()` waits for that step alone - call it after launching the next step and the
        host never stalls the device."""
        if self._graphable(model, batch, optimizer):
            return self._graphed_step(model, batch, optimizer, collect_metrics)
        return self._eager_step(model, batch, optimizer, collect_metrics)

    @torch.no_grad()
    def eval_step(self, model, batch):
        """Forward only, through the same microbatches and stage boundaries as a training step: the mean
        cross-entropy of this rank's batch on the last pipeline stage (a 0-d tensor on the device), None on
        the other stages.  Nothing is kept for a backward pass.  The reference has the hook for this
        (`trainer.eval_every_step`, `DataParallel.prepare_valloader`) but its loop is commented out
        (src/train.py:187-205)."""
        x, y = batch
        n_mb = self.cfg.runtime.num_microbatches
        microbatch_x, microbatch_y = self.prepare_microbatch(x, y)
        self.microbatch_size = x.shape[0] // n_mb
        first, last = self.dim.is_pp_first_stage, self.dim.is_pp_last_stage
        if self.device.type == "cuda" and self.dim.ep_size > 1:
            from nanotitan_b200.parallel import ep_fused

            ep_fused.reset_pools()  # no backward runs here to hand the staging buffers back
        self._recv_waits = []
        losses = []
        recvs = [] if first else self._post_recvs(self.dim.prev_pp_rank, n_mb)
        for i, (mb_x, mb_y) in enumerate(zip(microbatch_x, microbatch_y, strict=False)):
            mb_x = mb_x.to(self.device, non_blocking=True) if first else self._recv(recvs[i], self.dim.prev_pp_rank)
            out, _ = model(mb_x)
            if last:
                mb_y = mb_y.to(self.device, non_blocking=True)
                losses.append(torch.nn.functional.cross_entropy(out.reshape(-1, out.size(-1)).float(), mb_y.reshape(-1)))
            else:
                self._send(out, self.dim.next_pp_rank)
        for _, work in self._pending:
            work.wait()
        self._pending = []
        return torch.stack(losses).mean() if last else None

    def _eager_step(self, model, batch, optimizer, collect_metrics):
        x, y = batch
        n_mb = self.cfg.runtime.num_microbatches
        clock = _Clock(self.device)
        host_start = time.perf_counter()
        clock.mark("start")
        if getattr(optimizer, "_bc_dev", None) is not None:
            optimizer.stage_step_constants()
        ce_losses, aux_losses, stats_list = self._run(model, x, y, optimizer, clock)
        clock.mark("end")
        for _, work in self._pending:
            work.wait()
        self._pending = []
        self._eager_steps += 1
        if not collect_metrics:
            return None
        floats, n_local = self._metric_floats(ce_losses, aux_losses, stats_list)
        pending = self._start_metrics(model, floats, n_local, clock, host_start, n_mb)
        return pending if collect_metrics == "deferred" else pending.result()

    def _run(self, model, x, y, optimizer, clock):
        """zero-grad, all forwards, all backwards, gradient sync, optimizer update.  `clock` may be
        None (inside a graph capture, where ordinary timing events cannot be recorded)."""
        n_mb = self.cfg.runtime.num_microbatches
        microbatch_x, microbatch_y = self.prepare_microbatch(x, y)
        self.microbatch_size = x.shape[0] // n_mb
        first, last = self.dim.is_pp_first_stage, self.dim.is_pp_last_stage

        def mark(name):
            if clock is not None:
                clock.mark(name)

        self._zero_grad(optimizer)
        self._recv_waits = []
        ce_losses, aux_losses, stats_list = [], [], []
        with nvtx_range("forward_pass"):
            recvs = [] if first else self._post_recvs(self.dim.prev_pp_rank, n_mb)
            for i, (mb_x, mb_y) in enumerate(zip(microbatch_x, microbatch_y, strict=False)):
                if first:
                    mb_x = mb_x.to(self.device, non_blocking=True)
                else:
                    mb_x = self._recv(recvs[i], self.dim.prev_pp_rank)
                    mb_x.requires_grad_()
                    self.stage_inputs.append(mb_x)
                if last:
                    mb_y = mb_y.to(self.device, non_blocking=True)
                    if self.use_fused_loss and hasattr(model, "forward_loss"):
                        loss, stats = model.forward_loss(mb_x, mb_y)
                    else:
                        logits, stats = model(mb_x)
                        loss = torch.nn.functional.cross_entropy(
                            logits.reshape(-1, logits.size(-1)).float(), mb_y.reshape(-1)
                        )
                    ce_losses.append(loss)
                else:
                    out, stats = model(mb_x)
                    self.stage_outputs.append(out)
                    self._send(out.detach(), self.dim.next_pp_rank)
                    ce_losses.append(None)
                aux = torch.stack([s.aux_loss for s in stats]).mean() / self.dim.pp_size
                aux_losses.append(aux)
                stats_list.append(stats)
        mark("forward_end")

        with nvtx_range("backward_pass"):
            grads_in = [] if last else self._post_recvs(self.dim.next_pp_rank, n_mb)
            for step_idx, mb in enumerate(reversed(range(n_mb))):
                for reducer in self.reducers.values():
                    reducer.backward_grad_sync = mb == 0
                ce = ce_losses[mb] / n_mb if last else None
                aux = aux_losses[mb] / n_mb
                incoming = None if last else grads_in[step_idx]
                self.backward(ce, aux, model, mb, incoming)
            for reducer in self.reducers.values():
                reducer.prepare_missing_grad()
            self.finalize_backward()
        mark("backward_end")

        with nvtx_range("optimizer_step"):
            optimizer.step()
        return ce_losses, aux_losses, stats_list

    # ------------------------------------------------------------------ CUDA graph
    def _graphable(self, model, batch, optimizer) -> bool:
        if not self.graph_enabled or not hasattr(optimizer, "enable_device_constants"):
            return False
        if not (self.use_fused_loss and hasattr(model, "forward_loss")):
            return False
        if self._graph is not None:
            return self._graph.key == self._graph_key(model, batch, optimizer)
        return self._eager_steps >= EAGER_STEPS_BEFORE_CAPTURE

    @staticmethod
    def _graph_key(model, batch, optimizer):
        x, y = batch
        return (id(model), id(optimizer), tuple(x.shape), tuple(y.shape), x.dtype, y.dtype)

    def _capture(self, model, batch, optimizer) -> _StepGraph:
        """Record one whole step into a CUDA graph.  Nothing executes during the capture; the caller
        replays the graph to actually take the step."""
        from nanotitan_b200.ops import ext

        x, y = batch
        g = _StepGraph()
        g.key = self._graph_key(model, batch, optimizer)
        g.x = torch.empty(x.shape, dtype=x.dtype, device=self.device)
        g.y = torch.empty(y.shape, dtype=y.dtype, device=self.device)
        g.x.copy_(x)
        g.y.copy_(y)
        optimizer.enable_device_constants(self.device)
        optimizer.stage_step_constants()
        native = ext.get_ext() if ext.have_ext() else None
        torch.cuda.synchronize(self.device)
        before, before_by = (native.launch_count(), native.launch_counts()) if native else (0, {})
        step_before = optimizer._step
        g.graph = torch.cuda.CUDAGraph()
        try:
            with torch.cuda.graph(g.graph):
                ce_losses, aux_losses, stats_list = self._run(model, g.x, g.y, optimizer, None)
                g.floats, g.n_local = self._metric_floats(ce_losses, aux_losses, stats_list)
        except Exception as exc:
            raise RuntimeError(
                f"capturing the training step in a CUDA graph failed ({type(exc).__name__}: {exc}); "
                "set NT_CUDA_GRAPH=0 (or runtime.cuda_graph = false) to run the step eagerly") from exc
        optimizer._step = step_before  # the capture ran optimizer.step()'s bookkeeping, not the update
        if native:
            g.launches = native.launch_count() - before
            g.launches_by_kernel = {k: v - before_by.get(k, 0) for k, v in native.launch_counts().items()
                                    if v - before_by.get(k, 0)}
        logger.info("training step captured in a CUDA graph (%d kernels of this library per replay)", g.launches)
        return g

    def _graphed_step(self, model, batch, optimizer, collect_metrics):
        if self._graph is None:
            self._graph = self._capture(model, batch, optimizer)
        g = self._graph
        x, y = batch
        n_mb = self.cfg.runtime.num_microbatches
        clock = _Clock(self.device)
        host_start = time.perf_counter()
        clock.mark("start")
        g.x.copy_(x, non_blocking=True)  # from pinned host memory: the step's host-to-device copy
        g.y.copy_(y, non_blocking=True)
        optimizer.stage_step_constants()
        g.graph.replay()
        optimizer._step += 1
        self.graph_replays += 1
        clock.mark("end")
        clock.marks["forward_end"] = clock.marks["backward_end"] = None  # not separable inside a graph
        if not collect_metrics:
            return None
        pending = self._start_metrics(model, g.floats, g.n_local, clock, host_start, n_mb)
        return pending if collect_metrics == "deferred" else pending.result()

    def launches_last_step(self) -> tuple[int, dict]:
        """(kernels of this library, by entry point) a replayed step runs; (0, {}) while eager."""
        if self._graph is None:
            return 0, {}
        return self._graph.launches, dict(self._graph.launches_by_kernel)

    def _metric_floats(self, ce_losses, aux_losses, stats_list):
        """One fp32 device tensor [ce_sum, aux_sum, routing counts of the local layers...]."""
        last = self.dim.is_pp_last_stage
        zero = torch.zeros((), dtype=torch.float32, device=self.device)
        ce_sum = torch.stack([c.detach().float() for c in ce_losses]).sum() if last else zero
        aux_sum = torch.stack([a.detach().float() for a in aux_losses]).sum() if last else zero
        n_local = len(stats_list[0]) if stats_list and stats_list[0] else 0
        parts = [ce_sum.reshape(1), aux_sum.reshape(1)]
        if n_local:
            counts = torch.stack(
                [torch.stack([mb[i].tokens_per_expert.detach().float() for i in range(n_local)]) for mb in stats_list]
            ).sum(dim=0)  # [local layers, E]
            parts.append(counts.reshape(-1))
        return torch.cat(parts), n_local

    def _start_metrics(self, model, floats, n_local, clock, host_start, n_mb) -> "PendingMetrics":
        """Send everything the step's metrics need from the device (losses and routing counts in
        `floats`, the kernels' status word) to pinned host memory with two stream-ordered copies."""
        status = None
        if self.device.type == "cuda":
            from nanotitan_b200.ops import ext

            host_f = torch.empty(floats.shape, dtype=torch.float32, pin_memory=True)
            host_f.copy_(floats, non_blocking=True)
            if ext.have_ext():
                status = torch.empty(4, dtype=torch.int32, pin_memory=True)
                status.copy_(ext.get_ext().status_word_tensor(), non_blocking=True)
            done = torch.cuda.Event()
            done.record()
        else:
            host_f, done = floats, None
        return PendingMetrics(self, model, host_f, status, done, clock, host_start, n_mb, n_local)

    def _finish_metrics(self, pending: "PendingMetrics") -> dict:
        if pending.done is not None:
            pending.done.synchronize()  # this step only: later steps may already be running
        pending.recv_wait_s = sum(a.elapsed_time(b) for a, b in pending.recv_waits) / 1e3
        if pending.status is not None and int(pending.status[0]) != 0:
            self._raise_on_device_failure()
        values = pending.host_f.tolist()
        ce_sum, aux_sum = values[0], values[1]
        last, n_mb, clock = self.dim.is_pp_last_stage, pending.n_mb, pending.clock
        metrics = {
            "train/ce_loss": ScalarMetric(ce_sum / n_mb, reduce="sum"),
            "train/lb_loss": ScalarMetric(aux_sum / n_mb, reduce="sum"),
            # same precedence as the reference: sum(ce) + sum(aux)/n (src/parallel/pp.py:124)
            "train/total_loss": ScalarMetric(ce_sum + aux_sum / n_mb if last else 0.0, reduce="sum"),
            "time/step_time": ScalarMetric(clock.seconds("start", "end"), reduce="max"),
            # a replayed graph has no host-visible boundary between forward and backward: 0.0 there
            "time/forward_time": ScalarMetric(clock.seconds("start", "forward_end"), reduce="max"),
            "time/backward_time": ScalarMetric(clock.seconds("forward_end", "backward_end"), reduce="max"),
            "time/host_step_time": ScalarMetric(time.perf_counter() - pending.host_start, reduce="max"),
            # compute-stream idle time across the waits for stage-boundary tensors (0 without pipeline stages)
            "time/pp_recv_wait": ScalarMetric(pending.recv_wait_s, reduce="max"),
        }
        counts = None
        if pending.n_local:
            counts = pending.host_f[2:].reshape(pending.n_local, -1).clone()
        metrics.update(self._moe_route_fraction_metrics(pending.model, counts))
        return metrics

    def backward(self, ce_loss, moe_aux_loss, model, microbatch_idx, incoming=None) -> None:
        if self.dim.is_pp_last_stage:
            torch.autograd.backward([ce_loss, moe_aux_loss])
        else:
            out = self.stage_outputs[microbatch_idx]
            grad_buf = self._recv(incoming, self.dim.next_pp_rank)
            torch.autograd.backward([out, moe_aux_loss], [grad_buf, torch.ones_like(moe_aux_loss)])
        if not self.dim.is_pp_first_stage:
            self._send(self.stage_inputs[microbatch_idx].grad, self.dim.prev_pp_rank)

    def finalize_backward(self) -> None:
        self.stage_inputs = []
        self.stage_outputs = []
        for reducer in self.reducers.values():
            reducer.finalize_backward()

    # ------------------------------------------------------------------ metrics
    def _moe_route_fraction_metrics(self, model, counts) -> dict:
        """Per global layer, the fraction of assignments each expert received (`counts`: host tensor
        [local layers, E] or None); stages that do not own a layer contribute zeros so a SUM over
        ranks gives the DP mean."""
        metrics = {}
        local = {}
        if counts is not None:
            fracs = counts / counts.sum(dim=1, keepdim=True).clamp_min(1.0)
            for i in range(fracs.shape[0]):
                local[model.spec.layer_start + i] = fracs[i]
        # DP is folded over EP: dp*ep ranks per stage see different data.
        replicas = self.dim.dp_size * self.dim.ep_size
        for layer in range(self.cfg.model.n_layers):
            frac = local.get(layer)
            value = torch.zeros(self.cfg.model.num_experts, dtype=torch.float32)
            if frac is not None:
                value = frac / replicas
            metrics[f"moe/layer_{layer:02d}/route_frac_dist"] = HistogramMetric(value, reduce="sum")
        return metrics
