"""AdamW on flat buckets with fp32 master weights, one fused kernel per bucket.

Update rule of `torch.optim.AdamW` (the reference's optimizer, src/optim.py:6-10: weight
decay 0.1 on every parameter, betas (0.9, 0.999), eps 1e-8).  Parameters keep their storage
dtype (bf16 for the benchmark configs); the optimizer holds fp32 master copies and moments
and rewrites the bf16 values after each step.  When bound to the data-parallel reducers it
reuses their flat gradient buckets (gradients are views into them), so a step is one kernel
per bucket with no gather or scatter of tensors.

Buckets that the fused all-reduce engine updates (data-parallel groups of two or more GPUs) keep
optimizer state for this rank's 1/N slice of the bucket only (ZeRO-1): the engine's kernel
reduces that slice, applies AdamW to it and broadcasts the new bf16 values, so fp32 master
weights and moments of the other slices never exist on this rank.  `state_dict()` stores exactly
those slices; a checkpoint therefore resumes on the same data-parallel size and bucket plan.
"""
from __future__ import annotations

import torch

from nanotitan_b200.ops import reference as ref
from nanotitan_b200.ops.ext import get_ext
from nanotitan_b200.parallel.reducer import ReducerV1


class _Chunk:
    def __init__(self, bucket, params, spans, engine=None):
        self.bucket = bucket
        self.params, self.spans = params, spans
        self.fused_by_engine = False
        self.group, self.group_size = None, 1  # the data-parallel group the bucket is reduced over
        n = bucket.buffer.numel()
        self.owned = (0, n)  # the part of the bucket whose optimizer state lives here
        if engine is not None:
            flat = engine.alloc(n, bucket.dtype, bucket.device)  # symmetric: peers write new values into it
            flat.zero_()
            self.owned = engine.owned_slice(n)
        else:
            flat = torch.zeros(n, dtype=bucket.dtype, device=bucket.device)
        for p, (lo, hi) in zip(params, spans):
            flat[lo:hi].copy_(p.data.reshape(-1))
            p.data = flat[lo:hi].view_as(p)
        self.flat_param = flat
        self.master = flat[self.owned[0] : self.owned[1]].float()
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)


class FusedAdamW(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.1, track_grad_norm=False):
        params = [p for p in params if p.requires_grad]
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self._params = params
        self._chunks: list[_Chunk] | None = None
        self._own_reducer: ReducerV1 | None = None
        self._step = 0
        self.track_grad_norm = track_grad_norm
        self._sq_parts: list[torch.Tensor] = []
        # Bias corrections of the step in flight, in device memory, for launches that are captured in a
        # CUDA graph (their arguments cannot change from step to step); None = computed per launch.
        self._bc_dev: torch.Tensor | None = None
        self._bc_host: torch.Tensor | None = None

    # ------------------------------------------------------------------ layout
    def bind_reducers(self, reducers: dict) -> None:
        """Adopt the reducers' buckets as the optimizer's flat layout."""
        assert self._chunks is None, "bind_reducers must precede the first step"
        owned = set()
        self._chunks = []
        for red in reducers.values():
            for b in red.buckets:
                engine = red._engine_for(b) if hasattr(red, "_engine_for") else None
                chunk = _Chunk(b, b.params, b.spans, engine)
                chunk.group, chunk.group_size = red.process_group, red.group_size
                if engine is not None:
                    engine.bind_optimizer(b, chunk.flat_param, chunk.master, chunk.exp_avg, chunk.exp_avg_sq, self)
                    chunk.fused_by_engine = True
                self._chunks.append(chunk)
                owned.update(id(p) for p in b.params)
        rest = [p for p in self._params if id(p) not in owned]
        if rest:
            self._own_reducer = ReducerV1(rest, 1, None, bucket_size=1 << 20)
            for b in self._own_reducer.buckets:
                self._chunks.append(_Chunk(b, b.params, b.spans))

    def enable_device_constants(self, device) -> None:
        """Keep the per-step bias corrections in device memory (see `stage_step_constants`)."""
        if self._bc_dev is None:
            self._bc_dev = torch.zeros(2, dtype=torch.float32, device=device)
            self._bc_host = torch.zeros(2, dtype=torch.float32).pin_memory()

    def stage_step_constants(self) -> None:
        """Copy the bias corrections of the next step to the device (one 8-byte stream-ordered copy);
        call before every step whose kernels were captured with `device_constants()`."""
        beta1, beta2 = self.param_groups[0]["betas"]
        t = self._step + 1
        self._bc_host[0] = 1.0 - beta1 ** t
        self._bc_host[1] = 1.0 / (1.0 - beta2 ** t) ** 0.5
        self._bc_dev.copy_(self._bc_host, non_blocking=True)

    def device_constants(self):
        return self._bc_dev

    def next_step(self) -> int:
        """Step number the update in flight belongs to (bucket kernels run before `step()`)."""
        return self._step + 1

    def _ensure_layout(self) -> None:
        if self._chunks is None:
            self.bind_reducers({})

    def zero_grad(self, set_to_none: bool = True) -> None:
        self._ensure_layout()
        for c in self._chunks:
            c.bucket.buffer.zero_()

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, closure=None):
        self._ensure_layout()
        self._step += 1
        group = self.param_groups[0]
        beta1, beta2 = group["betas"]
        self._sq_parts = []
        for c in self._chunks:
            if c.fused_by_engine:
                if not c.bucket.launched_this_step:
                    raise RuntimeError(
                        "a gradient bucket bound to the fused all-reduce engine was not reduced this step; its optimizer "
                        "state is sharded over the data-parallel ranks, so the update cannot run locally (run backward "
                        "through the reducers with backward_grad_sync set, as PipelineParallel.train_step does)")
                c.bucket.launched_this_step = False  # updated by the all-reduce kernel already
                continue
            grads = c.bucket.buffer
            for p, (lo, hi) in zip(c.params, c.spans):  # a gradient that is not the bucket view
                if p.grad is not None and p.grad.data_ptr() != grads[lo:hi].data_ptr():
                    grads[lo:hi].copy_(p.grad.reshape(-1))
                    p.grad = grads[lo:hi].view_as(p)
            if grads.is_cuda:
                part = get_ext().adamw_step(c.flat_param, grads, c.master, c.exp_avg, c.exp_avg_sq, self._step,
                                            group["lr"], beta1, beta2, group["eps"], group["weight_decay"], 1.0,
                                            self.track_grad_norm, self._bc_dev)
                if self.track_grad_norm:
                    self._sq_parts.append(part.sum())
            else:
                ref.adamw_step(c.master, grads.float(), c.exp_avg, c.exp_avg_sq, self._step, group["lr"], beta1, beta2,
                               group["eps"], group["weight_decay"])
                c.flat_param.copy_(c.master)
        return None

    def last_grad_norm(self) -> float:
        if not self._sq_parts:
            return 0.0
        return float(torch.stack(self._sq_parts).sum().sqrt().item())

    # ------------------------------------------------------------------ checkpoints
    def set_master_weights(self, values: dict) -> None:
        """Overwrite fp32 master weights (and the stored parameters) from `values`: id(param) -> tensor
        shaped like the parameter, e.g. fp32 weights of another run.  Each rank takes what falls into
        the slices it owns."""
        self._ensure_layout()
        with torch.no_grad():
            for c in self._chunks:
                olo, ohi = c.owned
                for p, (lo, hi) in zip(c.params, c.spans):
                    src = values.get(id(p))
                    if src is None:
                        continue
                    flat_src = src.reshape(-1).to(device=c.master.device, dtype=torch.float32)
                    c.flat_param[lo:hi].copy_(flat_src)
                    a, b = max(lo, olo), min(hi, ohi)
                    if a < b:
                        c.master[a - olo : b - olo].copy_(flat_src[a - lo : b - lo])

    def state_bytes(self) -> int:
        """Bytes of fp32 optimizer state (master + two moments) held by this rank."""
        self._ensure_layout()
        return sum(3 * 4 * c.master.numel() for c in self._chunks)

    # ------------------------------------------------------------------ layout-independent state
    def per_parameter_state(self, names: dict[int, str]) -> dict[str, dict[str, torch.Tensor]]:
        """fp32 master weights and both moments of every parameter, whole, on the host, keyed by
        `names[id(parameter)]`: the form that does not depend on buckets or on how the state is sharded.
        Collective over each sharded bucket's data-parallel group (every rank gathers the other ranks' slices)."""
        import torch.distributed as dist

        self._ensure_layout()
        out: dict[str, dict[str, torch.Tensor]] = {}
        for c in self._chunks:
            n = c.flat_param.numel()
            whole = {}
            for key in ("master", "exp_avg", "exp_avg_sq"):
                mine = getattr(c, key)
                if tuple(c.owned) == (0, n):
                    whole[key] = mine.detach().cpu()
                    continue
                width = ((n // 8 + c.group_size - 1) // c.group_size) * 8  # the slice width `owned_slice` hands out
                padded = torch.zeros(width, dtype=torch.float32, device=mine.device)
                padded[: mine.numel()].copy_(mine)
                parts = [torch.empty_like(padded) for _ in range(c.group_size)]
                dist.all_gather(parts, padded, group=c.group)
                whole[key] = torch.cat(parts)[:n].cpu()
            for p, (lo, hi) in zip(c.params, c.spans):
                out[names[id(p)]] = {key: whole[key][lo:hi].view(p.shape).clone() for key in whole}
        return out

    def load_per_parameter_state(self, state: dict[str, dict[str, torch.Tensor]], names: dict[int, str], step: int) -> None:
        """Inverse of `per_parameter_state` for whatever layout this run has: every rank keeps what falls into
        the slices it owns and rewrites the stored parameters there from the master weights."""
        self._ensure_layout()
        self._step = step
        with torch.no_grad():
            for c in self._chunks:
                olo, ohi = c.owned
                for p, (lo, hi) in zip(c.params, c.spans):
                    rec = state[names[id(p)]]
                    a, b = max(lo, olo), min(hi, ohi)
                    if a >= b:
                        continue
                    for key in ("master", "exp_avg", "exp_avg_sq"):
                        src = rec[key].reshape(-1).to(torch.float32)
                        getattr(c, key)[a - olo : b - olo].copy_(src[a - lo : b - lo])
                c.flat_param[olo:ohi].copy_(c.master)

    def state_dict(self):
        self._ensure_layout()
        chunks = []
        for c in self._chunks:
            chunks.append({"numel": c.flat_param.numel(), "owned": tuple(c.owned), "master": c.master.clone().cpu(),
                           "exp_avg": c.exp_avg.clone().cpu(), "exp_avg_sq": c.exp_avg_sq.clone().cpu()})
        return {"step": self._step, "chunks": chunks,
                "hyper": {k: v for k, v in self.param_groups[0].items() if k != "params"}}

    def load_state_dict(self, state):
        self._ensure_layout()
        self._step = state["step"]
        if len(state["chunks"]) != len(self._chunks):
            raise ValueError(f"checkpoint has {len(state['chunks'])} optimizer buckets, this run has {len(self._chunks)} "
                             "(different bucket size or model shard)")
        for c, rec in zip(self._chunks, state["chunks"]):
            if rec["numel"] != c.flat_param.numel() or tuple(rec["owned"]) != tuple(c.owned):
                raise ValueError(f"optimizer state was saved for slice {tuple(rec['owned'])} of a {rec['numel']}-element "
                                 f"bucket; this rank owns {tuple(c.owned)} of {c.flat_param.numel()} (the data-parallel "
                                 "size or the bucket plan changed)")
            c.master.copy_(rec["master"])
            c.exp_avg.copy_(rec["exp_avg"])
            c.exp_avg_sq.copy_(rec["exp_avg_sq"])
            # the stored parameters are the rounding of the master weights where this rank has them;
            # everywhere else they keep the values the model state dict restored
            c.flat_param[c.owned[0] : c.owned[1]].copy_(c.master)
        for k, v in state.get("hyper", {}).items():
            self.param_groups[0][k] = v
