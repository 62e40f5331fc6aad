"""What a configuration puts on each GPU, before any GPU is involved.

    python -m nanotitan_b200.plan configs/moe_3d.toml [--hbm-gb 180] [--capacity-factor f] [--sustained-tflops t] [--json]

For every distinct (pipeline stage, expert rank) of the layout the model shard is built on the meta device
(no memory) and the planner reports, per GPU:

  exact    parameters by synchronisation group, the gradient buckets the reducer will lay out, the optimizer
           state as `FusedAdamW` shards it (12 bytes per parameter of a 16-bit bucket divided over the bucket's
           data-parallel group, whole for fp32 buckets), the staging buffers of the fused expert exchange at
           their worst-case capacity, the padded logits buffer of the fused unembed + loss;
  estimate the activations autograd keeps for the backward pass, from the list of tensors the kernels' autograd
           nodes save per layer, times the micro-batches a GPipe stage holds in flight.

and compares the sum with the HBM size (180 GB on a B200).  The estimate is labelled as such in the output: it
counts the saved tensors, not allocator slack or temporaries.  The last line is the step-time floor: the model
FLOPs of a step at the sustained GEMM rate of MEASURED_PEAKS.json.  The reference has no counterpart.
"""
from __future__ import annotations

import argparse
import json
import math
import sys
from dataclasses import asdict, dataclass, field

import torch

from nanotitan_b200.config import AppConfig, load_config
from nanotitan_b200.models.model import NanoTitanModel
from nanotitan_b200.models.utils import get_model_shard_specs
from nanotitan_b200.parallel.fused_allreduce import owned_slice
from nanotitan_b200.parallel.reducer import plan_buckets
from nanotitan_b200.parallel_dims import RankLayout
from nanotitan_b200.utils import resolve_dtype

GB = 1e9


@dataclass
class ShardPlan:
    pp_rank: int
    ep_rank: int
    ranks: list[int]
    layers: tuple[int, int]
    experts: tuple[int, int]
    parameters: dict[str, int] = field(default_factory=dict)           # group -> count
    buckets: dict[str, int] = field(default_factory=dict)              # group -> number of gradient buckets
    bytes: dict[str, int] = field(default_factory=dict)                # item -> bytes on one GPU
    estimated: list[str] = field(default_factory=list)                 # which items of `bytes` are estimates

    @property
    def total(self) -> int:
        return sum(self.bytes.values())


def _layout(cfg: AppConfig, rank: int) -> RankLayout:
    rt = cfg.runtime
    world = rt.dp_size * rt.pp_size * rt.ep_size
    layout = RankLayout(world, rank, rt.dp_size, rt.pp_size, rt.ep_size, num_experts=cfg.model.num_experts)
    layout.ep_group = None  # `get_model_shard_specs` passes it on; nothing here communicates
    return layout


def _optimizer_bytes(buckets, group_size: int) -> int:
    total = 0
    for b in buckets:
        padded = (b.numel + 127) // 128 * 128
        sharded = group_size > 1 and b.dtype in (torch.bfloat16, torch.float16)
        lo, hi = owned_slice(padded, group_size, 0) if sharded else (0, padded)
        total += 12 * (hi - lo)  # fp32 master weight and two moments
    return total


def expert_capacity_rows(ep: int, assignments: int, factor: float = 0.0) -> int:
    """The rule of `FusedExchange.capacity_rows`: worst case unless a capacity factor bounds it."""
    worst = max(128, ep * assignments)
    if factor <= 0:
        return worst
    return max(128, min(worst, int(math.ceil(factor * assignments / 128.0)) * 128))


def saved_activation_bytes_per_layer(cfg: AppConfig, micro_tokens: int, expert_rows: int) -> int:
    """Bytes the autograd nodes of one transformer layer keep for backward, for `micro_tokens` tokens on this GPU
    and `expert_rows` rows in this GPU's experts: the layer input (residual stream), LayerNorm statistics, the
    normalised input of the QKV projection, Q / K / V, the attention output and its log-sum-exp, the input of the
    output projection, the second LayerNorm's input and output, and per expert row the packed input, the
    gate | value pre-activations and the SwiGLU output; plus routing (gates, ids, probabilities, slots)."""
    m = cfg.model
    e = resolve_dtype(m.dtype).itemsize
    width = m.n_heads * m.d_head
    t, d, f = micro_tokens, m.d_model, m.ffn_in
    attention = t * d * e * 3 + t * 8 * 2 + t * width * e * 4 + t * m.n_heads * 4 + t * width * e
    routing = t * (m.top_k * 12 + m.num_experts * 4)
    experts = expert_rows * (d * e + 2 * f * e + f * e) + t * m.top_k * d * e  # + returned rows kept for the combine
    return attention + routing + experts


def plan(cfg: AppConfig, capacity_factor: float = 0.0) -> list[ShardPlan]:
    rt, m = cfg.runtime, cfg.model
    elem = resolve_dtype(m.dtype).itemsize
    seen: dict[tuple[int, int], ShardPlan] = {}
    world = rt.dp_size * rt.pp_size * rt.ep_size
    for rank in range(world):
        layout = _layout(cfg, rank)
        key = (layout.pp_rank, layout.ep_rank)
        if key in seen:
            seen[key].ranks.append(rank)
            continue
        spec = get_model_shard_specs(layout, cfg)
        with torch.device("meta"):
            model = NanoTitanModel.from_specs(m, spec)
        shard = ShardPlan(layout.pp_rank, layout.ep_rank, [rank], (spec.layer_start, spec.layer_end),
                          (spec.start_expert_id, spec.end_expert_id))
        groups = model.parameter_sync_groups()
        sizes = {"shared": len(layout.shared_dp_group_ranks), "expert": len(layout.expert_dp_group_ranks)}
        param_bytes = grad_bytes = optim_bytes = 0
        for name, params in groups.items():
            params = [p for p in params if p.requires_grad]
            buckets = plan_buckets(params, rt.bucket_size * 1024 * 1024)
            shard.parameters[name] = sum(p.numel() for p in params)
            shard.buckets[name] = len(buckets)
            param_bytes += sum(p.numel() * p.element_size() for p in params)
            grad_bytes += sum((b.numel + 127) // 128 * 128 * torch.empty((), dtype=b.dtype).element_size() for b in buckets)
            optim_bytes += _optimizer_bytes(buckets, sizes[name])
        shard.bytes["parameters"] = param_bytes
        shard.bytes["gradient buckets"] = grad_bytes
        shard.bytes["optimizer state (fp32 master + 2 moments, sharded over the data-parallel group)"] = optim_bytes
        n_layers = spec.layer_end - spec.layer_start
        micro = cfg.trainer.per_device_batch_size // rt.num_microbatches
        micro_tokens = micro * m.max_seq_len
        assignments = micro_tokens * m.top_k
        in_flight = rt.num_microbatches  # GPipe: every micro-batch's forward runs before the first backward
        if rt.ep_size > 1:
            cap = expert_capacity_rows(rt.ep_size, assignments, capacity_factor)
            # per layer and micro-batch in flight: expert inputs and returned outputs; two more buffers serve every backward
            staging = n_layers * in_flight * (cap + assignments) * m.d_model * elem + (cap + assignments) * m.d_model * elem
            shard.bytes["expert exchange staging (symmetric memory)"] = staging
            expert_rows = cap
        else:
            expert_rows = assignments
        if spec.has_unembed_head:
            shard.bytes["logits buffer of the fused unembed + loss"] = micro_tokens * ((m.vocab_size + 63) // 64 * 64) * elem
        label = f"saved activations, {n_layers} layers x {in_flight} micro-batch(es) in flight (estimate)"
        shard.bytes[label] = n_layers * in_flight * saved_activation_bytes_per_layer(cfg, micro_tokens, expert_rows)
        shard.estimated.append(label)
        seen[key] = shard
    return list(seen.values())


def step_floor(cfg: AppConfig, sustained_tflops: float) -> dict:
    """Model FLOPs of one optimizer step over the whole job (the trainer's MFU numerator: 6 x active matmul
    parameters + causal attention, per token) and the time they take at `sustained_tflops` per GPU: the floor any
    measured step time is compared with."""
    from nanotitan_b200.train import model_flops_per_token

    rt, m = cfg.runtime, cfg.model
    with torch.device("meta"):
        layout = _layout(cfg, 0)
        layout_full = RankLayout(1, 0, 1, 1, 1, num_experts=m.num_experts)
        layout_full.ep_group = None
        whole = NanoTitanModel.from_specs(m, get_model_shard_specs(layout_full, cfg))
    active = float(whole.active_parameter_count())
    tokens = cfg.trainer.per_device_batch_size * layout.data_world_size * m.max_seq_len
    flops = model_flops_per_token(cfg, active) * tokens
    gpus = rt.dp_size * rt.pp_size * rt.ep_size
    return {"tokens_per_step": tokens, "tflop_per_step": flops / 1e12, "gpus": gpus,
            "floor_ms": flops / (sustained_tflops * 1e12 * gpus) * 1e3 if sustained_tflops > 0 else None}


def nvlink_bytes_per_step(cfg: AppConfig, shard: ShardPlan) -> dict[str, int]:
    """Bytes one GPU of `shard` sends (and, symmetrically, receives) over NVLink in one step, by cause:
    gradient buckets (the fused all-reduce moves one bucket out and one in per replica group larger than one),
    expert exchange (four transfers per MoE layer and micro-batch, the share of rows that leaves the GPU),
    pipeline boundaries (activations forward, their gradients backward)."""
    rt, m = cfg.runtime, cfg.model
    elem = resolve_dtype(m.dtype).itemsize
    layout = _layout(cfg, shard.ranks[0])
    out: dict[str, int] = {}
    replicas = {"shared": len(layout.shared_dp_group_ranks), "expert": len(layout.expert_dp_group_ranks)}
    out["gradient all-reduce"] = sum(shard.parameters[g] * elem for g in shard.parameters if replicas[g] > 1)
    micro_tokens = cfg.trainer.per_device_batch_size // rt.num_microbatches * m.max_seq_len
    n_layers = shard.layers[1] - shard.layers[0]
    if rt.ep_size > 1:
        rows = micro_tokens * m.top_k
        out["expert exchange"] = 4 * n_layers * rt.num_microbatches * rows * m.d_model * elem * (rt.ep_size - 1) // rt.ep_size
    if rt.pp_size > 1:
        sides = (0 if layout.is_pp_first_stage else 1) + (0 if layout.is_pp_last_stage else 1)
        out["pipeline boundaries"] = sides * rt.num_microbatches * micro_tokens * m.d_model * elem
    return out


def measured_sustained_tflops(default: float = 1400.0) -> float:
    """`bf16_tflops_sustained` of MEASURED_PEAKS.json next to the package's parent folder, else `default`."""
    from pathlib import Path

    path = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["bf16_tflops_sustained"])
    except (OSError, KeyError, ValueError):
        return default


LINK_GBS = 770.0  # measured peer-copy bandwidth per direction; 900 is the nominal figure


def render(shards: list[ShardPlan], hbm_gb: float, cfg: AppConfig | None = None) -> str:
    lines = []
    for s in shards:
        lines.append(f"pipeline stage {s.pp_rank}, expert rank {s.ep_rank} (ranks {s.ranks}): layers {s.layers[0]}..{s.layers[1] - 1}, "
                     f"experts {s.experts[0]}..{s.experts[1] - 1}")
        for group, count in s.parameters.items():
            lines.append(f"    {group:>7} parameters {count / 1e6:10.2f} M in {s.buckets[group]} gradient bucket(s)")
        for item, nbytes in s.bytes.items():
            lines.append(f"    {nbytes / GB:10.2f} GB  {item}")
        share = s.total / (hbm_gb * GB)
        verdict = "fits" if share < 0.9 else ("tight" if share < 1.0 else "DOES NOT FIT")
        lines.append(f"    {s.total / GB:10.2f} GB  total = {100 * share:.0f} % of {hbm_gb:.0f} GB: {verdict}")
        if cfg is not None:
            traffic = nvlink_bytes_per_step(cfg, s)
            total = sum(traffic.values())
            if total:
                parts = ", ".join(f"{k} {v / GB:.3f} GB" for k, v in traffic.items() if v)
                lines.append(f"    NVLink per step and direction: {parts}: >= {total / (LINK_GBS * 1e9) * 1e3:.2f} ms at "
                             f"{LINK_GBS:.0f} GB/s if nothing overlapped")
    return "\n".join(lines)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("config", help="TOML config path (as for the trainer)")
    ap.add_argument("--hbm-gb", type=float, default=180.0)
    ap.add_argument("--capacity-factor", type=float, default=0.0, help="NT_EP_CAPACITY_FACTOR the run will use (0: worst case)")
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--sustained-tflops", type=float, default=0.0,
                    help="dense bf16 GEMM rate per GPU for the step-time floor (default: MEASURED_PEAKS.json, else 1400)")
    args = ap.parse_args(argv)
    cfg = load_config(args.config.removeprefix("@"))
    shards = plan(cfg, args.capacity_factor)
    floor = step_floor(cfg, args.sustained_tflops or measured_sustained_tflops())
    if args.json:
        print(json.dumps({"shards": [dict(asdict(s), total=s.total, nvlink_bytes_per_step=nvlink_bytes_per_step(cfg, s)) for s in shards],
                          "step": floor}, indent=1))
    else:
        print(render(shards, args.hbm_gb, cfg))
        print(f"one step: {floor['tokens_per_step']} tokens, {floor['tflop_per_step']:.2f} TFLOP of model math over {floor['gpus']} GPU(s): "
              f">= {floor['floor_ms']:.2f} ms at {args.sustained_tflops or measured_sustained_tflops():.0f} TFLOP/s per GPU")
    return 0 if all(s.total < args.hbm_gb * GB for s in shards) else 1


if __name__ == "__main__":
    sys.exit(main())
