"""Per-kernel device-time table of one training step (torch.profiler / CUPTI), for finding the
hot kernels.  Numbers taken under a profiler are for ranking only, never for reporting.

    python benchmarks/profile_step.py [--config dense|moe] [--steps 2] [--top 40]
"""
from __future__ import annotations

import argparse
import collections
import re
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import bench  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="dense")
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--top", type=int, default=40)
    ap.add_argument("--batch", type=int, default=0)
    args = ap.parse_args()

    from nanotitan_b200.config import AppConfig
    from nanotitan_b200.dist_env import init_distributed, local_device
    from nanotitan_b200.parallel_dims import get_parallel_dims
    from nanotitan_b200.train import build_training
    from nanotitan_b200.utils import seed_everything

    batch = args.batch or bench.BATCH[args.config]
    cfg = AppConfig.model_validate(dict(
        run_name="profile", max_steps=10, model=dict(bench.MODELS[args.config], moe_backend="cuda"),
        trainer=dict(device_id=0, eval_every_step=-1, per_device_batch_size=batch, seed=1),
        data=dict(num_workers=1, train_tokens_path="unused", val_tokens_path="unused"),
        optim=dict(type="adam", lr=5e-4),
        runtime=dict(name="profile", dp_size=1, pp_size=1, ep_size=1, num_microbatches=1, bucket_size=25),
    ))
    init_distributed()
    device = local_device()
    seed_everything(1)
    dims = get_parallel_dims(cfg.runtime)
    model, _, step, opt = build_training(cfg, dims)
    ids = torch.randint(0, cfg.model.vocab_size, (batch, cfg.model.max_seq_len + 1), device=device)
    data = (ids[:, :-1].contiguous(), ids[:, 1:].contiguous())
    for _ in range(3):
        step.train_step(model, data, opt, collect_metrics=False)
    torch.cuda.synchronize()
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA, torch.profiler.ProfilerActivity.CPU]) as prof:
        for _ in range(args.steps):
            step.train_step(model, data, opt, collect_metrics=False)
        torch.cuda.synchronize()
    agg = collections.defaultdict(lambda: [0, 0.0])
    for ev in prof.events():
        if ev.device_type == torch.autograd.DeviceType.CUDA:
            name = ev.name.replace("(anonymous namespace)::", "")
            name = re.sub(r"\(.*", "", name)
            name = re.sub(r"^void ", "", name)
            dur = getattr(ev, "device_time_total", None) or getattr(ev, "cuda_time_total", 0.0)
            agg[name[:90]][0] += 1
            agg[name[:90]][1] += dur
    total = sum(v[1] for v in agg.values())
    print(f"device time per step: {total / args.steps / 1e3:.2f} ms over {sum(v[0] for v in agg.values()) / args.steps:.0f} kernels")
    for name, (n, us) in sorted(agg.items(), key=lambda kv: -kv[1][1])[: args.top]:
        print(f"{us / args.steps:10.1f} us/step {n / args.steps:7.1f} launches  avg {us / n:8.1f} us  {name}")


if __name__ == "__main__":
    main()
