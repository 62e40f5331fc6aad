"""Headline benchmark: training tokens/s of the 16-layer d512 LM, 40 x 768 tokens per GPU, bf16.

    python bench.py --gpus N --steps K --warmup W [--impl ours|reference] [--config dense|moe]

For N > 1 launch with `python -m torch.distributed.run --nnodes=1 --nproc-per-node N
--master-addr 127.0.0.1 --master-port P bench.py --gpus N ...` (one rank per GPU, NCCL).
Rank 0 prints ONE JSON line.  `value` is the whole-job tokens/s of K timed optimizer
steps (forward, backward, gradient all-reduce, AdamW) with inputs already on the
device, timed by CUDA events between barriers, max over ranks.  `e2e.value` is the
same metric through the public API (`PipelineParallel.train_step`), with each step's
token ids copied from pinned host memory and its loss read back to the host.
`--impl reference` runs the unmodified reference installed under baseline/_ref on
the same config through its own `PipelineParallel.train_step`.
Data are synthetic uniform-random token ids; weights are random-init.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PUBLISHED_TOK_S = {1: 16045.61, 2: 31928.99}  # reference README, hardware unstated

MODELS = {
    "dense": dict(vocab_size=50257, d_model=512, d_head=32, n_heads=16, n_layers=16, max_seq_len=768,
                  ffn_in=2048, num_experts=1, top_k=1, router_alpha=0.01, dtype="bfloat16"),
    "moe": dict(vocab_size=50257, d_model=512, d_head=32, n_heads=16, n_layers=16, max_seq_len=768,
                ffn_in=2048, num_experts=8, top_k=2, router_alpha=0.01, dtype="bfloat16"),
}
BATCH = {"dense": 40, "moe": 16}
LR, SEED = 5e-4, 42


class ClockSampler:
    """Samples SM clocks / throttle reasons of this rank's GPU while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            cols = [c.strip() for c in line.split(",")]
            if len(cols) < 9:
                continue
            try:
                sm.append(float(cols[1])); smax.append(float(cols[2])); power.append(float(cols[3]))
            except ValueError:
                continue
            for name, flag in zip(names, cols[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        loaded = [s for s, p in zip(sm, power) if p > 300.0] or sm
        return {
            "sm_mhz": statistics.median(loaded) if loaded else None,
            "sm_max_mhz": max(smax) if smax else None,
            "power_w_max": max(power) if power else None,
            "samples": len(sm),
            "reasons": sorted(reasons),
        }


def _parallelism(args) -> tuple[int, int, int, str]:
    if args.config == "moe":
        return 1, 1, args.gpus, f"ep{args.gpus}"
    return args.gpus, 1, 1, f"dp{args.gpus}"


def _timed_loop(torch, dist, step_fn, n_steps: int, flush, device, finish_fn=None):
    """K steps between barrier+sync pairs, CUDA-event timed; returns the max over ranks (ms).
    `finish_fn` runs after the last step, inside the timed region (reads still outstanding)."""
    if dist.is_initialized():
        dist.barrier()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    last = None
    for i in range(n_steps):
        flush.zero_()  # 256 MiB write: evicts the 126 MB L2 between steps
        last = step_fn(i)
    if finish_fn is not None:
        last = finish_fn()
    end.record()
    torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier()
    ms = torch.tensor([start.elapsed_time(end)], device=device, dtype=torch.float64)
    if dist.is_initialized():
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms.item(), last


def _host_batches(torch, vocab: int, batch: int, seq: int, count: int, seed: int):
    gen = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(count):
        ids = torch.randint(0, vocab, (batch, seq + 1), generator=gen, dtype=torch.int64)
        out.append((ids[:, :-1].contiguous().pin_memory(), ids[:, 1:].contiguous().pin_memory()))
    return out


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist

    from nanotitan_b200.config import AppConfig
    from nanotitan_b200.dist_env import init_distributed, local_device
    from nanotitan_b200.ops import ext
    from nanotitan_b200.parallel_dims import get_parallel_dims
    from nanotitan_b200.train import build_training
    from nanotitan_b200.utils import seed_everything

    dp, pp, ep, par = _parallelism(args)
    model_kw = dict(MODELS[args.config], moe_backend="cuda")
    batch = BATCH[args.config]
    cfg = AppConfig.model_validate(dict(
        run_name="bench", max_steps=1_000_000, model=model_kw,
        trainer=dict(device_id=0, eval_every_step=-1, per_device_batch_size=batch, seed=SEED),
        data=dict(num_workers=1, train_tokens_path="unused", val_tokens_path="unused"),
        optim=dict(type="adam", lr=LR),
        runtime=dict(name="bench", dp_size=dp, pp_size=pp, ep_size=ep, num_microbatches=1, bucket_size=25),
    ))
    init_distributed()
    device = local_device()
    seed_everything(SEED)
    dims = get_parallel_dims(cfg.runtime)
    model, _, step, optimizer = build_training(cfg, dims)
    seq, vocab = cfg.model.max_seq_len, cfg.model.vocab_size
    host = _host_batches(torch, vocab, batch, seq, 4, SEED + dims.data_rank)
    dev = [(x.to(device), y.to(device)) for x, y in host]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    tokens_per_step = batch * seq * dims.data_world_size

    def device_step(i):
        return step.train_step(model, dev[i % len(dev)], optimizer, collect_metrics=False)

    # End to end through the public API: token ids come from pinned host memory every step and
    # every step's loss is read back to the host.  The read is pipelined (`collect_metrics=
    # "deferred"`): step i's metrics are collected after step i+1 has been launched, the last
    # step's before the timed region closes.
    in_flight = []

    def api_step(i):
        in_flight.append(step.train_step(model, host[i % len(host)], optimizer, collect_metrics="deferred"))
        if len(in_flight) > 1:
            return in_flight.pop(0).result()["train/ce_loss"].value
        return None

    def api_finish():
        loss = None
        while in_flight:
            loss = in_flight.pop(0).result()["train/ce_loss"].value
        return loss

    for i in range(args.warmup):
        device_step(i)
    launches0 = ext.get_ext().launch_count() if ext.have_ext() else 0
    sampler = ClockSampler(device.index or 0)
    sampler.start()
    ms, _ = _timed_loop(torch, dist, device_step, args.steps, flush, device)
    launches = (ext.get_ext().launch_count() - launches0) if ext.have_ext() else 0
    for i in range(min(2, args.warmup)):
        api_step(i)
    api_finish()
    e2e_ms, loss = _timed_loop(torch, dist, api_step, args.steps, flush, device, finish_fn=api_finish)
    clocks = sampler.stop()
    value = tokens_per_step * args.steps / (ms / 1e3)
    e2e = tokens_per_step * args.steps / (e2e_ms / 1e3)
    return {
        "metric": "train_tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": value / PUBLISHED_TOK_S[args.gpus] if args.gpus in PUBLISHED_TOK_S and args.config == "dense" else None,
        "dtype": "bf16", "data": "synthetic uniform-random token ids, random-init weights",
        "impl": "ours",
        "config": {"model": f"nanotitan-{args.config} 16L d512 16x32 ffn2048 vocab50257"
                            + (" E8 top2" if args.config == "moe" else " (E1 top1, 118.6M params untied)"),
                   "global_batch": batch * dims.data_world_size, "seq_len": seq, "parallelism": par,
                   "optimizer": "AdamW lr5e-4 wd0.1, fp32 master weights", "l2": "256 MiB flush write between steps"},
        "clocks": clocks,
        "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                "h2d_bytes_per_step": 2 * batch * seq * 8,
                # two losses + per-layer routing counts as fp32, plus the 16-byte kernel status word
                "d2h_bytes_per_step": 4 * (2 + cfg.model.n_layers * cfg.model.num_experts) + 16,
                "last_loss": loss},
        "gpu_launches": int(launches),
    }


def run_reference(args) -> dict:
    sys.path.insert(0, str(ROOT / "baseline"))
    import ref_harness

    why = ref_harness.available()
    if why is not None:
        return {"impl": "reference", "unavailable": why}
    import torch
    import torch.distributed as dist

    dp, pp, ep, par = _parallelism(args)
    batch = BATCH[args.config]
    if dist.is_available() and "RANK" in os.environ and not dist.is_initialized():
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group(backend="nccl", init_method="env://")
    cfg, dims, model, step, optimizer = ref_harness.build(
        MODELS[args.config], batch, dp, pp, ep, 1, LR, SEED)
    device = torch.device("cuda", dims.local_rank)
    seq, vocab = cfg.model.max_seq_len, cfg.model.vocab_size
    host = _host_batches(torch, vocab, batch, seq, 4, SEED + dims.data_rank)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    tokens_per_step = batch * seq * dims.data_world_size

    def api_step(i):
        # the reference's only step API: inputs copied from the host, losses read back, every step
        return step.train_step(model, host[i % len(host)], optimizer)["train/ce_loss"].value

    for i in range(args.warmup):
        api_step(i)
    sampler = ClockSampler(device.index or 0)
    sampler.start()
    ms, loss = _timed_loop(torch, dist, api_step, args.steps, flush, device)
    clocks = sampler.stop()
    value = tokens_per_step * args.steps / (ms / 1e3)
    return {
        "metric": "train_tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": value / PUBLISHED_TOK_S[args.gpus] if args.gpus in PUBLISHED_TOK_S and args.config == "dense" else None,
        "dtype": "bf16", "data": "synthetic uniform-random token ids, random-init weights",
        "impl": "reference",
        "config": {"model": f"reference NanoTitanModel {args.config} 16L d512 16x32 ffn2048 vocab50257, moe_backend=torch",
                   "global_batch": batch * dims.data_world_size, "seq_len": seq, "parallelism": par,
                   "optimizer": "AdamW lr5e-4 wd0.1, bf16 params", "l2": "256 MiB flush write between steps"},
        "clocks": clocks,
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 2 * batch * seq * 8,
                "d2h_bytes_per_step": 24, "last_loss": loss,
                "note": "the reference's only step API copies inputs from host and reads losses back every step"},
        "gpu_launches": None,
    }


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--config", choices=["dense", "moe"], default="dense")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            # re-launch ourselves under torchrun so `python bench.py --gpus N` also works
            port = 29600 + int(time.time()) % 300
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", str(port), __file__, *sys.argv[1:]]
            raise SystemExit(subprocess.call(cmd))
        raise SystemExit(f"WORLD_SIZE={world} but --gpus {args.gpus}")
    try:
        result = run_reference(args) if args.impl == "reference" else run_ours(args)
    except Exception as exc:  # the reference arm must always print its line and exit 0
        if args.impl != "reference":
            raise
        result = {"impl": "reference", "unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(result), flush=True)
    try:
        import torch.distributed as dist

        if dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass


if __name__ == "__main__":
    main()
