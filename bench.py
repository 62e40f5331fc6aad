"""Headline benchmark: training tokens/s of the 16-layer d512 LM, 40 x 768 tokens per GPU, bf16.

    python bench.py --gpus N --steps K --warmup W [--impl ours|reference]
                    [--config dense|moe|moe3d] [--no-moe] [--parity]

For N > 1 launch with `python -m torch.distributed.run --nnodes=1 --nproc-per-node N
--master-addr 127.0.0.1 --master-port P bench.py --gpus N ...` (one rank per GPU, NCCL).
Rank 0 prints ONE JSON line.

Top level (`--config dense`, the default): the dense model under data parallelism.
`value` is the whole-job tokens/s of K timed optimizer steps (forward, backward, gradient
all-reduce, AdamW) with inputs already on the device, timed by CUDA events between
barriers, max over ranks.  `e2e.value` is the same metric through the public API
(`PipelineParallel.train_step`), with each step's token ids copied from pinned host memory
and its loss read back to the host.

`moe` block (added to the same line unless `--no-moe`): the 8-expert top-2 variant of the
model under expert parallelism (EP = N, 16 x 768 tokens per GPU): tokens/s, ms/step, the
end-to-end figure, and `layer_fwd_bwd_ms`, the device time of one MoE layer's forward +
backward on that batch.  `--config moe` / `--config moe3d` print only that model's line
(`moe3d`: 32 layers, d 1024, 16 experts, pipeline 2 x expert 4, 8 microbatches of 4; 8 GPUs).

`paths` says which kernels moved the gradients and the expert rows ("fused_multimem",
"fused_p2p" or "nccl"), `launches_by_kernel` counts this library's launches inside the timed
region, `replicas_identical` compares every replica's parameters after the timed steps.

`--impl reference` runs the unmodified reference installed under baseline/_ref on the same
configs through its own `PipelineParallel.train_step`.  `--parity` trains both
implementations from one set of weights on the same batches and prints the two loss curves.
Data are synthetic uniform-random token ids; weights are random-init.
"""
from __future__ import annotations

import argparse
import gc
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
    "moe3d": dict(vocab_size=50257, d_model=1024, d_head=64, n_heads=16, n_layers=32, max_seq_len=1024,
                  ffn_in=4096, num_experts=16, top_k=2, router_alpha=0.01, dtype="bfloat16"),
}
MODEL_LABEL = {
    "dense": "16L d512 16x32 ffn2048 vocab50257 E1 top1 (118.6M params, untied)",
    "moe": "16L d512 16x32 ffn2048 vocab50257 E8 top2",
    "moe3d": "32L d1024 16x64 ffn4096 vocab50257 E16 top2",
}
BATCH = {"dense": 40, "moe": 16, "moe3d": 32}
MICROBATCHES = {"dense": 1, "moe": 1, "moe3d": 8}
SEEDS = {"dense": 42, "moe": 42, "moe3d": 0}
LR = 5e-4


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


def _parallelism(config: str, gpus: int) -> tuple[int, int, int, str]:
    """-> dp, pp, ep, label."""
    if config == "moe":
        return 1, 1, gpus, f"ep{gpus}"
    if config == "moe3d":
        if gpus != 8:
            raise SystemExit("--config moe3d is the 8-GPU pipeline 2 x expert 4 layout: run it with --gpus 8")
        return 1, 2, 4, "dp1 x pp2 x ep4, 8 microbatches of 4"
    return gpus, 1, 1, f"dp{gpus}"


def _config_dict(config: str, batch: int, data_world: int, seq: int, par: str) -> dict:
    """Identical wording in both arms; what differs between them goes to `impl_notes`."""
    return {"model": MODEL_LABEL[config], "global_batch": batch * data_world, "seq_len": seq, "parallelism": par,
            "optimizer": "AdamW lr5e-4 wd0.1", "l2": "256 MiB flush write between steps"}


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


def _moe_layer_ms(torch, dist, ffn, params, batch: int, seq: int, d_model: int, flush, device, iters: int = 10):
    """Device time of forward + backward of one MoE layer (all expert-parallel ranks take part),
    L2 flushed before every iteration, mean over `iters`, max over ranks."""
    gen = torch.Generator(device=device).manual_seed(1234 + (dist.get_rank() if dist.is_initialized() else 0))
    x = torch.randn(batch, seq, d_model, device=device, dtype=torch.bfloat16, generator=gen).requires_grad_()
    dy = torch.randn(batch, seq, d_model, device=device, dtype=torch.bfloat16, generator=gen)
    times = []
    for it in range(3 + iters):
        x.grad = None
        for p in params:
            p.grad = None
        flush.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        out = ffn(x)
        out = out[0] if isinstance(out, tuple) else out
        out.backward(dy)
        end.record()
        torch.cuda.synchronize()
        if it >= 3:
            times.append(start.elapsed_time(end))
    ms = torch.tensor([sum(times) / len(times)], device=device, dtype=torch.float64)
    if dist.is_initialized():
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    for p in params:
        p.grad = None
    return ms.item()


def _replicas_identical(torch, dist, reducers) -> bool | None:
    """True when every replica of every data-parallel group holds bit-identical parameters."""
    checked = False
    same = True
    for red in reducers.values():
        if red.group_size < 2:
            continue
        for p in red.params:
            checked = True
            mine = p.detach().float().contiguous()
            hi = mine.clone()
            dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=red.process_group)
            lo = mine.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=red.process_group)
            same = same and bool(torch.equal(hi, lo))
    if not checked:
        return None
    flag = torch.tensor([1 if same else 0], device="cuda", dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(flag.item())


def _paths(model, reducers, dims) -> dict:
    """Which transport carried the gradient buckets and the expert rows in this run."""
    allreduce = None
    for red in reducers.values():
        if red.group_size < 2:
            continue
        engine = red.bucket_engine
        if engine is None:
            kind = "nccl"
        else:
            kind = "fused_multimem" if any(getattr(b, "_mc", 0) for b in red.buckets) else "fused_p2p"
        allreduce = kind if allreduce in (None, kind) else "mixed"
    ep = None
    if dims.ep_size > 1:
        kinds = set()
        for block in model.blocks:
            backend = getattr(getattr(block, "ffn", None), "moe_backend", None)
            if backend is not None and hasattr(backend, "fused_exchange"):
                kinds.add("fused_p2p" if backend.fused_exchange is not None else "nccl")
        ep = kinds.pop() if len(kinds) == 1 else ("mixed" if kinds else None)
    return {"allreduce": allreduce, "ep": ep}


def run_ours(args, config: str) -> dict:
    import torch
    import torch.distributed as dist

    from nanotitan_b200.config import AppConfig
    from nanotitan_b200.dist_env import init_distributed, local_device
    from nanotitan_b200.ops import ext
    from nanotitan_b200.parallel_dims import get_parallel_dims
    from nanotitan_b200.train import build_training
    from nanotitan_b200.utils import seed_everything

    os.environ.setdefault("NT_STRICT", "1")  # an op that would leave this library's kernels raises instead
    os.environ.setdefault("NT_COMM_WAIT_MS", "20000")  # a peer that never arrives ends the wait (and the run) in 20 s
    dp, pp, ep, par = _parallelism(config, args.gpus)
    model_kw = dict(MODELS[config], moe_backend="cuda")
    batch, seed = BATCH[config], SEEDS[config]
    cfg = AppConfig.model_validate(dict(
        run_name="bench", max_steps=1_000_000, model=model_kw,
        # weights: trainer seed (the reference's schema wants it > 0); token ids: `seed` itself
        trainer=dict(device_id=0, eval_every_step=-1, per_device_batch_size=batch, seed=seed or 1),
        data=dict(num_workers=1, train_tokens_path="unused", val_tokens_path="unused"),
        optim=dict(type="adam", lr=LR),
        runtime=dict(name="bench", dp_size=dp, pp_size=pp, ep_size=ep, num_microbatches=MICROBATCHES[config],
                     bucket_size=25),
    ))
    init_distributed()
    device = local_device()
    seed_everything(seed or 1)
    dims = get_parallel_dims(cfg.runtime)
    model, dp_wrap, step, optimizer = build_training(cfg, dims)
    reducers = dp_wrap.get_reducers()
    if args.gpus > 1 and dp * ep > 1 and os.environ.get("NT_FUSED_ALLREDUCE", "1") != "0":
        if reducers["shared"].bucket_engine is None:
            raise RuntimeError("the fused all-reduce engine could not be set up on this multi-GPU run; "
                               "set NT_FUSED_ALLREDUCE=0 to benchmark the NCCL path on purpose")
    seq, vocab = cfg.model.max_seq_len, cfg.model.vocab_size
    host = _host_batches(torch, vocab, batch, seq, 4, seed + dims.data_rank)
    dev = [(x.to(device), y.to(device)) for x, y in host]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    tokens_per_step = batch * seq * dims.data_world_size
    native = ext.get_ext()

    def device_step(i):
        return step.train_step(model, dev[i % len(dev)], optimizer, collect_metrics=False)

    # End to end through the public API: token ids come from pinned host memory every step and
    # every step's loss is read back to the host.  The read is pipelined (`collect_metrics=
    # "deferred"`): step i's metrics are collected after step i+1 has been launched, the last
    # step's before the timed region closes.
    in_flight = []

    recv_wait = []  # per step: compute-stream idle seconds across the waits for pipeline-boundary tensors

    def _collect(pending):
        metrics = pending.result()
        recv_wait.append(metrics["time/pp_recv_wait"].value)
        return metrics["train/ce_loss"].value

    def api_step(i):
        in_flight.append(step.train_step(model, host[i % len(host)], optimizer, collect_metrics="deferred"))
        if len(in_flight) > 1:
            return _collect(in_flight.pop(0))
        return None

    def api_finish():
        loss = None
        while in_flight:
            loss = _collect(in_flight.pop(0))
        return loss

    for i in range(max(args.warmup, 3)):  # two ordinary steps, then the step that captures the CUDA graph
        device_step(i)
        if os.environ.get("NT_BENCH_SYNC_WARMUP") == "1":  # debugging aid: name the warm-up step a fault belongs to
            torch.cuda.synchronize()
            print(f"[rank {dims.global_rank}] warm-up step {i} done, status {native.read_status(False)}", flush=True)
    torch.cuda.synchronize()
    if ep > 1 and os.environ.get("NT_FUSED_EP", "1") != "0" and _paths(model, reducers, dims)["ep"] != "fused_p2p":
        raise RuntimeError("the fused expert-parallel exchange could not be set up on this multi-GPU run; "
                           "set NT_FUSED_EP=0 to benchmark the NCCL path on purpose")
    launches0, by_kernel0 = native.launch_count(), native.launch_counts()
    sampler = ClockSampler(device.index or 0)
    sampler.start()
    ms, _ = _timed_loop(torch, dist, device_step, args.steps, flush, device)
    launches = native.launch_count() - launches0
    by_kernel = {k: v - by_kernel0.get(k, 0) for k, v in native.launch_counts().items() if v - by_kernel0.get(k, 0)}
    graphed = step.graph_replays > 0
    if graphed:  # a replayed CUDA graph launches its kernels without passing through the host-side counters
        per_step, per_kernel = step.launches_last_step()
        launches += per_step * args.steps
        for k, v in per_kernel.items():
            by_kernel[k] = by_kernel.get(k, 0) + v * args.steps
    status = native.read_status(True)  # a device-side wait that ran out or a failed check voids the run
    if status[0] != 0:
        raise RuntimeError(f"device status word after the timed steps: {status}")
    for i in range(min(2, args.warmup)):
        api_step(i)
    api_finish()
    e2e_ms, loss = _timed_loop(torch, dist, api_step, args.steps, flush, device, finish_fn=api_finish)
    clocks = sampler.stop()
    value = tokens_per_step * args.steps / (ms / 1e3)
    e2e = tokens_per_step * args.steps / (e2e_ms / 1e3)
    result = {
        "metric": "train_tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": value / PUBLISHED_TOK_S[args.gpus] if args.gpus in PUBLISHED_TOK_S and config == "dense" else None,
        "dtype": "bf16", "data": "synthetic uniform-random token ids, random-init weights",
        "impl": "ours",
        "config": _config_dict(config, batch, dims.data_world_size, seq, par),
        "impl_notes": "bf16 parameters with fp32 master weights; moe_backend=cuda (sm_100a kernels)",
        "clocks": clocks,
        "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                "h2d_bytes_per_step": 2 * batch * seq * 8,
                # two losses + per-layer routing counts as fp32, plus the 16-byte kernel status word
                "d2h_bytes_per_step": 4 * (2 + (cfg.model.n_layers // pp) * cfg.model.num_experts) + 16,
                "last_loss": loss},
        "gpu_launches": int(launches),
        "launches_by_kernel": by_kernel,
        "cuda_graph": graphed,
        "paths": _paths(model, reducers, dims),
        "replicas_identical": _replicas_identical(torch, dist, reducers) if args.gpus > 1 else None,
    }
    if pp > 1:
        # stage idle time waiting for boundary tensors, mean over the timed end-to-end steps, max over ranks
        w = torch.tensor([sum(recv_wait[-args.steps:]) / max(1, args.steps) * 1e3], device=device, dtype=torch.float64)
        dist.all_reduce(w, op=dist.ReduceOp.MAX)
        result["pp_recv_wait_ms_per_step"] = w.item()
        result["pp_prepost"] = os.environ.get("NT_PP_PREPOST", "1") != "0"
    if cfg.model.num_experts > 1:
        ffn = next(b.ffn for b in model.blocks if hasattr(b, "ffn"))
        result["layer_fwd_bwd_ms"] = _moe_layer_ms(torch, dist, ffn, list(ffn.parameters()), batch // MICROBATCHES[config],
                                                   seq, cfg.model.d_model, flush, device)
    del model, step, optimizer, dp_wrap, reducers, dev
    gc.collect()
    torch.cuda.empty_cache()
    return result


def run_reference(args, config: str) -> dict:
    sys.path.insert(0, str(ROOT / "baseline"))
    import ref_harness

    why = ref_harness.available()
    if why is not None:
        return {"impl": "reference", "unavailable": why}
    import torch
    import torch.distributed as dist

    dp, pp, ep, par = _parallelism(config, args.gpus)
    batch, seed = BATCH[config], SEEDS[config]
    if dist.is_available() and "RANK" in os.environ and not dist.is_initialized():
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group(backend="nccl", init_method="env://")
    cfg, dims, model, step, optimizer = ref_harness.build(
        MODELS[config], batch, dp, pp, ep, MICROBATCHES[config], LR, seed or 1)
    device = torch.device("cuda", dims.local_rank)
    seq, vocab = cfg.model.max_seq_len, cfg.model.vocab_size
    host = _host_batches(torch, vocab, batch, seq, 4, seed + dims.data_rank)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    tokens_per_step = batch * seq * dims.data_world_size

    def api_step(i):
        # the reference's only step API: inputs copied from the host, losses read back, every step
        return step.train_step(model, host[i % len(host)], optimizer)["train/ce_loss"].value

    # With expert parallelism the reference builds its permutation with one host-side tensor write per
    # row (src/model/torch_backend.py:111-124): seconds per step.  Three warm-up and at most two timed
    # steps keep its run within minutes.
    n_warm, n_steps = (3, min(args.steps, 2)) if ep > 1 else (args.warmup, args.steps)
    for i in range(n_warm):
        api_step(i)
    sampler = ClockSampler(device.index or 0)
    sampler.start()
    ms, loss = _timed_loop(torch, dist, api_step, n_steps, flush, device)
    clocks = sampler.stop()
    value = tokens_per_step * n_steps / (ms / 1e3)
    result = {
        "metric": "train_tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": n_steps, "warmup": n_warm, "ms_per_step": ms / n_steps,
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": value / PUBLISHED_TOK_S[args.gpus] if args.gpus in PUBLISHED_TOK_S and config == "dense" else None,
        "dtype": "bf16", "data": "synthetic uniform-random token ids, random-init weights",
        "impl": "reference",
        "config": _config_dict(config, batch, dims.data_world_size, seq, par),
        "impl_notes": "bf16 parameters, no master weights; moe_backend=torch (the reference's only runnable / "
                      "expert-parallel backend); NCCL bucketed all-reduce and all_to_all_single",
        "clocks": clocks,
        "e2e": {"value": value, "unit": "tokens/s", "ms_per_step": ms / n_steps,
                "h2d_bytes_per_step": 2 * batch * seq * 8,
                "d2h_bytes_per_step": 24, "last_loss": loss,
                "note": "the reference's only step API copies inputs from host and reads losses back every step"},
        "gpu_launches": None,
    }
    if cfg.model.num_experts > 1:
        ffn = next(b.ffn for b in model.blocks if hasattr(b, "ffn"))
        result["layer_fwd_bwd_ms"] = _moe_layer_ms(torch, dist, ffn, list(ffn.parameters()), batch // MICROBATCHES[config],
                                                   seq, cfg.model.d_model, flush, device, iters=2 if ep > 1 else 10)
    del model, step, optimizer
    gc.collect()
    torch.cuda.empty_cache()
    return result


MOE_KEYS = ("value", "unit", "ms_per_step", "steps", "warmup", "config", "e2e", "layer_fwd_bwd_ms", "gpu_launches",
            "launches_by_kernel", "cuda_graph", "paths", "replicas_identical", "unavailable")


def run(args) -> dict:
    one = run_reference if args.impl == "reference" else run_ours
    result = one(args, args.config)
    if args.config == "dense" and not args.no_moe and "unavailable" not in result:
        try:
            moe = one(args, "moe")
        except Exception as exc:  # the dense headline stands on its own; the block says why it is missing
            print(f"[bench] the expert-parallel block failed on rank {os.environ.get('RANK', '0')}: "
                  f"{type(exc).__name__}: {exc}", file=sys.stderr, flush=True)
            moe = {"unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"}
        result["moe"] = {k: moe[k] for k in MOE_KEYS if k in moe}
        result["moe"]["metric"] = "train_tokens_per_sec (8 experts top-2, expert parallel over all GPUs); layer_fwd_bwd_ms = one MoE layer forward+backward"
    return result


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--config", choices=["dense", "moe", "moe3d"], default="dense")
    ap.add_argument("--no-moe", action="store_true", help="skip the expert-parallel block of the default run")
    ap.add_argument("--parity", action="store_true",
                    help="loss curves of both implementations from the same weights and batches (1 GPU)")
    ap.add_argument("--parity-steps", type=int, default=20)
    args = ap.parse_args()
    if args.parity:
        sys.path.insert(0, str(ROOT / "benchmarks"))
        import parity

        print(json.dumps(parity.run_parity(MODELS["moe" if args.config == "moe" else "dense"],
                                           BATCH[args.config], args.parity_steps, LR)), flush=True)
        return
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
        result = run(args)
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
