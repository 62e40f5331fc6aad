"""Runs the UNMODIFIED reference (installed under baseline/_ref) through its own public API.

The install flattens the reference's `src` package into baseline/_ref (config.py,
model/, parallel/, ...), while its modules import each other as `src.<name>`; a
module object named `src` whose `__path__` is that folder restores the import path
without touching a file.  The call sequence below is the reference's `main()`
(src/train.py:81-185): config -> ParallelDims -> shard spec -> NanoTitanModel ->
DataParallel.prepare_model -> PipelineParallel.train_step in a loop.  Work-arounds for
defects of the reference that would stop any run, none of which changes what is timed:
  * the process group is initialised here (the reference skips it for one process and
    then calls `dist.new_group`);
  * `moe_backend = "torch"` (its CUDA backend cannot be constructed: 4 arguments are
    passed to a 3-argument constructor, and it has no expert-parallel path);
  * batches come from pinned host tensors of uniform-random ids (what its DataLoader
    with `pin_memory=True` over a synthetic token file would yield).
Nothing of `nanotitan_b200` is imported on this path.
"""
from __future__ import annotations

import os
import sys
import types
from pathlib import Path

REF_DIR = Path(__file__).resolve().parent / "_ref"


def available() -> str | None:
    """None when the install is usable, else a one-line reason."""
    if not (REF_DIR / "train.py").exists():
        return f"reference not installed under {REF_DIR}"
    return None


def _alias_src() -> None:
    if "src" in sys.modules:
        return
    pkg = types.ModuleType("src")
    pkg.__path__ = [str(REF_DIR)]
    sys.modules["src"] = pkg
    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))  # for the reference's own `nanotitan_cuda`


def build(model_kw: dict, per_device_batch: int, dp: int, pp: int, ep: int, microbatches: int,
          lr: float, seed: int, bucket_mib: int = 25):
    """Returns (cfg, dims, model, pp_step, optimizer) built by reference code only."""
    import torch
    import torch.distributed as dist

    _alias_src()
    from src.config import AppConfig
    from src.model.model import NanoTitanModel
    from src.model.utils import get_model_shard_specs
    from src.optim import setup_optimizer
    from src.parallel import DataParallel, PipelineParallel
    from src.parallel_dims import get_parallel_dims
    from src.utils import resolve_dtype, seed_everything

    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
        dist.init_process_group(backend="nccl", init_method="env://")

    cfg = AppConfig.model_validate(dict(
        run_name="reference_bench", max_steps=1_000_000,
        model=dict(model_kw, moe_backend="torch"),
        trainer=dict(device_id=0, eval_every_step=-1, per_device_batch_size=per_device_batch, seed=seed),
        data=dict(num_workers=1, train_tokens_path="unused", val_tokens_path="unused"),
        optim=dict(type="adam", lr=lr),
        runtime=dict(name="bench", dp_size=dp, pp_size=pp, ep_size=ep,
                     num_microbatches=microbatches, bucket_size=bucket_mib),
    ))
    seed_everything(cfg.trainer.seed)
    dims = get_parallel_dims(cfg.runtime)
    spec = get_model_shard_specs(dims, cfg)
    cfg.model.dtype = resolve_dtype(cfg.model.dtype)
    cfg.model.moe_router_dtype = resolve_dtype(cfg.model.moe_router_dtype)
    model = NanoTitanModel.from_specs(cfg.model, spec)
    dp_wrap = DataParallel(cfg, dims)
    dp_wrap.prepare_model(model)
    step = PipelineParallel(cfg, dims, dp_wrap.get_reducers())
    optimizer = setup_optimizer(cfg.optim, model)
    return cfg, dims, model, step, optimizer
