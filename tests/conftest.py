"""Shared fixtures: the `gpu` marker and a multi-process (gloo, CPU) launcher."""
from __future__ import annotations

import os
import sys
import tempfile
import traceback
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs on a B200)")
    config.addinivalue_line("markers", "cuda: alias kept for the reference's marker name")
    config.addinivalue_line("markers", "distributed: spawns several torch.distributed ranks")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _repo_cwd(monkeypatch):
    monkeypatch.chdir(ROOT)


def _worker(rank, world_size, init_file, fn, args, err_dir, backend="gloo"):
    import torch.distributed as dist

    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world_size))
    try:
        if backend == "nccl":
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
            torch.cuda.set_device(rank)
            dist.init_process_group("nccl", init_method=f"file://{init_file}", rank=rank, world_size=world_size,
                                    device_id=torch.device("cuda", rank))
        else:
            dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world_size)
        fn(rank, world_size, *args)
    except Exception:
        Path(err_dir, f"rank{rank}.err").write_text(traceback.format_exc())
        raise
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_distributed(fn, world_size: int, *args, timeout: float = 240.0, backend: str = "gloo"):
    """Run `fn(rank, world_size, *args)` on `world_size` ranks (gloo on CPU, or nccl with one GPU
    per rank); re-raise the first failure."""
    import torch.multiprocessing as mp

    with tempfile.TemporaryDirectory() as tmp:
        init_file = os.path.join(tmp, "rdzv")
        ctx = mp.spawn(_worker, args=(world_size, init_file, fn, args, tmp, backend), nprocs=world_size, join=False)
        try:
            ok = ctx.join(timeout)
            while not ok:
                ok = ctx.join(timeout)
        except Exception as exc:
            errs = sorted(Path(tmp).glob("*.err"))
            detail = "\n".join(p.read_text() for p in errs)
            raise AssertionError(f"distributed test failed:\n{detail or exc}") from exc
