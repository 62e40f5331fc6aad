"""Process-group bootstrap helpers.

Same surface as the reference (src/dist_env.py:7-48) with four differences: the
backend is NCCL when CUDA is present and gloo otherwise, a single process also gets
a (size-1) group so the rank-layout code never special-cases it, and every group
carries a finite timeout so a lost peer ends a collective with an error instead of
a hang; and ranks restarted by the launcher rendezvous under a store prefix of their attempt.
"""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist


def pick_backend() -> str:
    return "nccl" if torch.cuda.is_available() else "gloo"


def init_distributed(timeout_s: float = 600.0, backend: str | None = None) -> None:
    if is_distributed():
        return
    backend = backend or pick_backend()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = get_local_rank()
    if backend == "nccl":
        torch.cuda.set_device(local_rank)
    timeout = datetime.timedelta(seconds=timeout_s)
    if world == 1 and "MASTER_ADDR" not in os.environ:
        # No launcher: rendezvous with ourselves through a file-less TCP store on loopback.
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", str(29500 + os.getpid() % 2000))
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
    kwargs = {}
    if backend == "nccl":
        kwargs["device_id"] = torch.device("cuda", local_rank)
    restart = int(os.environ.get("TORCHELASTIC_RESTART_COUNT", "0"))
    if restart > 0 and os.environ.get("TORCHELASTIC_USE_AGENT_STORE") == str(True):
        # A launcher restart (torchrun --max-restarts) reuses the agent's store, which still holds the
        # rendezvous keys of the attempt that died: the new ranks would read the dead ranks' addresses from
        # it and wait for them.  Every attempt after the first therefore works under a prefix of its own.
        store = dist.TCPStore(os.environ["MASTER_ADDR"], int(os.environ["MASTER_PORT"]), world, is_master=False, timeout=timeout)
        dist.init_process_group(backend=backend, store=dist.PrefixStore(f"nt_attempt_{restart}/", store),
                                rank=int(os.environ["RANK"]), world_size=world, timeout=timeout, **kwargs)
        return
    dist.init_process_group(backend=backend, init_method="env://", timeout=timeout, **kwargs)


def is_distributed() -> bool:
    return dist.is_available() and dist.is_initialized()


def get_world_size() -> int:
    return dist.get_world_size() if is_distributed() else 1


def get_local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", "0"))


def get_rank() -> int:
    return dist.get_rank() if is_distributed() else 0


def is_main_process() -> bool:
    return get_rank() == 0


def barrier() -> None:
    if is_distributed():
        dist.barrier()


def cleanup() -> None:
    if is_distributed():
        dist.destroy_process_group()


def local_device() -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda", get_local_rank())
    return torch.device("cpu")
