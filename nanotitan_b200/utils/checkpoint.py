"""Sharded checkpoints: one file per rank plus a manifest, written atomically.

The reference never saves anything; the layout to honour is its `state_dict()` key
scheme (stage-local `blocks.<i>` indices, local expert slices).  A shard file holds
that state dict (tensors cloned out of the flat buckets they view into), the
optimizer state, step, token count, the loader position (epoch and batches taken from it),
RNG states and the rank's coordinates.
`consolidate` rebuilds the single-process view (global layer indices, all experts)
so weights can be exchanged with a reference run.
"""
from __future__ import annotations

import copy
import json
import os
import re
import threading
import time
from pathlib import Path

import torch

_STEP_DIR = re.compile(r"step_(\d+)$")


def _rank_file(step_dir: Path, rank: int) -> Path:
    return step_dir / f"rank_{rank:05d}.pt"


def _snapshot(step: int, tokens_seen: int, model, optimizer, dims, data_state, portable_optimizer: bool) -> dict:
    """Everything one rank stores, copied to host memory: nothing in it aliases tensors that training goes on
    changing.  Collective when `portable_optimizer` is set (the sharded optimizer state is gathered)."""
    if optimizer is None:
        optimizer_state = None
    elif hasattr(optimizer, "per_parameter_state"):
        optimizer_state = optimizer.state_dict()  # FusedAdamW: already host copies
    else:
        optimizer_state = copy.deepcopy(optimizer.state_dict())  # torch.optim: the dict refers to the live moments
    return {
        "model": {k: v.detach().clone().cpu() for k, v in model.state_dict().items()},
        "optimizer": optimizer_state,
        "optimizer_by_name": _optimizer_by_name(model, optimizer, dims) if portable_optimizer else None,
        "step": step,
        "tokens_seen": tokens_seen,
        "data": dict(data_state) if data_state else None,
        "rng": {
            "torch": torch.get_rng_state(),
            "cuda": torch.cuda.get_rng_state_all() if torch.cuda.is_available() else None,
        },
        "coords": {
            "global_rank": dims.global_rank, "dp_rank": dims.dp_rank, "pp_rank": dims.pp_rank,
            "ep_rank": dims.ep_rank, "dp_size": dims.dp_size, "pp_size": dims.pp_size,
            "ep_size": dims.ep_size,
        },
        "spec": {
            "layer_start": model.spec.layer_start, "layer_end": model.spec.layer_end,
            "start_expert_id": model.spec.start_expert_id, "end_expert_id": model.spec.end_expert_id,
            "has_token_embed": model.spec.has_token_embed, "has_unembed_head": model.spec.has_unembed_head,
        },
    }


def _manifest(step: int, tokens_seen: int, dims, cfg, data_state) -> dict:
    return {"step": step, "tokens_seen": tokens_seen, "world_size": dims.world_size,
            "data": dict(data_state) if data_state else None,
            "data_world_size": getattr(dims, "data_world_size", None),
            "config": cfg.model_dump(mode="json") if cfg is not None and hasattr(cfg, "model_dump") else None}


def _write_shard(step_dir: Path, rank: int, payload: dict) -> None:
    step_dir.mkdir(parents=True, exist_ok=True)
    target = _rank_file(step_dir, rank)
    tmp = target.with_suffix(".tmp")
    torch.save(payload, tmp)
    os.replace(tmp, target)


def _write_manifest(step_dir: Path, manifest: dict) -> None:
    mtmp = step_dir / "manifest.tmp"
    mtmp.write_text(json.dumps(manifest, indent=2, default=str))
    os.replace(mtmp, step_dir / "manifest.json")


def _step_dir(directory, step: int) -> Path:
    return Path(directory) / f"step_{step:08d}"


def save_checkpoint(directory, step: int, tokens_seen: int, model, optimizer, dims, cfg=None, data_state=None,
                    portable_optimizer: bool = False) -> Path:
    """`data_state` is the loader position ({"epoch", "batches_done"}): a resumed run continues with the batch
    the interrupted one would have taken next.  `portable_optimizer` also stores the optimizer state per
    parameter (whole fp32 tensors under the parameter's name), from which `consolidate_optimizer` +
    `load_full_optimizer` restore it on any dp x pp x ep layout; the bucket-shaped state that is always stored
    resumes on the same layout only."""
    import torch.distributed as dist

    step_dir = _step_dir(directory, step)
    _write_shard(step_dir, dims.global_rank, _snapshot(step, tokens_seen, model, optimizer, dims, data_state, portable_optimizer))
    # The manifest means "every shard is on disk": rank 0 writes it only after all ranks have
    # renamed their file into place.
    many = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
    if many:
        dist.barrier()
    if dims.global_rank == 0:
        _write_manifest(step_dir, _manifest(step, tokens_seen, dims, cfg, data_state))
    if many:
        dist.barrier()  # every rank returns to a complete checkpoint (it may read it back at once)
    return step_dir


class AsyncCheckpointer:
    """`save()` copies this rank's state to host memory and returns; a background thread serialises it and
    renames it into place, so training waits for the copy, not for the disk.  The thread uses no collectives:
    rank 0's thread writes the manifest once it sees every rank's shard file (it polls the folder, for at most
    `timeout_s`).  One save is in flight at a time - the next `save()` and `wait()` join the previous one and
    re-raise what it failed with.  Call `wait()` before the process ends."""

    def __init__(self, timeout_s: float = 600.0):
        self.timeout_s = timeout_s
        self._thread: threading.Thread | None = None
        self._error: BaseException | None = None

    def save(self, directory, step: int, tokens_seen: int, model, optimizer, dims, cfg=None, data_state=None,
             portable_optimizer: bool = False) -> Path:
        self.wait()
        step_dir = _step_dir(directory, step)
        payload = _snapshot(step, tokens_seen, model, optimizer, dims, data_state, portable_optimizer)
        manifest = _manifest(step, tokens_seen, dims, cfg, data_state) if dims.global_rank == 0 else None
        self._thread = threading.Thread(target=self._write, name=f"checkpoint-step-{step}", daemon=True,
                                        args=(step_dir, dims.global_rank, dims.world_size, payload, manifest))
        self._thread.start()
        return step_dir

    def _write(self, step_dir: Path, rank: int, world: int, payload: dict, manifest: dict | None) -> None:
        try:
            _write_shard(step_dir, rank, payload)
            if manifest is None:
                return
            deadline = time.monotonic() + self.timeout_s
            while not all(_rank_file(step_dir, r).exists() for r in range(world)):
                if time.monotonic() > deadline:
                    raise TimeoutError(f"{step_dir}: not every rank's shard appeared within {self.timeout_s:.0f} s; "
                                       "no manifest written, the checkpoint stays incomplete")
                time.sleep(0.05)
            _write_manifest(step_dir, manifest)
        except BaseException as exc:  # noqa: BLE001 - handed to the training thread by wait()
            self._error = exc

    def in_flight(self) -> bool:
        return self._thread is not None and self._thread.is_alive()

    def wait(self) -> None:
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        if self._error is not None:
            error, self._error = self._error, None
            raise RuntimeError(f"asynchronous checkpoint failed: {error}") from error


def _parameter_names(model) -> dict[int, str]:
    return {id(p): name for name, p in model.named_parameters()}


def _optimizer_by_name(model, optimizer, dims):
    names = _parameter_names(model)
    if hasattr(optimizer, "per_parameter_state"):  # FusedAdamW: flat buckets, possibly sharded
        step, state = optimizer._step, optimizer.per_parameter_state(names)  # collective: every rank takes part
    else:  # torch.optim.AdamW: the parameters are their own master weights
        step, state = 0, {}
        for group in optimizer.param_groups:
            for p in group["params"]:
                st = optimizer.state.get(p, {})
                zeros = torch.zeros(p.shape, dtype=torch.float32)
                state[names[id(p)]] = {"master": p.detach().float().cpu().clone(),
                                       "exp_avg": st["exp_avg"].detach().float().cpu().clone() if "exp_avg" in st else zeros,
                                       "exp_avg_sq": st["exp_avg_sq"].detach().float().cpu().clone() if "exp_avg_sq" in st else zeros.clone()}
                step = max(step, int(st.get("step", 0)))
    if dims.dp_rank != 0:
        return None  # replicas of dp rank 0: nothing new to store
    return {"step": step, "state": state}


def is_complete(step_dir) -> bool:
    """A manifest plus one shard file per rank it names."""
    step_dir = Path(step_dir)
    manifest = step_dir / "manifest.json"
    if not manifest.exists():
        return False
    try:
        world = int(json.loads(manifest.read_text())["world_size"])
    except (ValueError, KeyError, json.JSONDecodeError):
        return False
    return all(_rank_file(step_dir, r).exists() for r in range(world))


def latest_checkpoint(directory) -> Path | None:
    """Newest `step_*` folder whose save completed (manifest written and every rank's shard present)."""
    root = Path(directory)
    if _STEP_DIR.search(root.name) and is_complete(root):
        return root
    best = None
    for child in root.glob("step_*"):
        m = _STEP_DIR.search(child.name)
        if m and is_complete(child):
            if best is None or int(m.group(1)) > best[0]:
                best = (int(m.group(1)), child)
    return None if best is None else best[1]


def load_checkpoint(step_dir, model, optimizer, dims) -> dict:
    payload = torch.load(_rank_file(Path(step_dir), dims.global_rank), map_location="cpu", weights_only=False)
    saved = payload["coords"]
    now = {"global_rank": dims.global_rank, "dp_rank": dims.dp_rank, "pp_rank": dims.pp_rank, "ep_rank": dims.ep_rank,
           "dp_size": dims.dp_size, "pp_size": dims.pp_size, "ep_size": dims.ep_size}
    if saved != now:
        raise ValueError(f"checkpoint shard was written at {saved}, this rank is {now}: resume on the same "
                         "dp x pp x ep layout, or rebuild the weights with `consolidate` + `load_full_state`")
    spec_now = {"layer_start": model.spec.layer_start, "layer_end": model.spec.layer_end,
                "start_expert_id": model.spec.start_expert_id, "end_expert_id": model.spec.end_expert_id,
                "has_token_embed": model.spec.has_token_embed, "has_unembed_head": model.spec.has_unembed_head}
    if payload["spec"] != spec_now:
        raise ValueError(f"checkpoint shard covers {payload['spec']}, this rank's model shard is {spec_now}")
    with torch.no_grad():
        own = model.state_dict()
        for key, value in payload["model"].items():
            own[key].copy_(value)  # in place: parameters may view into flat buckets
    if optimizer is not None and payload["optimizer"] is not None:
        optimizer.load_state_dict(payload["optimizer"])
    torch.set_rng_state(payload["rng"]["torch"])
    if payload["rng"]["cuda"] is not None and torch.cuda.is_available():
        torch.cuda.set_rng_state_all(payload["rng"]["cuda"])
    return {"step": payload["step"], "tokens_seen": payload["tokens_seen"], "data": payload.get("data")}


def _load_shards(step_dir) -> list[dict]:
    if not is_complete(step_dir):
        raise FileNotFoundError(f"{step_dir} is not a complete checkpoint (manifest or rank shards missing)")
    shards = [torch.load(p, map_location="cpu", weights_only=False) for p in sorted(Path(step_dir).glob("rank_*.pt"))]
    return [s for s in shards if s["coords"]["dp_rank"] == 0]


def _merge(shards: list[dict], tensors_of) -> dict[str, torch.Tensor]:
    """Single-process view of per-shard {stage-local key: tensor} maps (`tensors_of(shard)`): global block
    indices, expert slices concatenated in expert-rank order, keys in `state_dict()` order."""
    merged: dict[str, torch.Tensor] = {}
    expert_parts: dict[str, dict[int, torch.Tensor]] = {}
    seen: list[str] = []  # keys in the order a model lists them within a block
    for s in shards:
        shift = (s["spec"]["layer_start"] + 1) - (1 if s["spec"]["has_token_embed"] else 0)
        for key, value in tensors_of(s).items():
            m = re.match(r"blocks\.(\d+)\.(.*)", key)
            local, rest = int(m.group(1)), m.group(2)
            if rest.startswith(("token_embed", "position_embed")):
                new_key = f"blocks.0.{rest}"
            else:
                new_key = f"blocks.{local + shift}.{rest}"
            if new_key not in merged and new_key not in expert_parts:
                seen.append(new_key)
            if ".ffn.experts." in new_key:
                expert_parts.setdefault(new_key, {})[s["coords"]["ep_rank"]] = value
            elif s["coords"]["ep_rank"] == 0:
                merged[new_key] = value
    for key, parts in expert_parts.items():
        merged[key] = torch.cat([parts[r] for r in sorted(parts)], dim=0)
    # blocks in ascending order, keys of a block in the model's own order: the order of `state_dict()`
    ordered = sorted(range(len(seen)), key=lambda i: (int(seen[i].split(".")[1]), i))
    return {seen[i]: merged[seen[i]] for i in ordered if seen[i] in merged}


def consolidate(step_dir) -> dict[str, torch.Tensor]:
    """Merge the dp_rank-0 shards of every (pp, ep) coordinate into the state dict a
    single-process model (pp_size = ep_size = 1) would have."""
    return _merge(_load_shards(step_dir), lambda s: s["model"])


def consolidate_optimizer(step_dir) -> dict:
    """{"step": n, "state": {"master" | "exp_avg" | "exp_avg_sq": {single-process parameter name: fp32 tensor}}} of a
    checkpoint saved with `portable_optimizer=True`."""
    shards = _load_shards(step_dir)
    if any(s.get("optimizer_by_name") is None for s in shards):
        raise ValueError(f"{step_dir} was saved without the per-parameter optimizer state (checkpoint.portable_optimizer)")
    state = {key: _merge(shards, lambda s, key=key: {name: rec[key] for name, rec in s["optimizer_by_name"]["state"].items()})
             for key in ("master", "exp_avg", "exp_avg_sq")}
    return {"step": shards[0]["optimizer_by_name"]["step"], "state": state}


def shard_from_full(full_state: dict[str, torch.Tensor], spec) -> dict[str, torch.Tensor]:
    """Inverse of `consolidate` for one rank: pick this stage's blocks (renumbered from the
    stage-local index 0) and this rank's expert slice out of a single-process state dict."""
    n_total = max(int(k.split(".")[1]) for k in full_state)  # index of the unembed block
    out: dict[str, torch.Tensor] = {}
    shift = (spec.layer_start + 1) - (1 if spec.has_token_embed else 0)
    for key, value in full_state.items():
        idx, rest = int(key.split(".")[1]), key.split(".", 2)[2]
        if idx == 0:
            if not spec.has_token_embed:
                continue
            local = 0
        elif idx == n_total:
            if not spec.has_unembed_head:
                continue
            local = idx - shift
        else:
            layer = idx - 1
            if not (spec.layer_start <= layer < spec.layer_end):
                continue
            local = idx - shift
        if ".ffn.experts." in key:
            value = value[spec.start_expert_id : spec.end_expert_id]
        out[f"blocks.{local}.{rest}"] = value
    return out


def load_full_state(model, full_state: dict[str, torch.Tensor]) -> None:
    """Copy a single-process state dict into this rank's shard, in place."""
    own = model.state_dict()
    with torch.no_grad():
        for key, value in shard_from_full(full_state, model.spec).items():
            own[key].copy_(value)


def load_full_optimizer(model, optimizer, full: dict) -> None:
    """Give this rank's optimizer its part of a consolidated optimizer state (`consolidate_optimizer`), whatever the
    layout: this stage's blocks, this rank's expert slice, and of those the bucket slices this rank owns."""
    own = {key: shard_from_full(full["state"][key], model.spec) for key in ("master", "exp_avg", "exp_avg_sq")}
    names = _parameter_names(model)
    by_name = {name: {key: own[key][name] for key in own} for name in names.values()}
    if hasattr(optimizer, "load_per_parameter_state"):
        optimizer.load_per_parameter_state(by_name, names, full["step"])
        return
    with torch.no_grad():  # torch.optim.AdamW
        for group in optimizer.param_groups:
            for p in group["params"]:
                rec = by_name[names[id(p)]]
                p.copy_(rec["master"].to(p.dtype))
                optimizer.state[p] = {"step": torch.tensor(float(full["step"])),
                                      "exp_avg": rec["exp_avg"].to(device=p.device, dtype=p.dtype).clone(),
                                      "exp_avg_sq": rec["exp_avg_sq"].to(device=p.device, dtype=p.dtype).clone()}


def main(argv=None) -> int:
    """`python -m nanotitan_b200.utils.checkpoint consolidate <checkpoint dir or step dir> <out.pt>`: write the
    single-process state dict (the reference's key layout) of a sharded checkpoint, e.g. to load it into the
    reference's model, or with `load_full_state` into a run of another pp x ep layout."""
    import argparse

    ap = argparse.ArgumentParser(description=main.__doc__)
    sub = ap.add_subparsers(dest="command", required=True)
    cons = sub.add_parser("consolidate", help="merge the rank shards into one state dict")
    cons.add_argument("checkpoint", help="a step_* folder, or the folder holding them (newest complete one is taken)")
    cons.add_argument("out", help="file to write (torch.save of {key: tensor})")
    cons.add_argument("--with-optimizer", action="store_true",
                      help="write {'model': ..., 'optimizer': ...} instead (needs checkpoint.portable_optimizer = true)")
    args = ap.parse_args(argv)
    found = latest_checkpoint(args.checkpoint)
    if found is None:
        raise SystemExit(f"no complete checkpoint under {args.checkpoint}")
    state = consolidate(found)
    manifest = json.loads((found / "manifest.json").read_text())
    if args.with_optimizer:
        torch.save({"model": state, "optimizer": consolidate_optimizer(found), "step": manifest["step"],
                    "tokens_seen": manifest["tokens_seen"], "data": manifest.get("data"),
                    "data_world_size": manifest.get("data_world_size")}, args.out)
    else:
        torch.save(state, args.out)
    n = sum(v.numel() for v in state.values())
    print(f"{found}: {len(state)} tensors, {n / 1e6:.2f} M values -> {args.out}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

