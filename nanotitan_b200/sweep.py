"""Grid sweeps: ``python -m nanotitan_b200.sweep <sweep.toml> [--dry-run] [--summarize] [--log-level L]``.

A sweep file names a base config and lists values per dotted key
(`"optim.lr" = [1e-3, 5e-4]`).  The runner works on the *flat* form of a config - a
`{"optim.lr": 0.001, "model.dtype": "bfloat16", ...}` map obtained from the validated
`AppConfig` - so that an override is a plain dict update, a grid point is the base map plus one
choice per swept key, and the TOML of a run is written straight from the flat map.  Every point is
validated again as an `AppConfig`, named ``<base>__<key>-<value>__...`` and launched as its own
`torch.distributed.run` job with dp*pp*ep processes (the reference's runner, scripts/sweep.py:97-144,
sizes the job without ep_size).
"""
from __future__ import annotations

import argparse
import itertools
import json
import re
import subprocess
import sys
import tempfile
import tomllib
from collections.abc import Iterator
from pathlib import Path
from typing import Any

from nanotitan_b200.config import AppConfig

Flat = dict[str, Any]


# ------------------------------------------------------------------ flat <-> nested
def flatten(tree: dict[str, Any], prefix: str = "") -> Flat:
    flat: Flat = {}
    for key, value in tree.items():
        path = f"{prefix}{key}"
        if isinstance(value, dict):
            flat.update(flatten(value, path + "."))
        else:
            flat[path] = value
    return flat


def unflatten(flat: Flat) -> dict[str, Any]:
    tree: dict[str, Any] = {}
    for path, value in flat.items():
        *tables, leaf = path.split(".")
        node = tree
        for name in tables:
            node = node.setdefault(name, {})
        node[leaf] = value
    return tree


def _scalar(value: Any) -> str:
    if isinstance(value, bool):
        return "true" if value else "false"
    if isinstance(value, (int, float)):
        return repr(value)
    if isinstance(value, (list, tuple)):
        return "[" + ", ".join(_scalar(v) for v in value) + "]"
    return json.dumps(str(value))


def dump_toml(config: dict[str, Any]) -> str:
    """TOML text of a nested config of scalars: top-level keys first, then one `[table]` per
    distinct key prefix in first-seen order."""
    flat = flatten(config)
    by_table: dict[str, list[str]] = {}
    for path, value in flat.items():
        if value is None:
            continue  # TOML has no null; absent means "use the default"
        table, _, leaf = path.rpartition(".")
        by_table.setdefault(table, []).append(f"{leaf} = {_scalar(value)}")
    chunks = ["\n".join(by_table.pop("", []))]
    chunks += [f"[{table}]\n" + "\n".join(lines) for table, lines in by_table.items()]
    return "\n\n".join(c for c in chunks if c) + "\n"


# ------------------------------------------------------------------ grid
def _slug(value: Any) -> str:
    text = str(value).lower() if isinstance(value, bool) else str(value)
    return re.sub(r"[^A-Za-z0-9_.-]+", "-", text).strip("-")


def grid_points(parameters: dict[str, list[Any]]) -> Iterator[Flat]:
    keys = list(parameters)
    for choice in itertools.product(*(parameters[k] for k in keys)):
        yield dict(zip(keys, choice, strict=True))


def run_name(base: str, overrides: Flat) -> str:
    return "__".join([_slug(base)] + [f"{_slug(k.replace('.', '-'))}-{_slug(v)}" for k, v in overrides.items()])


def build_runs(sweep_path: Path) -> tuple[Path, list[tuple[str, dict[str, Any]]]]:
    """-> (base config path, [(run name, nested config dict)]) for every grid point."""
    with Path(sweep_path).open("rb") as fh:
        sweep = tomllib.load(fh)
    base_path = Path(sweep["base_config"]).resolve()
    with base_path.open("rb") as fh:
        base = flatten(AppConfig.model_validate(tomllib.load(fh)).model_dump(mode="json"))
    runs = []
    for overrides in grid_points(sweep["parameters"]):
        unknown = [k for k in overrides if k not in base]
        if unknown:
            raise KeyError(f"sweep keys not in the config schema: {unknown}")
        point = {**base, **overrides, "run_name": run_name(str(base["run_name"]), overrides)}
        config = AppConfig.model_validate(unflatten(point)).model_dump(mode="json")
        runs.append((config["run_name"], config))
    return base_path, runs


# ------------------------------------------------------------------ launch
def launch_command(config: dict[str, Any], config_path: Path, log_level: str) -> list[str]:
    runtime = config["runtime"]
    ranks = runtime["dp_size"] * runtime["pp_size"] * runtime.get("ep_size", 1)
    return [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
            f"--nproc-per-node={ranks}", "-m", "nanotitan_b200.train", f"@{config_path}", f"--log.level={log_level}"]


# ------------------------------------------------------------------ results
def summarize(runs: list[tuple[str, dict[str, Any]]], log_root: Path = Path("runs"), tail: int = 10) -> list[dict[str, Any]]:
    """One row per run from the `metrics.jsonl` its trainer wrote: steps logged, mean cross-entropy and mean
    tokens/s over the last `tail` logged steps (None where a run has not logged anything yet)."""
    rows = []
    for name, _config in runs:
        path = Path(log_root) / name / "metrics.jsonl"
        records = []
        if path.exists():
            records = [json.loads(line) for line in path.read_text().splitlines() if line.strip()]
            records = [r for r in records if "train/ce_loss" in r]
        last = records[-tail:]

        def mean(key):
            values = [r[key] for r in last if key in r]
            return sum(values) / len(values) if values else None

        rows.append({"run": name, "steps": len(records), "ce_loss": mean("train/ce_loss"),
                     "tokens_per_second": mean("train/tokens_per_second")})
    return rows


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description="Run every point of a grid sweep described by a TOML file.")
    parser.add_argument("--summarize", action="store_true",
                        help="launch nothing: print what the runs of this sweep have logged so far, best loss first")
    parser.add_argument("sweep", type=Path, help="sweep TOML: base_config + [parameters]")
    parser.add_argument("--dry-run", action="store_true", help="validate and print the launch commands only")
    parser.add_argument("--log-level", default="INFO", help="logging level passed to the trainer")
    args = parser.parse_args(argv)
    base_path, runs = build_runs(args.sweep.resolve())
    print(f"{len(runs)} run(s) from {args.sweep} over {base_path}")
    if args.summarize:
        rows = sorted(summarize(runs), key=lambda r: (r["ce_loss"] is None, r["ce_loss"]))
        for r in rows:
            loss = "-" if r["ce_loss"] is None else f"{r['ce_loss']:.4f}"
            rate = "-" if r["tokens_per_second"] is None else f"{r['tokens_per_second']:.0f}"
            print(f"{loss:>10}  {rate:>12} tok/s  {r['steps']:>7} steps  {r['run']}")
        return 0
    with tempfile.TemporaryDirectory(prefix="nt-sweep-") as scratch:
        for number, (name, config) in enumerate(runs, start=1):
            toml_path = Path(scratch) / f"{number:04d}-{name[:80]}.toml"
            toml_path.write_text(dump_toml(config), encoding="utf-8")
            command = launch_command(config, toml_path, args.log_level)
            print(f"[{number}/{len(runs)}] {name}")
            if args.dry_run:
                print("    " + subprocess.list2cmdline(command))
            else:
                subprocess.run(command, check=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
