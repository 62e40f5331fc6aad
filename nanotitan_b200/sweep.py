"""Grid sweeps: ``python -m nanotitan_b200.sweep <sweep.toml> [--dry-run] [--log-level L]``.

A sweep file names a base config and lists values per dotted key; every point of the
cartesian product is validated, named ``<base>__<key>-<value>__...`` and launched as
its own `torch.distributed.run` job (reference: scripts/sweep.py:18-146).  The launch
uses dp*pp*ep processes (the reference forgets ep_size).
"""
from __future__ import annotations

import argparse
import copy
import itertools
import json
import re
import subprocess
import sys
import tempfile
import tomllib
from pathlib import Path
from typing import Any

from nanotitan_b200.config import AppConfig

_BARE_KEY = re.compile(r"[A-Za-z0-9_-]+")


def parse_args(argv=None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(description="Run a grid sweep described by TOML.")
    parser.add_argument("sweep", type=Path, help="Path to the sweep TOML file.")
    parser.add_argument("--dry-run", action="store_true", help="Validate and print every run only.")
    parser.add_argument("--log-level", default="INFO", help="Logging level forwarded to the trainer.")
    return parser.parse_args(argv)


def load_toml(path: Path) -> dict[str, Any]:
    with Path(path).open("rb") as fh:
        return tomllib.load(fh)


def set_dotted_value(config: dict[str, Any], dotted_key: str, value: Any) -> None:
    *parents, leaf = dotted_key.split(".")
    node = config
    for part in parents:
        node = node[part]
    node[leaf] = value


def safe_fragment(value: Any) -> str:
    text = str(value).lower() if isinstance(value, bool) else str(value)
    return re.sub(r"[^A-Za-z0-9_.-]+", "-", text).strip("-")


def make_run_name(base_name: str, overrides: dict[str, Any]) -> str:
    parts = [safe_fragment(base_name)]
    parts += [f"{safe_fragment(k.replace('.', '-'))}-{safe_fragment(v)}" for k, v in overrides.items()]
    return "__".join(parts)


def _toml_value(value: Any) -> str:
    if isinstance(value, bool):
        return "true" if value else "false"
    if isinstance(value, str):
        return json.dumps(value)
    return repr(value)


def _toml_key(key: str) -> str:
    return key if _BARE_KEY.fullmatch(key) else json.dumps(key)


def dump_toml(config: dict[str, Any]) -> str:
    """Minimal TOML writer for nested tables of scalars (enough for AppConfig dumps)."""
    out: list[str] = []

    def emit(table: dict[str, Any], path: tuple[str, ...]) -> None:
        if path:
            if out and out[-1] != "":
                out.append("")
            out.append("[" + ".".join(_toml_key(p) for p in path) + "]")
        out.extend(f"{_toml_key(k)} = {_toml_value(v)}" for k, v in table.items() if not isinstance(v, dict))
        for k, v in table.items():
            if isinstance(v, dict):
                emit(v, (*path, k))

    emit(config, ())
    return "\n".join(out) + "\n"


def build_runs(sweep_path: Path) -> tuple[Path, list[tuple[str, dict[str, Any]]]]:
    sweep = load_toml(sweep_path)
    base_path = Path(sweep["base_config"]).resolve()
    base = AppConfig.model_validate(load_toml(base_path)).model_dump(mode="json")
    keys = list(sweep["parameters"])
    runs = []
    for combo in itertools.product(*(sweep["parameters"][k] for k in keys)):
        overrides = dict(zip(keys, combo, strict=True))
        cfg = copy.deepcopy(base)
        for key, value in overrides.items():
            set_dotted_value(cfg, key, value)
        cfg["run_name"] = make_run_name(str(base["run_name"]), overrides)
        AppConfig.model_validate(cfg)
        runs.append((cfg["run_name"], cfg))
    return base_path, runs


def launch_command(config: dict[str, Any], config_path: Path, log_level: str) -> list[str]:
    rt = config["runtime"]
    world = rt["dp_size"] * rt["pp_size"] * rt.get("ep_size", 1)
    return [
        sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
        f"--nproc-per-node={world}", "-m", "nanotitan_b200.train", f"@{config_path}",
        f"--log.level={log_level}",
    ]


def main(argv=None) -> int:
    args = parse_args(argv)
    sweep_path = args.sweep.resolve()
    base_path, runs = build_runs(sweep_path)
    print(f"Loaded {len(runs)} run(s) from {sweep_path} using {base_path}")
    with tempfile.TemporaryDirectory(prefix="nanotitan-sweep-") as tmp:
        for i, (name, config) in enumerate(runs, start=1):
            cfg_path = Path(tmp) / f"run-{i:04d}.toml"
            cfg_path.write_text(dump_toml(config), encoding="utf-8")
            cmd = launch_command(config, cfg_path, args.log_level)
            print(f"[{i}/{len(runs)}] {name}")
            if args.dry_run:
                print("  " + subprocess.list2cmdline(cmd))
                continue
            subprocess.run(cmd, check=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
