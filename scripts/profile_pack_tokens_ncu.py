"""Nsight Compute capture of the token-packing kernel around benchmarks/bench_pack_tokens.py.

    python scripts/profile_pack_tokens_ncu.py [--results-dir profiles/raw/pack_tokens] [--set detailed]
        [--kernel-name 'regex:.*pack_fwd_kernel.*'] [--profile-launches 1] [--tokens 32768] [--hidden-dim 1024] ... [--dry-run]

The reference's launcher of the same name (scripts/profile_pack_tokens_ncu.py:16-140) with the same options.
It is a thin front end of `nanotitan_b200.ncu_kernel`: the capture skips the benchmark's warm-up launches of
the selected kernel, takes `--profile-launches` of them, never touches the GPU's clocks
(`--clock-control none`), and leaves `<stem>.ncu-rep`, `<stem>.log` and `<stem>.cmd.txt` in the results
folder.  Keep the case small: every captured launch is replayed once per pass of the metric set.
"""
from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

DEFAULT_RESULTS_DIR = Path("profiles/raw/pack_tokens")


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--results-dir", type=Path, default=DEFAULT_RESULTS_DIR)
    ap.add_argument("--ncu", default=os.environ.get("NCU", "ncu"))
    ap.add_argument("--set", dest="section_set", default="detailed")
    ap.add_argument("--kernel-name", default="regex:.*pack_fwd_kernel.*")
    ap.add_argument("--profile-launches", type=int, default=1)
    ap.add_argument("--no-force-overwrite", action="store_true")
    ap.add_argument("--dry-run", action="store_true", help="print the ncu command line and stop")
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--hidden-dim", type=int, default=1024)
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--num-experts", type=int, default=16)
    ap.add_argument("--dtype", choices=["fp32", "fp16", "bf16"], default="fp16")
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--check", action="store_true")
    return ap.parse_args(argv)


def stem(args) -> str:
    return f"pack_T{args.tokens}_d{args.hidden_dim}_k{args.top_k}_E{args.num_experts}_{args.dtype}"


def launcher_argv(args) -> list[str]:
    """Arguments for `nanotitan_b200.ncu_kernel.main`."""
    kernel = args.kernel_name[len("regex:"):] if args.kernel_name.startswith("regex:") else args.kernel_name
    bench = [sys.executable, str(ROOT / "benchmarks" / "bench_pack_tokens.py"), "--device", str(args.device),
             "--tokens", str(args.tokens), "--hidden-dim", str(args.hidden_dim), "--top-k", str(args.top_k),
             "--num-experts", str(args.num_experts), "--dtype", args.dtype, "--warmup", str(args.warmup),
             "--iters", str(args.iters)] + (["--check"] if args.check else [])
    out = args.results_dir / stem(args)
    argv = ["--kernel", kernel, "--skip", str(args.warmup), "--count", str(args.profile_launches), "--set", args.section_set,
            "--out", str(out), "--ncu", args.ncu]
    if args.dry_run:
        argv.append("--dry-run")
    return argv + ["--"] + bench


def main(argv=None) -> int:
    from nanotitan_b200 import ncu_kernel

    args = parse_args(argv)
    out = (args.results_dir / stem(args)).with_suffix(".ncu-rep")
    if args.no_force_overwrite and out.exists():
        print(f"{out} exists; not overwriting", file=sys.stderr)
        return 1
    return ncu_kernel.main(launcher_argv(args))


if __name__ == "__main__":
    raise SystemExit(main())
