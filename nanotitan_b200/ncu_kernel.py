"""Nsight Compute launcher for one kernel of one command.

    python -m nanotitan_b200.ncu_kernel --kernel gemm_tc_kernel --skip 3 --count 1 \\
        --out profiles/raw/gemm -- python benchmarks/bench_kernels.py --only single --iters 2

Generalises the reference's pack-tokens-only launcher (scripts/profile_pack_tokens_ncu.py:16-140):
any kernel-name regex, any command, `--set` / `--section` selection, and always
`--clock-control none` so the GPU's clocks are left alone.  The command line is also written next
to the report (`<out>.cmd.txt`) and ncu's log is teed to `<out>.log`.  Keep the profiled case
small: a capture replays every selected launch dozens of times.
"""
from __future__ import annotations

import argparse
import shlex
import shutil
import subprocess
import sys
from pathlib import Path


def build_command(args, target: list[str]) -> list[str]:
    cmd = [args.ncu, "--clock-control", "none", "--target-processes", "all"]
    if args.sections:
        for sec in args.sections:
            cmd += ["--section", sec]
    else:
        cmd += ["--set", args.set]
    if args.kernel:
        cmd += ["--kernel-name", f"regex:{args.kernel}"]
    cmd += ["--launch-skip", str(args.skip), "--launch-count", str(args.count), "--force-overwrite",
            "--export", str(args.out)]
    return cmd + target


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--kernel", default="", help="regex on the kernel name")
    ap.add_argument("--skip", type=int, default=0, help="matching launches to skip (warm-up)")
    ap.add_argument("--count", type=int, default=1, help="matching launches to capture (keep it at 1-3)")
    ap.add_argument("--set", default="full", help="ncu metric set when no --section is given")
    ap.add_argument("--section", dest="sections", action="append", help="ncu section (repeatable)")
    ap.add_argument("--out", type=Path, default=Path("profiles/raw/capture"))
    ap.add_argument("--ncu", default=shutil.which("ncu") or "ncu")
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("target", nargs=argparse.REMAINDER, help="-- command to profile")
    args = ap.parse_args(argv)
    target = args.target[1:] if args.target[:1] == ["--"] else args.target
    if not target:
        ap.error("give the command to profile after --")
    cmd = build_command(args, target)
    line = " ".join(shlex.quote(c) for c in cmd)
    if args.dry_run:
        print(line)
        return 0
    args.out.parent.mkdir(parents=True, exist_ok=True)
    args.out.with_suffix(".cmd.txt").write_text(line + "\n")
    with args.out.with_suffix(".log").open("w") as log:
        proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        for out_line in proc.stdout:
            sys.stdout.write(out_line)
            log.write(out_line)
        return proc.wait()


if __name__ == "__main__":
    raise SystemExit(main())
