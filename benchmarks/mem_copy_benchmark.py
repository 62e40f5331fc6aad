"""Copy-bandwidth microbenchmark: element-wise vs 16-byte vector copy kernels vs `torch.Tensor.copy_`
at several sizes, and GPU-to-GPU peer copy when two GPUs are visible (reference:
benchmarks/mem_copy_benchmark.py, whose peer-copy case calls a function its extension never binds).

    python benchmarks/mem_copy_benchmark.py [--sizes-gib 1 4] [--iters 10]
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from nanotitan_b200.ops.ext import get_ext  # noqa: E402


def timed(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes-gib", type=float, nargs="+", default=[1.0, 4.0])
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    ext = get_ext()
    for gib in args.sizes_gib:
        n = int(gib * (1 << 30)) // 4
        src = torch.randn(n, device="cuda")
        dst = torch.empty_like(src)
        for name, fn in (("copy_scalar", lambda: ext.copy_scalar(src, dst, n)), ("copy_vector", lambda: ext.copy_vector(src, dst)),
                         ("torch.copy_", lambda: dst.copy_(src))):
            ms = timed(fn, args.iters)
            print(json.dumps({"case": f"{name} {gib} GiB", "ms": round(ms, 3), "gbs_read_plus_write": round(2 * n * 4 / ms / 1e6, 1)}))
        if torch.cuda.device_count() > 1:
            peer = torch.empty(n, device="cuda:1")
            ms = timed(lambda: ext.peer_copy_scalar(src, peer), args.iters)
            print(json.dumps({"case": f"peer_copy 0->1 {gib} GiB", "ms": round(ms, 3), "gbs_one_direction": round(n * 4 / ms / 1e6, 1)}))
        del src, dst


if __name__ == "__main__":
    main()
