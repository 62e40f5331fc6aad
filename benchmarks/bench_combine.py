"""Gate-weighted combine of expert rows on one GPU: the CUDA kernel next to the PyTorch `index_add_` form.

    python benchmarks/bench_combine.py [--backend both] [--tokens 32768] [--hidden-dim 1024] [--top-k 2]
                                       [--dtype fp16] [--warmup 20] [--iters 100] [--check]

Same command line as the reference's benchmarks/bench_combine.py (its :19-30 is the torch form, :97-100 the
printed comparison).  out[t] = sum over the k assignments a of token t of w[a] * y[a], fp32 out.  CUDA-event
times with the 256 MiB L2 flush between iterations, algorithmic bytes, fraction of the measured HBM copy
bandwidth; `--check` compares the two backends.
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

DTYPES = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--backend", choices=["torch", "cuda", "both"], default="both")
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--hidden-dim", type=int, default=1024)
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--dtype", choices=sorted(DTYPES), default="fp16")
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--check", action="store_true")
    return ap.parse_args(argv)


def combine_bytes(tokens: int, hidden: int, k: int, elem: int) -> int:
    """Every expert row read once, the fp32 result written once, token id and gate per assignment."""
    return tokens * k * hidden * elem + tokens * hidden * 4 + tokens * k * 8


def torch_combine(y, token, w, tokens):
    out = torch.zeros(tokens, y.size(1), device=y.device, dtype=torch.float32)
    return out.index_add_(0, token.long(), y.float() * w[:, None])


def main(argv=None) -> int:
    args = parse_args(argv)
    from benchmarks.bench_kernels import report, timed
    from nanotitan_b200.ops.ext import get_ext

    torch.cuda.set_device(args.device)
    device = torch.device("cuda", args.device)
    gen = torch.Generator(device=device).manual_seed(0)
    rows = args.tokens * args.top_k
    y = torch.randn(rows, args.hidden_dim, device=device, generator=gen).to(DTYPES[args.dtype])
    token = torch.arange(args.tokens, device=device, dtype=torch.int32).repeat_interleave(args.top_k)
    token = token[torch.randperm(rows, device=device, generator=gen)].contiguous()  # rows arrive grouped by expert, not by token
    w = torch.rand(rows, device=device, generator=gen)
    nbytes = combine_bytes(args.tokens, args.hidden_dim, args.top_k, y.element_size())
    shape = f"T{args.tokens} d{args.hidden_dim} k{args.top_k} {args.dtype}"
    ext = get_ext()
    if args.backend in ("cuda", "both"):
        ms = timed(lambda: ext.combine_tokens_kernel(y, token, w, args.tokens, args.hidden_dim), args.iters, args.warmup)
        report(f"combine_tokens_kernel {shape}", ms, nbytes=nbytes)
    if args.backend in ("torch", "both"):
        ms = timed(lambda: torch_combine(y, token, w, args.tokens), args.iters, args.warmup)
        report(f"torch index_add_ {shape}", ms, nbytes=nbytes)
    if args.check:
        got = ext.combine_tokens_kernel(y, token, w, args.tokens, args.hidden_dim)
        torch.testing.assert_close(got, torch_combine(y, token, w, args.tokens), rtol=1e-4, atol=1e-4)
        print("check passed")
    status = ext.read_status(True)
    assert status[0] == 0, status
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
