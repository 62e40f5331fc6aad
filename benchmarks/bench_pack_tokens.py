"""Token packing on one GPU: count -> slot assignment -> pack, through the reference-compatible entry points.

    python benchmarks/bench_pack_tokens.py [--tokens 32768] [--hidden-dim 1024] [--top-k 2] [--num-experts 16]
                                           [--dtype fp16] [--warmup 20] [--iters 100] [--check]

Same command line and the same three stages as the reference's benchmarks/bench_pack_tokens.py (its
:161-207 times `count_expert_kernel`, the offsets and `pack_tokens_kernel` with CUDA events and prints an
approximate GB/s).  Here each stage is timed with the 256 MiB L2 flush between iterations and reported with
its algorithmic bytes and the fraction of the measured HBM copy bandwidth (MEASURED_PEAKS.json, 6650 GB/s
when that file is absent); `--check` compares the packed rows with a plain PyTorch gather.
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
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--hidden-dim", type=int, default=1024)
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--num-experts", type=int, default=16)
    ap.add_argument("--dtype", choices=sorted(DTYPES), default="fp16")
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--check", action="store_true")
    args = ap.parse_args(argv)
    if not 1 <= args.top_k <= min(32, args.num_experts):
        ap.error("--top-k must be between 1 and min(32, --num-experts)")
    return args


def stage_bytes(tokens: int, hidden: int, k: int, experts: int, elem: int) -> dict[str, int]:
    """Bytes each stage has to move: ids in / counts out; ids in / slots out; one read of every token row,
    k writes of it, plus the per-assignment token id, expert id and gate."""
    return {
        "count": tokens * k * 4 + experts * 4,
        "assign_slots": tokens * k * 4 * 2 + experts * 4 * 2,
        "pack": tokens * hidden * elem * (1 + k) + tokens * k * (4 + 4 + 4 + 4),
    }


def make_inputs(args, device):
    gen = torch.Generator(device=device).manual_seed(0)
    x = torch.randn(args.tokens, args.hidden_dim, device=device, generator=gen).to(DTYPES[args.dtype])
    scores = torch.rand(args.tokens, args.num_experts, device=device, generator=gen)
    gates, idx = scores.topk(args.top_k, dim=1)  # distinct experts per token, as a router produces
    return x, gates.float().contiguous(), idx.to(torch.int32).contiguous()


def main(argv=None) -> int:
    args = parse_args(argv)
    from benchmarks.bench_kernels import report, timed
    from nanotitan_b200.ops.ext import get_ext

    torch.cuda.set_device(args.device)
    device = torch.device("cuda", args.device)
    ext = get_ext()
    x, gates, idx = make_inputs(args, device)
    nbytes = stage_bytes(args.tokens, args.hidden_dim, args.top_k, args.num_experts, x.element_size())
    shape = f"T{args.tokens} d{args.hidden_dim} k{args.top_k} E{args.num_experts} {args.dtype}"
    no_mask = idx.new_empty(0)

    ms = timed(lambda: ext.count_expert_kernel(idx, no_mask, args.num_experts, args.top_k), args.iters, args.warmup)
    report(f"count_expert_kernel {shape}", ms, nbytes=nbytes["count"])
    counts = ext.count_expert_kernel(idx, no_mask, args.num_experts, args.top_k)
    ms = timed(lambda: ext.assign_slots(idx, counts), args.iters, args.warmup)
    report(f"assign_slots {shape}", ms, nbytes=nbytes["assign_slots"])
    offsets, _ = ext.assign_slots(idx, counts)
    ms = timed(lambda: ext.pack_tokens_kernel(x, gates, idx, offsets.clone()), args.iters, args.warmup)
    report(f"pack_tokens_kernel {shape}", ms, nbytes=nbytes["pack"])

    if args.check:
        px, ptok, pexp, pw = ext.pack_tokens_kernel(x, gates, idx, offsets.clone())
        assert torch.equal(px, x[ptok.long()]), "packed rows differ from a gather of the token rows"
        assert torch.equal(torch.bincount(pexp.long(), minlength=args.num_experts), counts.long())
        assert (pexp.long().diff() >= 0).all(), "rows are not grouped by expert"
        hit = idx.long()[ptok.long()] == pexp.long()[:, None]
        assert torch.equal(pw, gates[ptok.long()][hit]), "gate weights do not follow their rows"
        print("check passed")
    status = ext.read_status(True)
    assert status[0] == 0, status
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
