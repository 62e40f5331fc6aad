"""MoE layer microbenchmark: forward + backward milliseconds of one MoE layer and of its stages
(router, pack, grouped SwiGLU GEMMs, combine), single GPU or expert-parallel.

    python benchmarks/bench_moe.py [--tokens 32768] [--hidden 512] [--ffn 2048] [--experts 64] [--top-k 8]
    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/bench_moe.py --ep 2 [--exchange p2p|nccl]

This is the "dispatch / combine + grouped-GEMM" benchmark: uniform ~N(0,1) activations, router
logits ~N(0,1), expert weights ~N(0, 0.02), CUDA-event timed (max over ranks), with an L2 flush
between iterations.  The reference's counterpart (benchmarks/bench_moe.py) no longer runs against its
own model class.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from nanotitan_b200.config import ModelConfig  # noqa: E402
from nanotitan_b200.models.feed_fwd import MoE  # noqa: E402
from nanotitan_b200.models.utils import ModelShardSpec  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--hidden", type=int, default=512)
    ap.add_argument("--ffn", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--ep", type=int, default=1)
    ap.add_argument("--exchange", choices=["p2p", "nccl"], default="p2p")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    if args.exchange == "nccl":
        os.environ["NT_FUSED_EP"] = "0"
    rank, world = 0, 1
    if args.ep > 1:
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        rank, world = dist.get_rank(), dist.get_world_size()
        assert world == args.ep
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = ModelConfig(vocab_size=8, d_model=args.hidden, d_head=32, n_heads=1, n_layers=1, max_seq_len=8, ffn_in=args.ffn,
                      num_experts=args.experts, top_k=args.top_k, router_alpha=0.01, moe_backend="cuda", dtype="bfloat16")
    per = args.experts // world
    spec = ModelShardSpec(0, 1, False, False, False, per, rank * per, (rank + 1) * per, ep_size=world,
                          ep_group=dist.group.WORLD if world > 1 else None)
    torch.manual_seed(0)
    moe = MoE(cfg, spec).to(dev)
    with torch.no_grad():
        for p in moe.experts.parameters():
            p.normal_(0, 0.02)
        moe.router.weight.normal_(0, 1.0 / args.hidden**0.5)
        if world > 1:
            dist.broadcast(moe.router.weight, src=0)
    torch.manual_seed(1 + rank)
    x = torch.randn(1, args.tokens, args.hidden, device=dev).bfloat16().requires_grad_()
    g = torch.randn_like(x)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step():
        out, _ = moe(x)
        out.backward(g)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(args.iters):
        flush.zero_()
        if world > 1:
            dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    ms = torch.tensor([total / args.iters], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        flops = 3 * 3 * 2.0 * args.tokens * args.top_k * args.hidden * args.ffn  # 3 GEMMs, fwd + 2x bwd
        print(json.dumps({"case": f"moe layer fwd+bwd T{args.tokens} d{args.hidden} f{args.ffn} E{args.experts} k{args.top_k} ep{world} {args.exchange}",
                          "ms": round(ms.item(), 3), "expert_gemm_tflops_per_gpu": round(flops / ms.item() / 1e9, 1)}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
