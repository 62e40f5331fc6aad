"""MoE layer microbenchmark: forward + backward milliseconds of one MoE layer and of its stages
(router, pack, grouped SwiGLU GEMMs, combine), single GPU or expert-parallel.

    python benchmarks/bench_moe.py [--tokens 32768] [--hidden 512] [--ffn 2048] [--experts 64] [--top-k 8]
    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/bench_moe.py --ep 2 [--exchange p2p|nccl]

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/bench_moe.py --ep 2 --impl reference

This is the "dispatch / combine + grouped-GEMM" benchmark: uniform ~N(0,1) activations, router
logits ~N(0,1), expert weights ~N(0, 0.02), CUDA-event timed (max over ranks), with an L2 flush
between iterations.

`--impl reference` times the same layer built from the reference's own pieces, installed under
baseline/_ref: its extension's kernels through its autograd wrappers (`pack_tokens_fn`,
`grouped_gemm_fn` x3 with the SwiGLU as torch ops, `combine_tokens_fn`, src/model/moe_ops.py:10-125,
in the order of src/model/cuda_backend.py:24-75) and, for expert parallelism, its autograd
`all_to_all_single` (src/model/moe_ops.py:128-160) with host-side split sizes.  The reference has no
expert-parallel path on these kernels (its CUDA backend is single-rank and its torch backend builds
the regrouping permutation one row at a time in Python), so the regrouping between the source-major
layout the collective delivers and the expert-major layout the grouped GEMM wants is done here with
a handful of vectorised torch ops: the reference arm is charged for its kernels and for NCCL, not
for that loop.  Nothing of `nanotitan_b200` is imported on that path.  The reference's own
benchmarks/bench_moe.py no longer runs against its model class.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def reference_layer(args, rank, world, dev):
    """-> (step function, parameters) of the layer assembled from the reference's kernels."""
    sys.path.insert(0, str(ROOT / "baseline"))
    import ref_harness

    why = ref_harness.available()
    if why is not None:
        raise SystemExit(json.dumps({"impl": "reference", "unavailable": why}))
    ref_harness._alias_src()
    from src.model import moe_ops
    from src.model.cuda_extension import get_cuda_extension

    ext = get_cuda_extension()
    E, k, d, f = args.experts, args.top_k, args.hidden, args.ffn
    E_loc = E // world
    torch.manual_seed(0)
    router = torch.nn.Parameter(torch.randn(E, d, device=dev) / d**0.5)
    if world > 1:
        dist.broadcast(router.data, src=0)
    torch.manual_seed(10 + rank)
    w_gate, w_val, w_out = (torch.nn.Parameter((torch.randn(*shape, device=dev) * 0.02).to(getattr(torch, args.dtype)))
                            for shape in ((E_loc, d, f), (E_loc, d, f), (E_loc, f, d)))
    params = [router, w_gate, w_val, w_out]

    def experts(rows, offsets):
        gate = moe_ops.grouped_gemm_fn(rows, w_gate, offsets)
        value = moe_ops.grouped_gemm_fn(rows, w_val, offsets)
        return moe_ops.grouped_gemm_fn(torch.nn.functional.silu(gate) * value, w_out, offsets)

    def step(x, g):
        flat = x.reshape(-1, d)
        tokens = flat.shape[0]
        probs = torch.nn.functional.linear(flat.float(), router).softmax(dim=-1)
        top_w, top_e = torch.topk(probs, k=k, dim=-1)
        gates = top_w / top_w.sum(dim=-1, keepdim=True)
        top_e = top_e.to(torch.int32)
        counts = ext.count_expert_kernel(top_e, torch.ones(tokens, device=dev, dtype=torch.int32), E, k)
        offsets = torch.zeros(E + 1, device=dev, dtype=torch.int32)
        offsets[1:] = torch.cumsum(counts, dim=0)
        packed, token_id, _, packed_w = moe_ops.pack_tokens_fn(flat, gates, top_e, offsets.clone())
        if world == 1:
            out_rows = experts(packed, offsets)
        else:
            send = counts.view(world, E_loc).to(torch.int64)
            recv = torch.empty_like(send)
            dist.all_to_all_single(recv, send, [1] * world, [1] * world)
            send_splits, recv_splits = send.sum(dim=1).tolist(), recv.sum(dim=1).tolist()
            got = moe_ops.torch_backend_all_to_all(packed, send_splits, recv_splits, dist.group.WORLD)
            # source-major -> expert-major: the row at (source s, local expert l, i) goes to expert l's segment
            src_start = torch.cumsum(recv.reshape(-1), 0) - recv.reshape(-1)          # [world * E_loc], source-major
            seg = torch.repeat_interleave(torch.arange(world * E_loc, device=dev), recv.reshape(-1))
            within = torch.arange(got.shape[0], device=dev) - src_start[seg]
            by_expert = recv.t().contiguous().reshape(-1)                               # [E_loc * world], expert-major
            dst_start = (torch.cumsum(by_expert, 0) - by_expert).view(E_loc, world).t().reshape(-1)
            dest = dst_start[seg] + within
            rows = torch.empty_like(got).index_copy(0, dest, got)
            local_offsets = torch.zeros(E_loc + 1, device=dev, dtype=torch.int32)
            local_offsets[1:] = torch.cumsum(recv.sum(dim=0), 0)
            out_local = experts(rows, local_offsets)
            out_rows = moe_ops.torch_backend_all_to_all(out_local[dest], recv_splits, send_splits, dist.group.WORLD)
        pool = moe_ops.combine_tokens_fn(out_rows, token_id, packed_w, tokens, d).to(packed.dtype)
        pool.reshape(x.shape).backward(g)

    return step, params


def parse_args(argv=None):
    """This benchmark's options, plus the spellings of the reference's benchmarks/bench_moe.py:51-61
    (`--batch` x `--seq-len` tokens, `--d-model`, `--ffn-in`, `--num-experts`, `--backend`, `--dtype`, `--device`)."""
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--batch", type=int, default=0, help="with --seq-len: tokens = batch x seq-len")
    ap.add_argument("--seq-len", type=int, default=0)
    ap.add_argument("--hidden", "--d-model", dest="hidden", type=int, default=512)
    ap.add_argument("--ffn", "--ffn-in", dest="ffn", type=int, default=2048)
    ap.add_argument("--experts", "--num-experts", dest="experts", type=int, default=64)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--ep", type=int, default=1)
    ap.add_argument("--exchange", choices=["p2p", "nccl"], default="p2p")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--backend", choices=["cuda", "torch"], default="cuda",
                    help="ours: the sm_100a kernels, or the portable torch modules (single rank)")
    ap.add_argument("--dtype", choices=["float16", "bfloat16"], default="bfloat16")
    ap.add_argument("--device", type=int, default=None, help="single-rank runs: CUDA device index")
    args = ap.parse_args(argv)
    if args.batch or args.seq_len:
        if not (args.batch and args.seq_len):
            ap.error("--batch and --seq-len go together")
        args.tokens = args.batch * args.seq_len
    if args.experts % args.ep:
        ap.error("--experts must be a multiple of --ep")
    if args.backend == "torch" and args.ep > 1 and args.impl == "ours":
        ap.error("--backend torch is a single-rank comparison")
    return args


def main(argv=None):
    args = parse_args(argv)
    if args.device is not None and args.ep == 1:
        torch.cuda.set_device(args.device)
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
    torch.manual_seed(1 + rank)
    x = torch.randn(1, args.tokens, args.hidden, device=dev).to(getattr(torch, args.dtype)).requires_grad_()
    g = torch.randn_like(x)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    if args.impl == "reference":
        ref_step, params = reference_layer(args, rank, world, dev)

        def step():
            x.grad = None
            for p in params:
                p.grad = None
            ref_step(x, g)

        label = "reference kernels" + (" + NCCL all_to_all" if world > 1 else "")
        report(args, time_steps(step, args.iters, flush, world, dev), rank, world, label)
        return
    from nanotitan_b200.config import ModelConfig
    from nanotitan_b200.models.feed_fwd import MoE
    from nanotitan_b200.models.utils import ModelShardSpec

    cfg = ModelConfig(vocab_size=8, d_model=args.hidden, d_head=32, n_heads=1, n_layers=1, max_seq_len=8, ffn_in=args.ffn,
                      num_experts=args.experts, top_k=args.top_k, router_alpha=0.01, moe_backend=args.backend, dtype=args.dtype)
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

    def step():
        x.grad = None
        for p in moe.parameters():
            p.grad = None
        out, _ = moe(x)
        out.backward(g)

    label = ("sm_100a kernels" if args.backend == "cuda" else "torch modules") + ((" + fused peer-store exchange" if args.exchange == "p2p" else " + NCCL all_to_all") if world > 1 else "")
    report(args, time_steps(step, args.iters, flush, world, dev), rank, world, label)


def time_steps(step, iters, flush, world, dev) -> float:
    """Mean CUDA-event milliseconds of `step` over `iters` runs after 3 warm-up runs, L2 flushed before
    each, maximum over the ranks."""
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        if world > 1:
            dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    ms = torch.tensor([total / iters], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms.item()


def report(args, ms, rank, world, label) -> None:
    if rank == 0:
        flops = 3 * 3 * 2.0 * args.tokens * args.top_k * args.hidden * args.ffn  # 3 GEMMs, fwd + 2x bwd
        print(json.dumps({"case": f"moe layer fwd+bwd T{args.tokens} d{args.hidden} f{args.ffn} E{args.experts} k{args.top_k} ep{world}",
                          "impl": label, "ms": round(ms, 3), "expert_gemm_tflops_per_gpu": round(flops / ms / 1e9, 1)}), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
