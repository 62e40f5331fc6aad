"""The fused collective kernels in isolation, against their NVLink roofline and against NCCL.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29531 benchmarks/bench_collectives.py [--iters 20] [--json out.json]

One rank per GPU.  Every figure is CUDA-event device time of one launch, mean over `--iters`
launches after 3 warm-up launches, maximum over the ranks.  Inputs are larger than the L2 or the
256 MiB flush buffer is rewritten between launches.

Rows:
  * `bucket_allreduce` (csrc/kernels/allreduce_adamw.cu) on 25 MiB and 256 MiB bf16 gradient
    buckets, reduce-only and with the fused AdamW, on the multicast (`multimem`) path (with the 64
    CTAs training uses, and with 148) and on the peer-load path, next to `dist.all_reduce` (NCCL) on
    the same buffer.  NVLink bytes per GPU per
    direction: one bucket (the slice exchange out, the reduced / updated values in).
  * `ep_dispatch` and `ep_push_rows` (csrc/kernels/ep_exchange.cu) on the expert-parallel model
    config (12288 tokens x top-2, 8 experts, d 512) and on the microbenchmark shapes (32768 tokens
    x top-8 of 64 experts, d 512 and 2048), uniform random routing, next to
    `dist.all_to_all_single` (NCCL) moving the same rows with equal splits.  NVLink bytes per GPU
    per direction: rows x d x 2 x (N-1)/N.
`frac` = achieved GB/s per GPU per direction / 770 GB/s (the peer-copy bandwidth measured on this
machine class; 900 GB/s is the nominal figure).  The reference's counterpart is its raw NCCL
all-reduce loop (benchmarks/bench.cpp:21-103).
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

LINK_GBS = 770.0


def timed(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        total += start.elapsed_time(end)
    ms = torch.tensor([total / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms.item()


def row(name, shape, ms, link_bytes):
    gbs = link_bytes / (ms * 1e-3) / 1e9
    return {"kernel": name, "shape": shape, "ms": round(ms, 4), "nvlink_gb_per_gpu_per_dir": round(link_bytes / 1e9, 4),
            "gbs_per_gpu_per_dir": round(gbs, 1), "frac_of_770": round(gbs / LINK_GBS, 3), "frac_of_900": round(gbs / 900.0, 3)}


def bench_allreduce(world, rank, dev, iters, flush, out):
    from nanotitan_b200.ops.adamw import FusedAdamW
    from nanotitan_b200.parallel import fused_allreduce
    from nanotitan_b200.parallel.reducer import ReducerV1

    for mib in (25, 256):
        n = mib * (1 << 20) // 2
        for multimem, blocks in ((True, 64), (True, 148), (False, 64)):
            # 64 CTAs is what training uses (the kernel shares the GPU with the backward pass); 148 shows the
            # kernel alone on the machine
            os.environ["NT_MULTIMEM"] = "1" if multimem else "0"
            os.environ["NT_ALLREDUCE_BLOCKS"] = str(blocks)
            engine = fused_allreduce.make_engine(dist.group.WORLD, world, dev)
            for adam in (False, True):
                param = torch.nn.Parameter(torch.zeros(n, dtype=torch.bfloat16, device=dev))
                red = ReducerV1([param], world, dist.group.WORLD, bucket_size=mib + 1, engine=engine)
                bucket = red.buckets[0]
                bucket.buffer.normal_()
                if adam:
                    opt = FusedAdamW([param], lr=1e-4)
                    opt.bind_reducers({"all": red})

                def launch():
                    bucket.work = engine.launch(red, bucket)
                    engine.finish(red, bucket)

                ms = timed(launch, iters, flush)
                kind = ("multimem" if multimem and bucket._mc else "peer loads") + f", {blocks} CTAs" + (" + AdamW" if adam else "")
                out.append(row(f"bucket_allreduce ({kind})", f"{mib} MiB bf16, {world} ranks", ms, n * 2))
                red.remove_hooks()
                del red, param
            del engine
        buf = torch.randn(n, device=dev).bfloat16()
        ms = timed(lambda: dist.all_reduce(buf), iters, flush)
        out.append(row("NCCL all_reduce", f"{mib} MiB bf16, {world} ranks", ms, n * 2))
        del buf
        torch.cuda.empty_cache()


def bench_exchange(world, rank, dev, iters, flush, out):
    from nanotitan_b200.ops.ext import get_ext
    from nanotitan_b200.parallel import ep_fused

    ext = get_ext()
    shapes = [("model config: 12288 tokens top-2 of 8 experts, d 512", 12288, 2, 8, 512),
              ("microbench: 32768 tokens top-8 of 64 experts, d 512", 32768, 8, 64, 512),
              ("microbench: 32768 tokens top-8 of 64 experts, d 2048", 32768, 8, 64, 2048)]
    for label, tokens, k, experts, d in shapes:
        if experts % world:
            continue
        ex = ep_fused.FusedExchange(dist.group.WORLD, experts, dev)
        gen = torch.Generator(device=dev).manual_seed(7 + rank)
        x = torch.randn(tokens, d, device=dev, generator=gen).bfloat16()
        idx = torch.rand(tokens, experts, device=dev, generator=gen).topk(k, dim=1).indices.to(torch.int32).contiguous()
        gates = torch.full((tokens, k), 1.0 / k, device=dev)
        counts = torch.bincount(idx.reshape(-1).long(), minlength=experts).to(torch.int32)
        offsets, slot_of = ext.assign_slots(idx, counts)
        A = tokens * k
        cap = ex.capacity_rows(A)
        x_in = ex.acquire(cap, d, x.dtype)
        y_home = ex.acquire(A, d, x.dtype)
        link = A * d * 2 * (world - 1) / world
        state = {}

        def dispatch():
            state["out"] = ext.ep_dispatch(x, gates, idx, slot_of, counts, offsets, ex.cmat, ex.cmat_peers, x_in.peers, cap,
                                           ex.E_loc, ex.block_counter, ex.flags, ex.flag_peers, ex.rank, ex.ep, ex.epoch_counter,
                                           ex.wait_ms, ex.blocks)

        ms = timed(dispatch, iters, flush)
        out.append(row("ep_dispatch (count exchange + pack + push)", f"{label}, {world} ranks", ms, link))
        cmat = state["out"][0]
        expert_rows = x_in.view(cap, d)
        for direction, src, dst, dst_rows, name in ((1, expert_rows, y_home, A, "ep_push_rows (return)"),
                                                    (0, y_home.view(A, d), x_in, cap, "ep_push_rows (combine-backward)")):
            ms = timed(lambda: ex.push(src, cmat, direction, dst, dst_rows, entry_barrier=True), iters, flush)
            out.append(row(name, f"{label}, {world} ranks", ms, link))
        # NCCL moving the same number of rows with equal splits
        rows_each = A // world
        send = x.new_empty(rows_each * world, d).normal_()
        recv = torch.empty_like(send)
        ms = timed(lambda: dist.all_to_all_single(recv, send), iters, flush)
        out.append(row("NCCL all_to_all_single (rows only, equal splits)", f"{label}, {world} ranks", ms, rows_each * (world - 1) * d * 2))
        status = ext.read_status(True)
        assert status[0] == 0, status
        del ex, x_in, y_home, send, recv
        torch.cuda.empty_cache()


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", default="")
    ap.add_argument("--only", choices=["allreduce", "exchange", "all"], default="all")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    out: list[dict] = []
    if args.only in ("allreduce", "all"):
        bench_allreduce(world, rank, dev, args.iters, flush, out)
    if args.only in ("exchange", "all"):
        bench_exchange(world, rank, dev, args.iters, flush, out)
    if rank == 0:
        for r in out:
            print(f"{r['kernel']:<52} {r['shape']:<64} {r['ms']:9.4f} ms  {r['gbs_per_gpu_per_dir']:7.1f} GB/s/GPU/dir  "
                  f"{100 * r['frac_of_770']:5.1f} % of 770  {100 * r['frac_of_900']:5.1f} % of 900")
        if args.json:
            Path(args.json).write_text(json.dumps(out, indent=1))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
