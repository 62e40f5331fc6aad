"""Per-kernel microbenchmarks on one GPU: CUDA-event timed, warm-up first, inputs larger than L2
or an explicit L2 flush between iterations.  Prints one JSON line per case with the achieved
TFLOP/s or GB/s and its fraction of the measured peaks in MEASURED_PEAKS.json (fallback
1590 TFLOP/s / 6650 GB/s when that file is absent).

    python benchmarks/bench_kernels.py [--only gemm,attn,moe,norm,ce,adamw] [--iters 20]
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from nanotitan_b200.ops import native  # noqa: E402
from nanotitan_b200.ops.ext import get_ext  # noqa: E402


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        p = json.loads(path.read_text())
        return p["bf16_tflops"], p["hbm_gbs"], "measured"
    return 1590.0, 6650.0, "fallback"


_FLUSH = None


def timed(fn, iters=20, warmup=3, flush=True):
    global _FLUSH
    if flush and _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush:
            _FLUSH.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters


def report(name, ms, flops=None, nbytes=None, **extra):
    tf, gbs, kind = peaks()
    rec = {"case": name, "ms": round(ms, 4)}
    if flops:
        rec["tflops"] = round(flops / ms / 1e9, 1)
        rec["frac_of_%s_gemm_peak" % kind] = round(flops / ms / 1e9 / tf, 3)
    if nbytes:
        rec["gbs"] = round(nbytes / ms / 1e6, 1)
        rec["frac_of_%s_hbm" % kind] = round(nbytes / ms / 1e6 / gbs, 3)
    rec.update(extra)
    print(json.dumps(rec), flush=True)


def rnd(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


def bench_gemm(iters):
    T = 30720
    cases = [("qkv/o proj fwd", T, 512, 512, False, True), ("ffn down fwd", T, 512, 2048, False, True),
             ("ffn up fwd", T, 2048, 512, False, True), ("wgrad 512x2048", 512, 2048, T, True, True),
             ("wgrad 2048x512", 2048, 512, T, True, True), ("wgrad 512x1536", 512, 1536, T, True, True),
             ("wgrad unembed", 512, 50257, T, True, True),
             ("dgrad unembed", T, 512, 50257, False, True), ("unembed fwd", T, 50257, 512, False, False),
             ("square 8192", 8192, 8192, 8192, False, False)]
    for name, M, N, K, a_mn, b_mn in cases:
        pad = lambda n: (n + 63) // 64 * 64  # noqa: E731  (TMA wants 16-byte row strides)
        a = rnd(K, pad(M))[:, :M] if a_mn else rnd(M, pad(K))[:, :K]
        b = rnd(K, pad(N), scale=0.05)[:, :N] if b_mn else rnd(N, pad(K), scale=0.05)[:, :K]
        ld = pad(N)
        c = torch.empty(M, ld, device="cuda", dtype=torch.bfloat16)[:, :N]
        if a_mn:  # weight gradient: the training path (reduction cut over the SMs, fp32 partials folded in order)
            ms = timed(lambda: native.wgrad(a, b, [c]), iters)
        else:
            ms = timed(lambda: native.gemm_tc(a, a_mn, [b], b_mn, [c]), iters)
        report(f"gemm_tc {name} M{M} N{N} K{K}", ms, flops=2.0 * M * N * K)
        at, bt = (a.t() if a_mn else a), (b if b_mn else b.t())
        ms = timed(lambda: torch.matmul(at, bt), iters)
        report(f"cublas  {name} M{M} N{N} K{K}", ms, flops=2.0 * M * N * K)
    # fused SwiGLU expert FFN (one expert = the dense config), forward and backward
    x = rnd(T, 512).requires_grad_()
    wg, wv = (rnd(1, 512, 2048, scale=0.03).requires_grad_() for _ in range(2))
    wo = rnd(1, 2048, 512, scale=0.03).requires_grad_()
    off = torch.tensor([0, T], device="cuda", dtype=torch.int32)
    ms = timed(lambda: native.swiglu_experts(x, wg, wv, wo, off), iters)
    report("swiglu experts fwd T30720 d512 f2048", ms, flops=6.0 * T * 512 * 2048)
    y = native.swiglu_experts(x, wg, wv, wo, off)
    g = torch.randn_like(y)
    ms = timed(lambda: torch.autograd.grad(y, (x, wg, wv, wo), g, retain_graph=True), iters)
    report("swiglu experts bwd T30720 d512 f2048", ms, flops=12.0 * T * 512 * 2048)


ATTN_SHAPES = [(40, 768, 16, 32), (4, 1024, 16, 64), (16, 2048, 8, 64)]


def bench_attn(iters):
    ext = get_ext()
    if not hasattr(ext, "flash_fwd"):
        return
    for B, S, H, Dh in ATTN_SHAPES:
        q, k, v = (rnd(B, S, H, Dh) for _ in range(3))
        scale = Dh**-0.5
        flops = 2.0 * B * H * S * S * Dh  # causal: half of 4*S*S*Dh
        ms = timed(lambda: ext.flash_fwd(q, k, v, scale), iters)
        report(f"flash fwd B{B} S{S} H{H} Dh{Dh}", ms, flops=flops)
        out, lse = ext.flash_fwd(q, k, v, scale)
        g = torch.randn_like(out)
        ms = timed(lambda: ext.flash_bwd(g, q, k, v, out, lse, scale), iters)
        report(f"flash bwd B{B} S{S} H{H} Dh{Dh}", ms, flops=2.5 * flops)
        qt, kt, vt = (t.transpose(1, 2) for t in (q, k, v))
        ms = timed(lambda: torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, is_causal=True), iters)
        report(f"sdpa  fwd B{B} S{S} H{H} Dh{Dh}", ms, flops=flops)


def bench_moe(iters):
    ext = get_ext()
    for T, d, E, k in ((12288, 512, 8, 2), (32768, 512, 64, 8), (32768, 2048, 64, 8)):
        x = rnd(T, d)
        w = torch.randn(E, d, device="cuda") * 0.1
        ms = timed(lambda: ext.router_topk(x, w, k), iters)
        report(f"router_topk T{T} d{d} E{E} k{k}", ms, nbytes=T * d * 2 + T * E * 4)
        if os.environ.get("NT_ROUTER_GEMM") == "1":  # the other router path, only when asked for
            ms = timed(lambda: ext.router_from_logits(native.router_logits_tc(x, w), k), iters)
            report(f"router via GEMM logits T{T} d{d} E{E} k{k}", ms, nbytes=T * d * 2 * 2 + T * E * 4 * 3)
        gates, idx, probs, counts = ext.router_topk(x, w, k)[:4]
        ms = timed(lambda: ext.assign_slots(idx, counts), iters)
        report(f"assign_slots T{T} E{E} k{k}", ms, nbytes=T * k * 8)
        offsets, slot_of = ext.assign_slots(idx, counts)
        ms = timed(lambda: ext.pack_fwd(x, gates, idx, slot_of), iters)
        report(f"pack_fwd T{T} d{d} k{k}", ms, nbytes=T * d * 2 * (1 + k))
        px, ptok, pexp, pgate = ext.pack_fwd(x, gates, idx, slot_of)
        ms = timed(lambda: ext.combine_fwd(px, pgate, slot_of.view(-1), None, T, x, False), iters)
        report(f"combine_fwd T{T} d{d} k{k}", ms, nbytes=T * d * 2 * (2 + k))
        ms = timed(lambda: ext.combine_bwd(px, ptok, pgate, x), iters)
        report(f"combine_bwd T{T} d{d} k{k}", ms, nbytes=T * d * 2 * 3 * k)
        ms = timed(lambda: ext.pack_bwd(px, slot_of.view(-1), None, T), iters)
        report(f"pack_bwd T{T} d{d} k{k}", ms, nbytes=T * d * 2 * (1 + k))


def bench_norm(iters):
    ext = get_ext()
    x = rnd(30720, 512)
    g, b = torch.ones(512, device="cuda").bfloat16(), torch.zeros(512, device="cuda").bfloat16()
    ms = timed(lambda: ext.layer_norm_fwd(x, g, b, 1e-8), iters)
    report("layer_norm fwd 30720x512", ms, nbytes=x.numel() * 4)
    y, mean, rstd = ext.layer_norm_fwd(x, g, b, 1e-8)
    ms = timed(lambda: ext.layer_norm_bwd(y, x, g, mean, rstd), iters)
    report("layer_norm bwd 30720x512", ms, nbytes=x.numel() * 6)


def bench_ce(iters):
    ext = get_ext()
    rows, V, ld = 8192, 50257, 50304
    logits = rnd(rows, ld)
    tgt = torch.randint(0, V, (rows,), device="cuda")
    ms = timed(lambda: ext.cross_entropy_fwd_bwd(logits, tgt, V, 1.0 / rows, True), iters, flush=False)
    report(f"cross_entropy fwd+bwd {rows}x{V}", ms, nbytes=rows * ld * 2 * 3)


def bench_adamw(iters):
    ext = get_ext()
    n = 118_600_000 // 8 * 8
    p = rnd(n)
    g = rnd(n)
    master, m, v = p.float(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    ms = timed(lambda: ext.adamw_step(p, g, master, m, v, 1, 1e-3, 0.9, 0.999, 1e-8, 0.1, 1.0, False), iters, flush=False)
    report(f"adamw {n / 1e6:.1f}M params", ms, nbytes=n * (2 + 2 + 12 + 12))


def bench_single(iters, shape, b_mn):
    """One dense tcgen05 GEMM (the case to put under ncu): A [M,K] K-major, B [N,K] or [K,N]."""
    M, N, K = shape
    a = rnd(M, K)
    b = rnd(K, N, scale=0.05) if b_mn else rnd(N, K, scale=0.05)
    c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    ms = timed(lambda: native.gemm_tc(a, False, [b], b_mn, [c]), iters)
    report(f"gemm_tc single M{M} N{N} K{K} b_mn={int(b_mn)}", ms, flops=2.0 * M * N * K)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="30720,512,2048", help="M,N,K of --only single")
    ap.add_argument("--b-mn", type=int, default=1, help="--only single: 1 = B stored [K,N]")
    ap.add_argument("--attn-shape", default="", help="B,S,H,Dh: run --only attn on this one shape")
    ap.add_argument("--only", default="gemm,attn,moe,norm,ce,adamw")
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    table = {"gemm": bench_gemm, "attn": bench_attn, "moe": bench_moe, "norm": bench_norm, "ce": bench_ce, "adamw": bench_adamw}
    if args.attn_shape:
        ATTN_SHAPES[:] = [tuple(int(v) for v in args.attn_shape.split(","))]
    for key in args.only.split(","):
        if key.strip() == "single":
            bench_single(args.iters, tuple(int(v) for v in args.shape.split(",")), bool(args.b_mn))
        else:
            table[key.strip()](args.iters)


if __name__ == "__main__":
    main()
