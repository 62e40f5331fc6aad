"""Command lines of the stand-alone benchmarks and of the ncu launcher (what runs without a GPU): the options of
the reference's scripts of the same names are accepted, byte counts are what the kernels must move, and the
capture command leaves the clocks alone."""
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def test_pack_benchmark_arguments_and_bytes():
    from benchmarks import bench_pack_tokens as b

    args = b.parse_args([])
    assert (args.tokens, args.hidden_dim, args.top_k, args.num_experts, args.dtype, args.warmup, args.iters) == \
        (32768, 1024, 2, 16, "fp16", 20, 100)
    sizes = b.stage_bytes(tokens=1000, hidden=64, k=2, experts=8, elem=2)
    assert sizes["pack"] == 1000 * 64 * 2 * 3 + 1000 * 2 * 16
    assert sizes["count"] == 1000 * 2 * 4 + 32


def test_combine_benchmark_arguments_and_bytes():
    from benchmarks import bench_combine as b

    args = b.parse_args(["--backend", "cuda", "--dtype", "bf16", "--tokens", "64"])
    assert (args.backend, args.dtype, args.tokens, args.hidden_dim, args.top_k) == ("cuda", "bf16", 64, 1024, 2)
    assert b.combine_bytes(tokens=10, hidden=8, k=2, elem=2) == 10 * 2 * 8 * 2 + 10 * 8 * 4 + 10 * 2 * 8


def test_combine_oracle_is_the_weighted_sum_per_token():
    import torch

    from benchmarks.bench_combine import torch_combine

    y = torch.tensor([[1.0, 2.0], [10.0, 20.0], [100.0, 200.0]])
    out = torch_combine(y, torch.tensor([1, 0, 1]), torch.tensor([0.5, 1.0, 2.0]), tokens=2)
    assert out.tolist() == [[10.0, 20.0], [200.5, 401.0]]


def test_ncu_launcher_command(capsys):
    from scripts import profile_pack_tokens_ncu as p

    rc = p.main(["--dry-run", "--tokens", "4096", "--dtype", "bf16", "--warmup", "3", "--profile-launches", "2", "--ncu", "ncu"])
    assert rc == 0
    line = capsys.readouterr().out.strip()
    assert line.startswith("ncu --clock-control none ")
    assert "--launch-skip 3 --launch-count 2" in line and "--set detailed" in line
    assert "regex:.*pack_fwd_kernel.*" in line
    assert "profiles/raw/pack_tokens/pack_T4096_d1024_k2_E16_bf16" in line
    assert "bench_pack_tokens.py" in line and "--tokens 4096" in line and "--warmup 3" in line


def test_moe_benchmark_accepts_its_own_and_the_reference_spellings():
    from benchmarks import bench_moe as b

    args = b.parse_args([])
    assert (args.tokens, args.hidden, args.ffn, args.experts, args.top_k, args.backend, args.dtype) == \
        (32768, 512, 2048, 64, 8, "cuda", "bfloat16")
    args = b.parse_args(["--batch", "8", "--seq-len", "1024", "--d-model", "1024", "--ffn-in", "4096", "--num-experts", "16",
                         "--top-k", "2", "--backend", "torch", "--dtype", "float16", "--device", "0"])
    assert (args.tokens, args.hidden, args.ffn, args.experts, args.top_k, args.backend, args.dtype) == \
        (8192, 1024, 4096, 16, 2, "torch", "float16")
