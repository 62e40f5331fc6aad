"""Host-side pieces of bench.py: the parallel layouts per config, one wording of `config` for both arms, and the
clock record parsed from nvidia-smi's CSV (against a stand-in `nvidia-smi` on PATH)."""
import importlib.util
import os
import stat
import sys
import time
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    module = importlib.util.module_from_spec(spec)
    sys.modules["bench_under_test"] = module
    spec.loader.exec_module(module)
    return module


def test_layouts(bench):
    assert bench._parallelism("dense", 8) == (8, 1, 1, "dp8")
    assert bench._parallelism("moe", 4) == (1, 1, 4, "ep4")
    assert bench._parallelism("moe3d", 8)[:3] == (1, 2, 4)
    with pytest.raises(SystemExit):
        bench._parallelism("moe3d", 4)
    for name, model in bench.MODELS.items():
        assert model["n_heads"] * model["d_head"] == model["d_model"] and model["dtype"] == "bfloat16", name
        assert bench.BATCH[name] % bench.MICROBATCHES[name] == 0


def test_config_block_matches_the_published_benchmark(bench):
    cfg = bench._config_dict("dense", bench.BATCH["dense"], 8, bench.MODELS["dense"]["max_seq_len"], "dp8")
    assert cfg["global_batch"] == 320 and cfg["seq_len"] == 768 and cfg["parallelism"] == "dp8"
    assert "16L d512" in cfg["model"] and "vocab50257" in cfg["model"]
    assert set(cfg) == {"model", "global_batch", "seq_len", "parallelism", "optimizer", "l2"}


def test_clock_record_from_nvidia_smi_csv(bench, tmp_path, monkeypatch):
    fake = tmp_path / "nvidia-smi"
    fake.write_text("""#!/bin/sh
echo "0, 345, 1965, 180.10, 0x0000000000000001, Not Active, Not Active, Not Active, Not Active"
echo "0, 1852, 1965, 736.24, 0x0000000000000004, Not Active, Not Active, Not Active, Active"
echo "0, 1905, 1965, 701.00, 0x0000000000000004, Not Active, Not Active, Not Active, Active"
echo "0, 1800, 1965, 690.00, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active"
echo "garbage line"
exec sleep 30
""")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", f"{tmp_path}{os.pathsep}{os.environ['PATH']}")
    sampler = bench.ClockSampler(0)
    sampler.start()
    time.sleep(0.5)
    record = sampler.stop()
    assert record["samples"] == 4 and record["sm_max_mhz"] == 1965.0 and record["power_w_max"] == 736.24
    assert record["sm_mhz"] == 1852.0  # median of the samples taken under load (> 300 W)
    assert record["reasons"] == ["sw_power_cap"]


def test_clock_record_without_nvidia_smi(bench, monkeypatch, tmp_path):
    monkeypatch.setenv("PATH", str(tmp_path))
    sampler = bench.ClockSampler(0)
    sampler.start()
    assert sampler.stop()["reasons"] == ["nvidia-smi unavailable"]
