"""Small command-line tools and sinks that need no GPU: dataset preparation, the token file format, the metrics
sink and packed reduction, the generic Nsight Compute launcher."""
import numpy as np
import pytest
import torch

from tests.conftest import run_distributed


def test_token_file_round_trip_and_range_check(tmp_path):
    from nanotitan_b200.data.dataset import PackedTokenDataset
    from nanotitan_b200.data.prepare_dataset import write_token_file

    ids = list(range(0, 65536, 257)) + [65535, 0, 7]
    write_token_file(ids, tmp_path / "deep" / "tokens.bin")
    raw = np.fromfile(tmp_path / "deep" / "tokens.bin", dtype="<u2")
    assert raw.tolist() == ids
    ds = PackedTokenDataset(tmp_path / "deep" / "tokens.bin", seq_len=4)
    x, y = ds[1]
    assert x.tolist() == ids[4:8] and y.tolist() == ids[5:9] and x.dtype == torch.int64
    assert len(ds) == (len(ids) - 1) // 4
    with pytest.raises(ValueError, match="uint16"):
        write_token_file([1, 70000], tmp_path / "bad.bin")


def test_prepare_dataset_synthetic_writes_both_splits(tmp_path, monkeypatch, capsys):
    from nanotitan_b200.data import prepare_dataset

    monkeypatch.chdir(tmp_path)
    monkeypatch.setattr("sys.argv", ["prepare_dataset", "--synthetic", "1000", "--vocab-size", "300", "--seed", "5"])
    prepare_dataset.main()
    train = np.fromfile(tmp_path / "data/preprocessed/tinystories_train.bin", dtype="<u2")
    val = np.fromfile(tmp_path / "data/preprocessed/tinystories_val.bin", dtype="<u2")
    assert train.size == val.size == 1000 and train.max() < 300 and not np.array_equal(train, val)
    assert "synthetic tokens" in capsys.readouterr().out


def test_metrics_sink_writes_scalars_histograms_and_config(tmp_path):
    from tensorboard.backend.event_processing.event_accumulator import EventAccumulator

    from nanotitan_b200.metrics import MetricsLogger

    sink = MetricsLogger("run", log_root=str(tmp_path))
    sink.log_config({"lr": 1e-3})
    for step in range(3):
        sink.log(step, {"train/ce_loss": 4.0 - step, "moe/layer_00/route_frac_dist": torch.tensor([0.25, 0.75])})
    sink.close()
    events = EventAccumulator(str(tmp_path / "run"), size_guidance={"histograms": 0})
    events.Reload()
    assert [e.value for e in events.Scalars("train/ce_loss")] == [4.0, 3.0, 2.0]
    assert len(events.Histograms("moe/layer_00/route_frac_dist")) == 3
    assert "config/text_summary" in events.Tags()["tensors"]
    import json

    lines = [json.loads(line) for line in (tmp_path / "run" / "metrics.jsonl").read_text().splitlines()]
    assert lines == [{"step": i, "train/ce_loss": 4.0 - i} for i in range(3)]


def _reduce_worker(rank, world):
    from nanotitan_b200.metrics import HistogramMetric, ScalarMetric, reduce_metrics

    calls = []
    import torch.distributed as dist

    real = dist.all_reduce

    def counting(*args, **kwargs):
        calls.append(kwargs.get("op", args[1] if len(args) > 1 else None))
        return real(*args, **kwargs)

    dist.all_reduce = counting
    try:
        out = reduce_metrics({
            "loss": ScalarMetric(1.0 + rank, reduce="mean"),
            "tokens": ScalarMetric(10.0, reduce="sum"),
            "time": ScalarMetric(0.5 * (rank + 1), reduce="max"),
            "local": ScalarMetric(float(rank), reduce="none"),
            "hist": HistogramMetric(torch.tensor([1.0, float(rank)]), reduce="sum"),
            "time2": ScalarMetric(3.0 - rank, reduce="max"),
        }, torch.device("cpu"))
    finally:
        dist.all_reduce = real
    assert len(calls) == 2, "one collective per reduce kind, however many metrics"
    assert out["loss"] == 1.5 and out["tokens"] == 20.0 and out["time"] == 1.0 and out["time2"] == 3.0 and out["local"] == float(rank)
    assert out["hist"].tolist() == [2.0, 1.0] and list(out) == ["loss", "tokens", "time", "local", "hist", "time2"]


@pytest.mark.distributed
def test_metrics_are_reduced_in_two_collectives():
    run_distributed(_reduce_worker, 2)


def test_ncu_launcher_builds_a_capture_that_leaves_the_clocks_alone(capsys):
    from nanotitan_b200 import ncu_kernel

    rc = ncu_kernel.main(["--kernel", "gemm_tc_kernel", "--skip", "3", "--count", "2", "--section", "SpeedOfLight",
                          "--section", "MemoryWorkloadAnalysis", "--out", "profiles/raw/x", "--ncu", "ncu", "--dry-run", "--",
                          "python", "benchmarks/bench_kernels.py", "--only", "single"])
    line = capsys.readouterr().out.strip()
    assert rc == 0 and line.startswith("ncu --clock-control none")
    assert "--section SpeedOfLight --section MemoryWorkloadAnalysis" in line and "--set" not in line
    assert "--kernel-name regex:gemm_tc_kernel --launch-skip 3 --launch-count 2" in line
    assert line.endswith("python benchmarks/bench_kernels.py --only single")
    with pytest.raises(SystemExit):
        ncu_kernel.main(["--kernel", "x"])  # no command to profile
