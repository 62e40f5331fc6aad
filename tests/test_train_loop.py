"""The training entrypoint end to end on CPU: every step is reported once, in order, under the
reference's metric names; a run resumes from its own checkpoint; two gloo ranks agree on the metrics."""
from pathlib import Path

import pytest

from tests.conftest import run_distributed
from tests.helpers import tiny_app_cfg


def _write_cfg(tmp, name, **over):
    from nanotitan_b200.sweep import dump_toml

    cfg = tiny_app_cfg(**over.pop("layout", {})).model_dump(mode="json")
    cfg.update(over)
    path = Path(tmp) / name
    path.write_text(dump_toml(cfg), encoding="utf-8")
    return path


def _run_main(path, logged, extra=()):
    from nanotitan_b200 import metrics, train

    plain = metrics.MetricsLogger.log

    def spy(self, step, metrics):
        logged.append((step, dict(metrics)))
        return plain(self, step, metrics)

    metrics.MetricsLogger.log = spy
    try:
        train.main([str(path), "--synthetic-data", "--log.level", "WARNING", *extra])
    finally:
        metrics.MetricsLogger.log = plain


def test_every_step_is_reported_once_in_order_with_the_reference_metric_names(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    path = _write_cfg(tmp_path, "run.toml", max_steps=4)
    logged = []
    _run_main(path, logged)
    assert [s for s, _ in logged] == [0, 1, 2, 3]
    names = set(logged[0][1])
    for want in ("train/ce_loss", "train/lb_loss", "train/total_loss", "time/step_time", "time/forward_time",
                 "train/tokens_per_step", "train/total_tokens_seen", "train/tokens_per_second", "moe/layer_00/route_frac_dist"):
        assert want in names, want
    seen = [m["train/total_tokens_seen"] for _, m in logged]
    per_step = logged[0][1]["train/tokens_per_step"]
    assert seen == [per_step * (i + 1) for i in range(4)]
    assert all(m["train/ce_loss"] == m["train/ce_loss"] for _, m in logged)  # no NaN


def test_a_run_resumes_from_its_own_checkpoint(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    ckpt = {"dir": str(tmp_path / "ckpt"), "every_steps": 2, "resume": False}
    first = _write_cfg(tmp_path, "a.toml", max_steps=2, checkpoint=ckpt)
    logged = []
    _run_main(first, logged)
    assert [s for s, _ in logged] == [0, 1]
    second = _write_cfg(tmp_path, "b.toml", max_steps=4, checkpoint=dict(ckpt, resume=True))
    more = []
    _run_main(second, more)
    assert [s for s, _ in more] == [2, 3]
    assert more[0][1]["train/total_tokens_seen"] == 3 * logged[0][1]["train/tokens_per_step"]

    # the command-line consolidation of that checkpoint loads into the reference-layout model
    import torch

    from nanotitan_b200.models import ModelShardSpec, NanoTitanModel
    from nanotitan_b200.utils import checkpoint

    out = tmp_path / "full.pt"
    assert checkpoint.main(["consolidate", str(tmp_path / "ckpt"), str(out)]) == 0
    state = torch.load(out)
    cfg = tiny_app_cfg().model
    model = NanoTitanModel(cfg, ModelShardSpec.full(cfg))
    assert list(state) == list(model.state_dict())
    model.load_state_dict(state)


def _two_rank_worker(rank, world, tmp):
    import os

    os.chdir(tmp)
    path = _write_cfg(tmp, f"r{rank}.toml", max_steps=3, layout=dict(dp=2, batch=2))
    logged = []
    _run_main(path, logged)
    if rank == 0:
        assert [s for s, _ in logged] == [0, 1, 2]
        # tokens per step count both data-parallel ranks
        assert logged[0][1]["train/tokens_per_step"] % 2 == 0 and logged[0][1]["train/tokens_per_step"] > 0


@pytest.mark.distributed
def test_two_data_parallel_ranks_train_through_the_entrypoint(tmp_path):
    run_distributed(_two_rank_worker, 2, str(tmp_path))


def test_a_packed_token_file_trains_through_the_native_loader(tmp_path, monkeypatch):
    """Without --synthetic-data the entrypoint reads `data.train_tokens_path`; with the extension built those
    batches come from the C++ window loader, across an epoch boundary (10 batches per epoch, 14 steps)."""
    from nanotitan_b200 import metrics, train
    from nanotitan_b200.data.dataset import write_synthetic_token_file
    from nanotitan_b200.ops.ext import have_ext

    if not have_ext():
        pytest.skip("the extension is not built")
    monkeypatch.chdir(tmp_path)
    tokens = write_synthetic_token_file(tmp_path / "train.bin", 61, 8 * 40 + 1, seed=1)  # 40 windows of 8 tokens
    data = {"num_workers": 1, "train_tokens_path": str(tokens), "val_tokens_path": str(tokens)}
    path = _write_cfg(tmp_path, "file.toml", max_steps=14, data=data)
    seen = []
    real = train.DataParallel.prepare_trainloader

    def spy(self, dataset):
        loader = real(self, dataset)
        seen.append(type(loader).__name__)
        return loader

    monkeypatch.setattr(train.DataParallel, "prepare_trainloader", spy)
    logged = []
    plain = metrics.MetricsLogger.log
    monkeypatch.setattr(metrics.MetricsLogger, "log",
                        lambda self, step, metrics: (logged.append(step), plain(self, step, metrics))[1])
    train.main([str(path), "--log.level", "WARNING"])
    assert seen == ["NativeTokenLoader"]
    assert logged == list(range(14))


def test_validation_loss_is_logged_on_the_configured_steps(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    cfg = tiny_app_cfg().model_dump(mode="json")
    cfg["max_steps"] = 5
    cfg["trainer"]["eval_every_step"] = 2
    from nanotitan_b200.sweep import dump_toml

    path = tmp_path / "eval.toml"
    path.write_text(dump_toml(cfg), encoding="utf-8")
    logged = []
    _run_main(path, logged, extra=("--eval-batches", "3"))
    val = [(s, m["val/ce_loss"]) for s, m in logged if "val/ce_loss" in m]
    assert [s for s, _ in val] == [1, 3]  # after the second and the fourth step
    assert all(0.0 < v < 10.0 for _, v in val)
    assert [s for s, m in logged if "train/ce_loss" in m] == [0, 1, 2, 3, 4]


def _pipeline_eval_worker(rank, world, tmp):
    import os

    os.chdir(tmp)
    cfg = tiny_app_cfg(pp=2, microbatches=2).model_dump(mode="json")
    cfg["max_steps"] = 2
    cfg["trainer"]["eval_every_step"] = 0  # after every step
    from nanotitan_b200.sweep import dump_toml

    path = Path(tmp) / f"pp{rank}.toml"
    path.write_text(dump_toml(cfg), encoding="utf-8")
    logged = []
    _run_main(path, logged, extra=("--eval-batches", "2"))
    if rank == 0:
        val = [(s, m["val/ce_loss"]) for s, m in logged if "val/ce_loss" in m]
        assert [s for s, _ in val] == [0, 1] and all(0.0 < v < 10.0 for _, v in val), val


@pytest.mark.distributed
def test_validation_runs_through_the_pipeline_stages(tmp_path):
    run_distributed(_pipeline_eval_worker, 2, str(tmp_path))


def _file_cfg(tmp, **over):
    """A config that trains from a packed token file (the same data whatever max_steps is)."""
    from nanotitan_b200.data.dataset import write_synthetic_token_file

    tokens = Path(tmp) / "train.bin"
    if not tokens.exists():
        write_synthetic_token_file(tokens, 61, 8 * 64 + 1, seed=2)
    cfg = tiny_app_cfg(**over.pop("layout", {})).model_dump(mode="json")
    cfg["data"] = {"num_workers": 1, "train_tokens_path": str(tokens), "val_tokens_path": str(tokens)}
    cfg.update(over)
    return cfg


def _train_from_file(tmp, name, cfg, extra=()):
    from nanotitan_b200 import train
    from nanotitan_b200.sweep import dump_toml

    path = Path(tmp) / f"{name}.toml"
    path.write_text(dump_toml(cfg), encoding="utf-8")
    train.main([str(path), "--log.level", "WARNING", *extra])


def _continue_on_two_stages(rank, world, tmp, full_file):
    import os

    os.chdir(tmp)
    cfg = _file_cfg(tmp, layout=dict(pp=2, microbatches=1), max_steps=4,
                    checkpoint={"dir": str(Path(tmp) / "ckpt_pp"), "every_steps": 0, "resume": False})
    _train_from_file(tmp, f"stage{rank}", cfg, extra=("--init-from", full_file))


@pytest.mark.distributed
def test_a_run_continues_on_another_layout_from_a_consolidated_checkpoint(tmp_path, monkeypatch):
    """Four steps on one process; against two steps on one process, consolidated with the optimizer state, then two
    more steps as two pipeline stages started with --init-from: same final weights."""
    import torch

    from nanotitan_b200.utils import checkpoint

    monkeypatch.chdir(tmp_path)

    def single(name, steps):
        cfg = _file_cfg(tmp_path, max_steps=steps, checkpoint={"dir": str(tmp_path / name), "every_steps": 0, "resume": False,
                                                               "portable_optimizer": True})
        _train_from_file(tmp_path, name, cfg)
        return checkpoint.consolidate(checkpoint.latest_checkpoint(tmp_path / name))

    straight = single("straight", 4)
    half = single("half", 2)
    assert any(not torch.equal(half[k], straight[k]) for k in straight), "two more steps must change the weights"
    full = tmp_path / "half_full.pt"
    assert checkpoint.main(["consolidate", str(tmp_path / "half"), str(full), "--with-optimizer"]) == 0
    run_distributed(_continue_on_two_stages, 2, str(tmp_path), str(full))
    found = checkpoint.latest_checkpoint(tmp_path / "ckpt_pp")
    assert found.name == "step_00000004"
    resumed = checkpoint.consolidate(found)
    assert list(resumed) == list(straight)
    for key in straight:
        torch.testing.assert_close(resumed[key], straight[key], rtol=1e-5, atol=1e-6, msg=lambda m, k=key: f"{k}: {m}")


def test_reporting_one_step_behind_still_reports_every_step_once(tmp_path, monkeypatch):
    """On GPUs the loop launches step i+1 before it collects the metrics of step i; forced on here, the same
    bookkeeping must log every step exactly once and in order, the last one after the loop, with the token
    counts of the step it belongs to."""
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("NT_RUN_AHEAD", "1")
    path = _write_cfg(tmp_path, "ahead.toml", max_steps=5,
                      checkpoint={"dir": str(tmp_path / "ckpt"), "every_steps": 2, "resume": False})
    logged = []
    _run_main(path, logged)
    train_steps = [(s, m) for s, m in logged if "train/ce_loss" in m]
    assert [s for s, _ in train_steps] == [0, 1, 2, 3, 4]
    per_step = train_steps[0][1]["train/tokens_per_step"]
    assert [m["train/total_tokens_seen"] for _, m in train_steps] == [per_step * (i + 1) for i in range(5)]

    monkeypatch.setenv("NT_RUN_AHEAD", "0")
    again = []
    _run_main(_write_cfg(tmp_path, "now.toml", max_steps=5), again)
    assert [m["train/ce_loss"] for _, m in again] == [m["train/ce_loss"] for _, m in train_steps], "same run, same losses"
