"""Background checkpoint writing: same files as the blocking save, complete only when every rank's shard is there,
failures surface in the training thread, and the state that was captured is the state at the call."""
import threading
from pathlib import Path

import pytest
import torch

from tests.conftest import run_distributed
from tests.helpers import fake_dims, full_spec, random_batch, tiny_app_cfg


def _single(cfg):
    from nanotitan_b200.models.model import NanoTitanModel
    from nanotitan_b200.parallel import PipelineParallel
    from nanotitan_b200.parallel.reducer import ReducerV1
    from nanotitan_b200.utils import seed_everything

    seed_everything(4)
    model = NanoTitanModel(cfg.model, full_spec(cfg.model))
    reducers = {k: ReducerV1(v, 1, None, 1) for k, v in model.parameter_sync_groups().items()}
    dims = fake_dims(num_experts=4)
    return model, PipelineParallel(cfg, dims, reducers), torch.optim.AdamW(model.parameters(), lr=1e-2, weight_decay=0.1), dims


def test_the_snapshot_is_taken_at_the_call_not_when_the_thread_gets_to_it(tmp_path, monkeypatch):
    from nanotitan_b200.utils import checkpoint

    cfg = tiny_app_cfg()
    model, step, opt, dims = _single(cfg)
    step.train_step(model, random_batch(cfg, 0), opt)
    blocking = checkpoint.save_checkpoint(tmp_path / "blocking", 1, 32, model, opt, dims, cfg)

    gate = threading.Event()
    real_write = checkpoint._write_shard

    def slow_write(*args):
        gate.wait(30)  # the disk is slow: training goes on meanwhile
        real_write(*args)

    monkeypatch.setattr(checkpoint, "_write_shard", slow_write)
    saver = checkpoint.AsyncCheckpointer(timeout_s=30)
    background = saver.save(tmp_path / "background", 1, 32, model, opt, dims, cfg)
    assert saver.in_flight() and not checkpoint.is_complete(background)
    step.train_step(model, random_batch(cfg, 1), opt)  # changes weights and moments in place
    gate.set()
    saver.wait()
    assert checkpoint.is_complete(background) and checkpoint.latest_checkpoint(tmp_path / "background") == background
    a = torch.load(blocking / "rank_00000.pt", weights_only=False)
    b = torch.load(background / "rank_00000.pt", weights_only=False)
    for key in a["model"]:
        assert torch.equal(a["model"][key], b["model"][key]), key
    for i, st in a["optimizer"]["state"].items():
        assert torch.equal(st["exp_avg"], b["optimizer"]["state"][i]["exp_avg"])
    assert not torch.equal(b["model"]["blocks.1.attn.W_O"], model.state_dict()["blocks.1.attn.W_O"])


def test_a_failed_write_is_raised_in_the_training_thread(tmp_path):
    from nanotitan_b200.utils import checkpoint

    cfg = tiny_app_cfg()
    model, _, opt, dims = _single(cfg)
    (tmp_path / "occupied").write_text("a file where the checkpoint folder should go")
    saver = checkpoint.AsyncCheckpointer()
    saver.save(tmp_path / "occupied", 1, 0, model, opt, dims, cfg)
    with pytest.raises(RuntimeError, match="asynchronous checkpoint failed"):
        saver.wait()
    saver.wait()  # the error is reported once


def test_no_manifest_while_a_rank_is_missing(tmp_path):
    from nanotitan_b200.utils import checkpoint

    cfg = tiny_app_cfg()
    model, _, opt, _ = _single(cfg)
    dims = fake_dims(num_experts=4, world_size=2)  # rank 0 of two; rank 1 never writes
    saver = checkpoint.AsyncCheckpointer(timeout_s=0.5)
    step_dir = saver.save(tmp_path, 7, 0, model, opt, dims, cfg)
    with pytest.raises(RuntimeError, match="not every rank"):
        saver.wait()
    assert (step_dir / "rank_00000.pt").exists() and not checkpoint.is_complete(step_dir)
    assert checkpoint.latest_checkpoint(tmp_path) is None


def _entrypoint_worker(rank, world, tmp):
    import os

    from nanotitan_b200 import train
    from nanotitan_b200.sweep import dump_toml
    from nanotitan_b200.utils.checkpoint import is_complete, latest_checkpoint

    os.chdir(tmp)
    cfg = tiny_app_cfg(dp=2, batch=2).model_dump(mode="json")
    cfg.update(max_steps=5, checkpoint={"dir": str(Path(tmp) / "ckpt"), "every_steps": 2, "resume": False, "async_save": True})
    path = Path(tmp) / f"r{rank}.toml"
    path.write_text(dump_toml(cfg), encoding="utf-8")
    train.main([str(path), "--synthetic-data", "--log.level", "WARNING"])
    # main() returns after its barrier: every save of the run is complete on every rank's view of the folder
    assert latest_checkpoint(Path(tmp) / "ckpt").name == "step_00000005"
    assert all(is_complete(Path(tmp) / "ckpt" / f"step_{n:08d}") for n in (2, 4, 5))


@pytest.mark.distributed
def test_two_ranks_train_with_background_saves(tmp_path):
    run_distributed(_entrypoint_worker, 2, str(tmp_path))
