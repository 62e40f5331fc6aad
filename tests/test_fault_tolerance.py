"""Failure detection, tested without faulting any GPU: failures are made on the host (a rank that
raises, a rank that never joins), liveness travels through heartbeat files, a lost peer ends a
collective through the process-group timeout, a device wait runs out on a flag nothing sets, and
training resumes bit-exactly from a checkpoint."""
import datetime
import os
import time
from pathlib import Path

import pytest
import torch

from tests.conftest import run_distributed
from tests.helpers import fake_dims, full_spec, random_batch, tiny_app_cfg

ROOT = Path(__file__).resolve().parent.parent


# ------------------------------------------------------------------ heartbeat
def test_heartbeat_marks_stale_and_missing_ranks(tmp_path):
    from nanotitan_b200.utils.heartbeat import Heartbeat, RankFailure, assert_peers_alive

    a, b = Heartbeat(tmp_path, 0), Heartbeat(tmp_path, 1)
    a.beat(3)
    b.beat(3)
    assert Heartbeat.stale_ranks(tmp_path, 3, max_age_s=60) == [2]  # rank 2 never wrote
    assert Heartbeat.read(tmp_path, 1)["step"] == 3
    later = time.time() + 120
    assert Heartbeat.stale_ranks(tmp_path, 2, max_age_s=60, now=later) == [0, 1]
    with pytest.raises(RankFailure, match=r"\[2\]"):
        assert_peers_alive(tmp_path, 3, 60)


def _lost_peer_worker(rank, world, hb_dir):
    """Rank 1 leaves between steps (no collective in flight).  Rank 0 learns it from the heartbeat
    before launching its next collective."""
    import torch.distributed as dist

    from nanotitan_b200.utils.heartbeat import Heartbeat, RankFailure, assert_peers_alive

    hb = Heartbeat(hb_dir, rank)
    t = torch.ones(4)
    dist.all_reduce(t)  # step 1 works
    hb.beat(1)
    dist.barrier()
    if rank == 1:
        return  # "dies" here
    time.sleep(1.5)
    hb.beat(2)
    with pytest.raises(RankFailure):
        assert_peers_alive(hb_dir, world, max_age_s=1.0)


@pytest.mark.distributed
def test_survivor_detects_lost_peer_before_next_collective(tmp_path):
    run_distributed(_lost_peer_worker, 2, str(tmp_path))


def _train_loop_worker(rank, world, tmp):
    """The training loop itself: rank 1 is configured for one step and leaves cleanly after it, rank 0
    for four.  Rank 0's loop must find rank 1 gone on the host, before it launches step 2."""
    from nanotitan_b200 import train
    from nanotitan_b200.parallel import PipelineParallel
    from nanotitan_b200.sweep import dump_toml
    from nanotitan_b200.utils.heartbeat import RankFailure
    from tests.helpers import tiny_app_cfg

    cfg = tiny_app_cfg(dp=2, batch=2).model_dump(mode="json")
    cfg["max_steps"] = 4 if rank == 0 else 1
    cfg["fault"] = {"pg_timeout_s": 30.0, "heartbeat_dir": str(Path(tmp) / "hb"), "heartbeat_stale_s": 60.0}
    path = Path(tmp) / f"cfg{rank}.toml"
    path.write_text(dump_toml(cfg), encoding="utf-8")
    plain_step = PipelineParallel.train_step
    steps_started = []

    def counted_step(self, *a, **kw):
        steps_started.append(1)
        return plain_step(self, *a, **kw)

    plain_check = train.assert_peers_alive

    def late_check(*a, **kw):
        if rank == 0 and steps_started:
            time.sleep(1.5)  # the leaving rank has written its marker by the time this rank looks
        return plain_check(*a, **kw)

    PipelineParallel.train_step = counted_step
    train.assert_peers_alive = late_check
    try:
        if rank == 0:
            with pytest.raises(RankFailure):
                train.main([str(path), "--synthetic-data", "--log.level", "WARNING"])
            assert len(steps_started) == 1, "the stale peer must be found before step 2 is launched"
        else:
            train.main([str(path), "--synthetic-data", "--log.level", "WARNING"])
    finally:
        PipelineParallel.train_step = plain_step
        train.assert_peers_alive = plain_check


@pytest.mark.distributed
def test_training_loop_stops_before_the_next_step_when_a_peer_left(tmp_path):
    run_distributed(_train_loop_worker, 2, str(tmp_path))


def _timeout_worker(rank, world, init_file):
    import torch.distributed as dist

    group = dist.new_group(ranks=[0, 1], timeout=datetime.timedelta(seconds=2))
    if rank == 1:
        time.sleep(6)  # never joins the collective within the limit
        return
    with pytest.raises(Exception):
        t = torch.ones(2)
        dist.all_reduce(t, group=group)
        dist.barrier(group=group)


@pytest.mark.distributed
def test_short_group_timeout_ends_a_collective_with_an_error(tmp_path):
    run_distributed(_timeout_worker, 2, str(tmp_path))


def _raising_worker(rank, world):
    if rank == 1:
        raise RuntimeError("injected host-side failure")
    time.sleep(0.2)


@pytest.mark.distributed
def test_a_raising_rank_is_reported_by_the_launcher():
    with pytest.raises(AssertionError, match="injected host-side failure"):
        run_distributed(_raising_worker, 2)


# ------------------------------------------------------------------ checkpoint / resume
def _steps(model, step_fn, opt, cfg, seeds):
    return [step_fn.train_step(model, random_batch(cfg, s), opt)["train/ce_loss"].value for s in seeds]


def test_resume_reproduces_the_uninterrupted_run(tmp_path):
    from nanotitan_b200.models.model import NanoTitanModel
    from nanotitan_b200.parallel import PipelineParallel
    from nanotitan_b200.parallel.reducer import ReducerV1
    from nanotitan_b200.utils import seed_everything
    from nanotitan_b200.utils.checkpoint import latest_checkpoint, load_checkpoint, save_checkpoint

    cfg = tiny_app_cfg()

    def build():
        seed_everything(9)
        model = NanoTitanModel(cfg.model, full_spec(cfg.model))
        reducers = {k: ReducerV1(v, 1, None, 1) for k, v in model.parameter_sync_groups().items()}
        dims = fake_dims(num_experts=4)
        return model, PipelineParallel(cfg, dims, reducers), torch.optim.AdamW(model.parameters(), lr=1e-2, weight_decay=0.1), dims

    model, step_fn, opt, dims = build()
    straight = _steps(model, step_fn, opt, cfg, range(6))

    model, step_fn, opt, dims = build()
    first = _steps(model, step_fn, opt, cfg, range(3))
    save_checkpoint(tmp_path, 3, 0, model, opt, dims, cfg)
    (tmp_path / "step_00000009").mkdir()  # a save that never finished (no manifest) is ignored
    model, step_fn, opt, dims = build()  # "restart"
    found = latest_checkpoint(tmp_path)
    assert found.name == "step_00000003"
    assert load_checkpoint(found, model, opt, dims)["step"] == 3
    resumed = _steps(model, step_fn, opt, cfg, range(3, 6))
    assert first + resumed == straight  # bitwise


# ------------------------------------------------------------------ device-side bounded wait
@pytest.mark.gpu
def test_device_wait_runs_out_and_reports_status():
    from nanotitan_b200.ops.ext import get_ext

    ext = get_ext()
    ext.read_status(True)
    assert ext.bounded_wait_probe(50.0) == 64  # every thread gave up, nobody hung
    code, kernel, detail, count = ext.read_status(True)
    assert (code, kernel) == (1, 7) and count >= 1
    # the context is intact and later kernels run (the status word was cleared by the read)
    x = torch.randn(256, 64, device="cuda").bfloat16()
    w = torch.randn(64, 64, device="cuda").bfloat16()
    from nanotitan_b200.ops import native

    y = torch.empty(256, 64, device="cuda", dtype=torch.bfloat16)
    native.gemm_tc(x, False, [w], False, [y])
    torch.testing.assert_close(y.float(), x.float() @ w.float().t(), rtol=2e-2, atol=0.3)
    assert ext.read_status(True)[0] == 0


@pytest.mark.gpu
def test_recorded_failure_turns_later_kernels_into_noops_until_cleared():
    from nanotitan_b200.ops import native
    from nanotitan_b200.ops.ext import get_ext

    ext = get_ext()
    ext.read_status(True)
    ext.bounded_wait_probe(20.0)
    x = torch.randn(128, 64, device="cuda").bfloat16()
    y = torch.full((128, 64), 7.0, device="cuda", dtype=torch.bfloat16)
    native.gemm_tc(x, False, [x[:64].contiguous()], False, [y])  # skipped: status word is set
    assert (y == 7.0).all()
    assert ext.read_status(True)[0] == 1
    native.gemm_tc(x, False, [x[:64].contiguous()], False, [y])
    assert not (y == 7.0).all()


@pytest.mark.gpu
def test_cross_rank_barrier_wait_runs_out_on_one_gpu():
    """The flag barrier of the expert-parallel kernels, made to give up without a second GPU and without
    any rank leaving: a two-entry peer table whose entries both point at this GPU's own flag pad, and a
    "peer" word that nobody ever writes.  The kernel returns after its 50 ms limit, the status word says
    time-out in the dispatch kernel, and the next kernel runs normally."""
    from nanotitan_b200.ops.ext import get_ext

    ext = get_ext()
    ext.read_status(True)
    dev = torch.device("cuda", 0)
    flags = torch.zeros(64, dtype=torch.int32, device=dev)
    cmat = torch.zeros(2, 4, dtype=torch.int32, device=dev)
    counts = torch.tensor([1, 2, 3, 4], dtype=torch.int32, device=dev)
    epoch = torch.zeros(1, dtype=torch.int32, device=dev)
    both_me = torch.tensor([flags.data_ptr(), flags.data_ptr()], dtype=torch.int64)
    cmat_me = torch.tensor([cmat.data_ptr(), cmat.data_ptr()], dtype=torch.int64)
    start = time.perf_counter()
    ext.ep_allgather_counts(counts, cmat_me, flags, both_me, 0, 2, epoch, 0, 50.0)
    torch.cuda.synchronize()
    assert time.perf_counter() - start < 5.0
    code, kernel, detail, count = ext.read_status(True)
    assert (code, kernel) == (1, 5) and count >= 1 and detail % 1000 == 1, (code, kernel, detail, count)
    assert int(epoch.item()) == 1  # the launch still advanced its epoch: later launches stay in step
    # the context is intact and later kernels are not no-ops once the word is cleared
    y = torch.empty(8, dtype=torch.float32, device=dev)
    ext.copy_vector(torch.arange(8, dtype=torch.float32, device=dev), y)
    assert y.tolist() == list(range(8))
    assert ext.read_status(True)[0] == 0


# ------------------------------------------------------------------ restart by the launcher
def _launch(tmp_path, name, ckpt_dir, env_extra, restarts):
    import os
    import socket
    import subprocess
    import sys

    from nanotitan_b200.sweep import dump_toml

    cfg = tiny_app_cfg(dp=2, batch=2).model_dump(mode="json")
    cfg.update(max_steps=6, run_name=name, checkpoint={"dir": str(ckpt_dir), "every_steps": 2, "resume": True})
    path = tmp_path / f"{name}.toml"
    path.write_text(dump_toml(cfg), encoding="utf-8")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=str(ROOT), **env_extra)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--max-restarts", str(restarts),
           "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "nanotitan_b200.train", str(path),
           "--synthetic-data", "--log.level", "INFO"]
    return subprocess.run(cmd, cwd=tmp_path, env=env, capture_output=True, text=True, timeout=240)


@pytest.mark.distributed
def test_launcher_restart_resumes_from_the_last_checkpoint_and_ends_where_a_clean_run_ends(tmp_path):
    """Rank 1 leaves the job before step 3 of the first attempt (host-side injection).  The launcher restarts
    both ranks; they resume from the step-2 checkpoint - weights, optimizer, RNG and loader position - and the
    final weights are bitwise those of a run that was never interrupted."""
    from nanotitan_b200.utils.checkpoint import consolidate, latest_checkpoint

    clean = _launch(tmp_path, "clean", tmp_path / "ckpt_clean", {}, restarts=0)
    assert clean.returncode == 0, clean.stderr[-3000:]
    broken = _launch(tmp_path, "broken", tmp_path / "ckpt_broken", {"NT_INJECT_EXIT": "1:3:0"}, restarts=1)
    assert broken.returncode == 0, broken.stderr[-3000:]
    log = broken.stdout + broken.stderr
    assert "NT_INJECT_EXIT: rank 1 leaves before step 3" in log
    assert "resumed from" in log and "at step 2" in log
    a, b = latest_checkpoint(tmp_path / "ckpt_clean"), latest_checkpoint(tmp_path / "ckpt_broken")
    assert a.name == b.name == "step_00000006"
    wa, wb = consolidate(a), consolidate(b)
    assert wa.keys() == wb.keys()
    for key in wa:
        assert torch.equal(wa[key], wb[key]), key
