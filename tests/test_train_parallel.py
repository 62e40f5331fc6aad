"""End-to-end steps on gloo ranks: DDP, GPipe PP, EP and 3-D layouts against one process."""
import pytest
import torch

from nanotitan_b200.models.model import NanoTitanModel
from nanotitan_b200.models.utils import get_model_shard_specs
from nanotitan_b200.parallel_dims import ParallelDims
from nanotitan_b200.train import build_training
from nanotitan_b200.utils import seed_everything
from nanotitan_b200.utils.checkpoint import consolidate, load_full_state, save_checkpoint
from tests.conftest import run_distributed
from tests.helpers import fake_dims, full_spec, random_batch, tiny_app_cfg


def _single_process_losses(cfg, batches, n_steps):
    """Whole model on one process, whole global batch, plain AdamW."""
    seed_everything(cfg.trainer.seed)
    model = NanoTitanModel(cfg.model, full_spec(cfg.model))
    opt = torch.optim.AdamW(model.parameters(), lr=cfg.optim.lr, weight_decay=0.1)
    losses = []
    for step in range(n_steps):
        x, y = batches[step]
        opt.zero_grad()
        logits, stats = model(x)
        ce = torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]), y.reshape(-1))
        aux = torch.stack([s.aux_loss for s in stats]).mean()
        (ce + aux).backward()
        opt.step()
        losses.append(ce.item())
    return losses, model


def _global_batches(cfg, data_world, n_steps):
    out = []
    for step in range(n_steps):
        parts = [random_batch(cfg, 1000 * step + r) for r in range(data_world)]
        out.append((torch.cat([p[0] for p in parts]), torch.cat([p[1] for p in parts])))
    return out


def _worker(rank, world, dp, pp, ep, microbatches, experts, tmpdir):
    cfg = tiny_app_cfg(dp=dp, pp=pp, ep=ep, microbatches=microbatches, batch=4,
                       num_experts=experts, top_k=min(2, experts), n_layers=2)
    seed_everything(cfg.trainer.seed)
    dims = ParallelDims(cfg.runtime)
    model, _, step_fn, opt = build_training(cfg, dims)
    # every rank starts from the weights the single-process model gets from this seed
    seed_everything(cfg.trainer.seed)
    load_full_state(model, NanoTitanModel(cfg.model, full_spec(cfg.model)).state_dict())
    n_steps = 3
    losses = []
    for step in range(n_steps):
        batch = random_batch(cfg, 1000 * step + dims.data_rank)
        m = step_fn.train_step(model, batch, opt)
        from nanotitan_b200.metrics import reduce_metrics
        red = reduce_metrics(m, torch.device("cpu"))
        losses.append(red["train/ce_loss"] / dims.data_world_size)
    if tmpdir:
        save_checkpoint(tmpdir, n_steps, 0, model, opt, dims, cfg)
        torch.distributed.barrier()
    if rank == 0:
        want, ref_model = _single_process_losses(cfg, _global_batches(cfg, dims.data_world_size, n_steps), n_steps)
        # With experts sharded or data split, every rank routes its own tokens, so the mean of
        # per-rank losses equals the global-batch loss; the load-balancing term differs slightly
        # between "per-rank fractions" and "global fractions", hence the looser tolerance with E>1.
        tol = 1e-4 if experts == 1 else 2e-3
        assert losses == pytest.approx(want, rel=tol, abs=tol), (losses, want)
        if tmpdir and experts == 1:
            merged = consolidate(f"{tmpdir}/step_{n_steps:08d}")
            want_sd = ref_model.state_dict()
            assert set(merged) == set(want_sd)
            for k, v in want_sd.items():
                torch.testing.assert_close(merged[k], v, rtol=1e-3, atol=1e-5, msg=k)


@pytest.mark.distributed
@pytest.mark.parametrize("dp,pp,ep,mb,experts", [
    (2, 1, 1, 1, 1),   # bucketed DDP (the CPU/gloo plumbing configuration, dense-equivalent)
    (1, 2, 1, 2, 1),   # GPipe, 2 stages, 2 microbatches
    (1, 1, 2, 1, 4),   # expert parallel
    (2, 2, 1, 2, 4),   # DP x PP with experts
])
def test_parallel_losses_match_single_process(dp, pp, ep, mb, experts, tmp_path):
    run_distributed(_worker, dp * pp * ep, dp, pp, ep, mb, experts, str(tmp_path))


@pytest.mark.distributed
def test_three_d_layout_runs():
    run_distributed(_worker, 8, 2, 2, 2, 2, 4, "")


def test_single_process_step_without_launcher_uses_fake_dims():
    cfg = tiny_app_cfg()
    seed_everything(3)
    from nanotitan_b200.parallel import PipelineParallel
    from nanotitan_b200.parallel.reducer import ReducerV1

    model = NanoTitanModel(cfg.model, full_spec(cfg.model))
    groups = model.parameter_sync_groups()
    reducers = {k: ReducerV1(v, 1, None, 1) for k, v in groups.items()}
    step_fn = PipelineParallel(cfg, fake_dims(num_experts=4), reducers)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2, weight_decay=0.1)
    first = step_fn.train_step(model, random_batch(cfg, 0), opt)["train/ce_loss"].value
    for _ in range(5):
        last = step_fn.train_step(model, random_batch(cfg, 0), opt)["train/ce_loss"].value
    assert last < first
    spec = get_model_shard_specs(fake_dims(num_experts=4, dp_size=1), cfg)
    assert spec.layer_end == cfg.model.n_layers and spec.has_unembed_head


def test_deferred_metrics_match_immediate_ones():
    """`collect_metrics="deferred"` returns at once; `.result()` later gives the step's own metrics."""
    from nanotitan_b200.parallel import PipelineParallel
    from nanotitan_b200.parallel.reducer import ReducerV1

    def run(mode):
        cfg = tiny_app_cfg()
        seed_everything(5)
        model = NanoTitanModel(cfg.model, full_spec(cfg.model))
        reducers = {k: ReducerV1(v, 1, None, 1) for k, v in model.parameter_sync_groups().items()}
        step_fn = PipelineParallel(cfg, fake_dims(num_experts=4), reducers)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-2, weight_decay=0.1)
        out = [step_fn.train_step(model, random_batch(cfg, s), opt, collect_metrics=mode) for s in range(3)]
        return [m.result() if mode == "deferred" else m for m in out]  # resolved only after all steps ran

    now, later = run(True), run("deferred")
    for a, b in zip(now, later):
        assert a.keys() == b.keys()
        assert a["train/ce_loss"].value == pytest.approx(b["train/ce_loss"].value, rel=1e-6)
        assert a["train/lb_loss"].value == pytest.approx(b["train/lb_loss"].value, rel=1e-6)
        key = "moe/layer_00/route_frac_dist"
        torch.testing.assert_close(a[key].value, b[key].value)
