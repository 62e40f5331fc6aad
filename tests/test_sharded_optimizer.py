"""Optimizer state sharded over the data-parallel ranks (the layout the fused all-reduce + AdamW
kernel works on), exercised on CPU: `HostBucketEngine` restates the kernel's data flow with gloo
collectives - all-reduce, 1/N, AdamW on the owned slice of the fp32 state, all-gather of the new
16-bit parameters - so that the layout, the checkpoint format and resume can be tested without GPUs."""
import pytest
import torch

from tests.conftest import run_distributed
from tests.helpers import random_batch, tiny_app_cfg


class HostBucketEngine:
    def __init__(self, group, world, rank):
        self.group, self.world, self.rank = group, world, rank
        self.bound = {}

    def alloc(self, numel, dtype, device):
        return torch.zeros(numel, dtype=dtype, device=device)

    def owned_slice(self, numel):
        from nanotitan_b200.parallel.fused_allreduce import owned_slice

        return owned_slice(numel, self.world, self.rank)

    def register(self, bucket):
        pass

    def bind_optimizer(self, bucket, flat_param, master, exp_avg, exp_avg_sq, optimizer):
        self.bound[id(bucket)] = (flat_param, master, exp_avg, exp_avg_sq, optimizer)

    def owns_update(self, bucket):
        return id(bucket) in self.bound

    def launch(self, reducer, bucket):
        import torch.distributed as dist

        from nanotitan_b200.ops import reference as ref

        grads = bucket.buffer.float()
        dist.all_reduce(grads, group=self.group)
        grads /= self.world
        bound = self.bound.get(id(bucket))
        if bound is None:
            bucket.buffer.copy_(grads)
            return None
        flat_param, master, m, v, opt = bound
        lo, hi = self.owned_slice(flat_param.numel())
        assert master.numel() == hi - lo, "optimizer state must cover the owned slice only"
        hyper = opt.param_groups[0]
        ref.adamw_step(master, grads[lo:hi], m, v, opt.next_step(), hyper["lr"], hyper["betas"][0], hyper["betas"][1],
                       hyper["eps"], hyper["weight_decay"])
        per = self.owned_slice(flat_param.numel())
        width = ((flat_param.numel() // 8 + self.world - 1) // self.world) * 8
        mine = torch.zeros(width, dtype=flat_param.dtype)
        mine[: hi - lo].copy_(master)
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine, group=self.group)
        flat_param.copy_(torch.cat(parts)[: flat_param.numel()])
        del per
        return None

    def finish(self, reducer, bucket):
        pass


def _build(cfg, dims, seed):
    from nanotitan_b200.models.model import NanoTitanModel
    from nanotitan_b200.models.utils import get_model_shard_specs
    from nanotitan_b200.ops.adamw import FusedAdamW
    from nanotitan_b200.parallel import PipelineParallel
    from nanotitan_b200.parallel.reducer import ReducerV1

    torch.manual_seed(seed)
    model = NanoTitanModel.from_specs(cfg.model, get_model_shard_specs(dims, cfg))
    groups = model.parameter_sync_groups()
    engine = HostBucketEngine(dims.shared_dp_group, dims.world_size, dims.global_rank)
    reducers = {
        "shared": ReducerV1(groups["shared"], dims.world_size, dims.shared_dp_group, 1, engine=engine),
        "expert": ReducerV1(groups["expert"], dims.world_size, dims.expert_dp_group, 1, engine=engine),
    }
    opt = FusedAdamW(list(model.parameters()), lr=cfg.optim.lr, weight_decay=0.1)
    opt.bind_reducers(reducers)
    return model, PipelineParallel(cfg, dims, reducers), opt


def _sharded_worker(rank, world, tmp):
    import torch.distributed as dist

    from nanotitan_b200.parallel_dims import ParallelDims
    from nanotitan_b200.utils.checkpoint import latest_checkpoint, load_checkpoint, save_checkpoint

    cfg = tiny_app_cfg(dp=world, batch=2, dtype="bfloat16", moe_backend="torch")
    dims = ParallelDims(cfg.runtime)

    def steps(model, step, opt, seeds):
        return [step.train_step(model, random_batch(cfg, 100 * s + rank), opt)["train/ce_loss"].value for s in seeds]

    model, step, opt = _build(cfg, dims, seed=3)
    # ZeRO-1: fp32 master + two moments for 1/N of every 16-bit bucket (the fp32 router weights are
    # reduced by the plain collective and keep whole-bucket state)
    sharded = [c for c in opt._chunks if c.flat_param.dtype == torch.bfloat16]
    whole = [c for c in opt._chunks if c.flat_param.dtype != torch.bfloat16]
    assert sharded and all(c.fused_by_engine and c.master.numel() == (c.flat_param.numel() // 8 + world - 1) // world * 8
                           for c in sharded)
    assert all(not c.fused_by_engine and c.master.numel() == c.flat_param.numel() for c in whole)
    assert opt.state_bytes() == 12 * sum(c.master.numel() for c in opt._chunks)
    straight = steps(model, step, opt, range(6))
    want = [p.detach().clone() for p in model.parameters()]

    model, step, opt = _build(cfg, dims, seed=3)
    first = steps(model, step, opt, range(3))
    save_checkpoint(tmp, 3, 0, model, opt, dims, cfg)
    model, step, opt = _build(cfg, dims, seed=99)  # different weights: the load has to restore everything
    state = load_checkpoint(latest_checkpoint(tmp), model, opt, dims)
    assert state["step"] == 3
    second = steps(model, step, opt, range(3, 6))
    assert first + second == straight
    for p, w in zip(model.parameters(), want):
        assert torch.equal(p.detach(), w)
    flat = torch.cat([p.detach().float().reshape(-1) for p in model.parameters()])
    other = flat.clone()
    dist.all_reduce(other, op=dist.ReduceOp.MAX)
    assert torch.equal(flat, other), "replicas diverged after the resume"

    # a bucket the engine owns cannot be updated locally: its state is not all here
    for r in step.reducers.values():
        r.zero_grad()
    with pytest.raises(RuntimeError, match="sharded"):
        opt.step()


@pytest.mark.distributed
def test_sharded_state_saves_loads_and_resumes_identically(tmp_path):
    run_distributed(_sharded_worker, 2, str(tmp_path))


def test_owned_slices_tile_the_bucket():
    from nanotitan_b200.parallel.fused_allreduce import owned_slice

    for numel in (128, 1152, 25 * 2**19, 8):
        for world in (1, 2, 3, 4, 8, 16):
            cuts = [owned_slice(numel, world, r) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == numel
            assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
            assert all(lo % 8 == 0 for lo, _ in cuts)


def test_load_refuses_a_different_layout():
    from nanotitan_b200.ops.adamw import FusedAdamW

    params = [torch.nn.Parameter(torch.randn(40, 8))]
    opt = FusedAdamW(params, lr=1e-3)
    state = opt.state_dict()
    state["chunks"][0]["owned"] = (0, 8)
    with pytest.raises(ValueError, match="slice"):
        FusedAdamW([torch.nn.Parameter(torch.randn(40, 8))], lr=1e-3).load_state_dict(state)


# ------------------------------------------------------------------ optimizer state across layouts
def _build_for(cfg, dims, seed):
    """Like `_build`, with each reducer on its own group size (an expert-parallel layout has one-rank expert groups)."""
    from nanotitan_b200.models.model import NanoTitanModel
    from nanotitan_b200.models.utils import get_model_shard_specs
    from nanotitan_b200.ops.adamw import FusedAdamW
    from nanotitan_b200.parallel import PipelineParallel
    from nanotitan_b200.parallel.reducer import ReducerV1

    torch.manual_seed(seed)
    model = NanoTitanModel.from_specs(cfg.model, get_model_shard_specs(dims, cfg))
    groups = model.parameter_sync_groups()
    reducers = {}
    for name, group, ranks in (("shared", dims.shared_dp_group, dims.shared_dp_group_ranks),
                               ("expert", dims.expert_dp_group, dims.expert_dp_group_ranks)):
        size = len(ranks)
        engine = HostBucketEngine(group, size, ranks.index(dims.global_rank)) if size > 1 else None
        reducers[name] = ReducerV1(groups[name], size, group, 1, engine=engine)
    opt = FusedAdamW(list(model.parameters()), lr=cfg.optim.lr, weight_decay=0.1)
    opt.bind_reducers(reducers)
    return model, PipelineParallel(cfg, dims, reducers), opt


def _relayout_worker(rank, world, tmp):
    from pathlib import Path

    from nanotitan_b200.parallel_dims import ParallelDims
    from nanotitan_b200.utils.checkpoint import (consolidate, consolidate_optimizer, load_full_optimizer, load_full_state,
                                                 save_checkpoint)

    tmp = Path(tmp)
    cfg_a = tiny_app_cfg(dp=world, batch=2, dtype="bfloat16", moe_backend="torch")
    dims_a = ParallelDims(cfg_a.runtime)
    model, step, opt = _build_for(cfg_a, dims_a, seed=3)
    assert any(c.master.numel() < c.flat_param.numel() for c in opt._chunks), "nothing is sharded: the test would be empty"
    for s in range(3):
        step.train_step(model, random_batch(cfg_a, 100 * s + rank), opt)
    save_checkpoint(tmp / "a", 3, 0, model, opt, dims_a, cfg_a, portable_optimizer=True)
    weights_a, optim_a = consolidate(tmp / "a" / "step_00000003"), consolidate_optimizer(tmp / "a" / "step_00000003")
    assert optim_a["step"] == 3 and set(optim_a["state"]) == {"master", "exp_avg", "exp_avg_sq"}
    assert set(optim_a["state"]["master"]) == {k for k, v in weights_a.items() if v.is_floating_point()} - _buffers(model)
    assert any(v.abs().max() > 0 for v in optim_a["state"]["exp_avg"].values())

    # the same two processes as an expert-parallel pair, then as two pipeline stages: other shards, other buckets,
    # other owners of every slice
    for name, layout in (("ep", dict(ep=world)), ("pp", dict(pp=world, microbatches=2))):
        cfg_b = tiny_app_cfg(batch=2, dtype="bfloat16", moe_backend="torch", **layout)
        dims_b = ParallelDims(cfg_b.runtime)
        model_b, step_b, opt_b = _build_for(cfg_b, dims_b, seed=99)
        load_full_state(model_b, weights_a)
        load_full_optimizer(model_b, opt_b, optim_a)
        save_checkpoint(tmp / name, 3, 0, model_b, opt_b, dims_b, cfg_b, portable_optimizer=True)
        weights_b, optim_b = consolidate(tmp / name / "step_00000003"), consolidate_optimizer(tmp / name / "step_00000003")
        assert list(weights_b) == list(weights_a)
        for key in weights_a:
            assert torch.equal(weights_a[key], weights_b[key]), (name, key)
        for part in ("master", "exp_avg", "exp_avg_sq"):
            for key, value in optim_a["state"][part].items():
                assert torch.equal(value, optim_b["state"][part][key]), (name, part, key)
        assert opt_b._step == 3
        loss = step_b.train_step(model_b, random_batch(cfg_b, 7 + dims_b.data_rank), opt_b)  # and it trains on
        assert loss is not None


def _buffers(model):
    return {name for name, _ in model.named_buffers()}


@pytest.mark.distributed
def test_optimizer_state_moves_between_layouts_exactly(tmp_path):
    run_distributed(_relayout_worker, 2, str(tmp_path))
