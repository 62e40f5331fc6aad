"""The per-GPU plan: its exact parts against the objects a run builds (parameters, bucket layout, optimizer state
bytes, expert staging capacity), and the command line."""
import pytest
import torch

from tests.helpers import fake_dims, full_spec, tiny_app_cfg


def test_exact_parts_match_what_a_single_process_run_builds():
    from nanotitan_b200 import plan
    from nanotitan_b200.models.model import NanoTitanModel
    from nanotitan_b200.ops.adamw import FusedAdamW
    from nanotitan_b200.parallel.reducer import ReducerV1

    cfg = tiny_app_cfg(dtype="bfloat16")
    (shard,) = plan.plan(cfg)
    model = NanoTitanModel(cfg.model, full_spec(cfg.model))
    groups = model.parameter_sync_groups()
    reducers = {k: ReducerV1(v, 1, None, cfg.runtime.bucket_size) for k, v in groups.items()}
    opt = FusedAdamW(list(model.parameters()), lr=1e-3)
    opt.bind_reducers(reducers)
    assert shard.parameters == {k: sum(p.numel() for p in v) for k, v in groups.items()}
    assert shard.buckets == {k: len(r.buckets) for k, r in reducers.items()}
    assert shard.bytes["parameters"] == sum(p.numel() * p.element_size() for p in model.parameters())
    assert shard.bytes["gradient buckets"] == sum(b.buffer.numel() * b.buffer.element_size() for r in reducers.values() for b in r.buckets)
    (optimizer_item,) = [k for k in shard.bytes if k.startswith("optimizer state")]
    assert shard.bytes[optimizer_item] == opt.state_bytes()
    assert shard.layers == (0, cfg.model.n_layers) and shard.ranks == [0]
    assert len(shard.estimated) == 1 and shard.estimated[0] in shard.bytes


def test_sharded_optimizer_state_and_layout_of_a_3d_run():
    from nanotitan_b200 import plan
    from nanotitan_b200.parallel.fused_allreduce import owned_slice

    cfg = tiny_app_cfg(dp=2, pp=2, ep=2, microbatches=2, batch=4, dtype="bfloat16")
    shards = plan.plan(cfg)
    assert [(s.pp_rank, s.ep_rank) for s in shards] == [(0, 0), (0, 1), (1, 0), (1, 1)]
    assert sorted(r for s in shards for r in s.ranks) == list(range(8))
    first, last = shards[0], shards[-1]
    assert first.layers == (0, 1) and last.layers == (1, 2) and first.experts == (0, 2) and shards[1].experts == (2, 4)
    assert any(k.startswith("logits buffer") for k in last.bytes) and not any(k.startswith("logits buffer") for k in first.bytes)
    assert any(k.startswith("expert exchange staging") for k in first.bytes)
    # shared parameters are replicated over dp x ep = 4 ranks, experts over dp = 2: 16-bit buckets keep 1/4 and 1/2
    single = plan.plan(tiny_app_cfg(pp=2, ep=2, microbatches=2, batch=4, dtype="bfloat16"))[0]
    key = next(k for k in first.bytes if k.startswith("optimizer state"))
    assert first.bytes[key] < single.bytes[key]
    assert owned_slice(1024, 4, 0) == (0, 256)


def test_capacity_rule_is_the_exchange_s_rule():
    from nanotitan_b200 import plan
    from nanotitan_b200.parallel.ep_fused import FusedExchange

    for ep, factor in ((4, 0.0), (8, 0.0), (4, 2.0), (8, 1.25)):
        ex = object.__new__(FusedExchange)
        ex.ep, ex.capacity_factor = ep, factor
        for assignments in (1, 100, 24576, 262144):
            assert plan.expert_capacity_rows(ep, assignments, factor) == ex.capacity_rows(assignments)


def test_command_line(tmp_path, capsys):
    import json

    from nanotitan_b200 import plan
    from nanotitan_b200.sweep import dump_toml

    path = tmp_path / "cfg.toml"
    path.write_text(dump_toml(tiny_app_cfg(ep=2, batch=2, dtype="bfloat16").model_dump(mode="json")), encoding="utf-8")
    assert plan.main([str(path)]) == 0
    text = capsys.readouterr().out
    assert "expert rank 1" in text and "fits" in text and "(estimate)" in text
    assert plan.main([str(path), "--hbm-gb", "0.000001"]) == 1
    assert "DOES NOT FIT" in capsys.readouterr().out
    assert plan.main(["@" + str(path), "--json"]) == 0
    out = json.loads(capsys.readouterr().out)
    rows = out["shards"]
    assert len(rows) == 2 and rows[0]["total"] == sum(rows[0]["bytes"].values())
    assert out["step"]["gpus"] == 2 and out["step"]["tokens_per_step"] == 2 * 2 * 8 and out["step"]["floor_ms"] > 0


def test_nvlink_traffic_by_cause():
    from nanotitan_b200 import plan

    cfg = tiny_app_cfg(dp=2, pp=2, ep=2, microbatches=2, batch=4, dtype="bfloat16")  # d 16, seq 8, top-2, 2 layers
    first, *_, last = plan.plan(cfg)
    a, b = plan.nvlink_bytes_per_step(cfg, first), plan.nvlink_bytes_per_step(cfg, last)
    # shared parameters are replicated over dp x ep = 4 ranks, experts over dp = 2: both groups all-reduce
    assert a["gradient all-reduce"] == 2 * (first.parameters["shared"] + first.parameters["expert"])
    # one layer per stage, two micro-batches of 2 x 8 tokens, top-2, half of the rows leave the GPU, four transfers
    assert a["expert exchange"] == 4 * 1 * 2 * (2 * 8 * 2) * 16 * 2 // 2
    # the first stage has one neighbour: activations out, gradients in - one direction each
    assert a["pipeline boundaries"] == 1 * 2 * (2 * 8) * 16 * 2 == b["pipeline boundaries"]
    alone = plan.plan(tiny_app_cfg(dtype="bfloat16"))[0]
    assert sum(plan.nvlink_bytes_per_step(tiny_app_cfg(dtype="bfloat16"), alone).values()) == 0


@pytest.mark.parametrize("name", ["dense_92m", "moe_ep8", "moe_3d", "dense_92m_cpu_ddp", "big_sabaka", "dist"])
def test_shipped_configs_load_and_fit_one_gpu(name):
    """Every configuration in configs/ validates against the schema, its layout tiles the ranks, and what it puts on
    each GPU (worst-case expert capacity included) is below 180 GB."""
    from pathlib import Path

    from nanotitan_b200 import plan
    from nanotitan_b200.config import load_config

    cfg = load_config(Path(__file__).resolve().parent.parent / "configs" / f"{name}.toml")
    shards = plan.plan(cfg)
    world = cfg.runtime.dp_size * cfg.runtime.pp_size * cfg.runtime.ep_size
    assert sorted(r for s in shards for r in s.ranks) == list(range(world))
    assert sum(s.layers[1] - s.layers[0] for s in shards if s.ep_rank == 0) == cfg.model.n_layers
    for s in shards:
        assert s.total < 180e9, (name, s.pp_rank, s.ep_rank, s.total / 1e9)
    floor = plan.step_floor(cfg, 1400.0)
    assert floor["gpus"] == world and floor["floor_ms"] > 0
