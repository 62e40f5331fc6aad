"""Small builders shared by the CPU tests."""
from __future__ import annotations

from types import SimpleNamespace

import torch

from nanotitan_b200.config import AppConfig, ModelConfig
from nanotitan_b200.models.utils import ModelShardSpec


def tiny_model_cfg(**over) -> ModelConfig:
    base = dict(vocab_size=61, d_model=16, d_head=4, n_heads=4, n_layers=2, max_seq_len=8,
                ffn_in=32, num_experts=4, top_k=2, router_alpha=0.01, moe_backend="torch")
    base.update(over)
    return ModelConfig(**base)


def tiny_app_cfg(dp=1, pp=1, ep=1, microbatches=1, batch=4, **model_over) -> AppConfig:
    model = tiny_model_cfg(**model_over).model_dump(mode="json")
    return AppConfig.model_validate(dict(
        run_name="test", max_steps=2, model=model,
        trainer=dict(device_id=0, eval_every_step=-1, per_device_batch_size=batch, seed=7),
        data=dict(num_workers=1, train_tokens_path="unused", val_tokens_path="unused"),
        optim=dict(type="adam", lr=1e-3),
        runtime=dict(name="t", dp_size=dp, pp_size=pp, ep_size=ep, num_microbatches=microbatches, bucket_size=1),
    ))


def full_spec(cfg, **over) -> ModelShardSpec:
    base = dict(layer_start=0, layer_end=cfg.n_layers, has_token_embed=True, has_pos_embed=True,
                has_unembed_head=True, per_rank_expert=cfg.num_experts, start_expert_id=0,
                end_expert_id=cfg.num_experts)
    base.update(over)
    return ModelShardSpec(**base)


def fake_dims(**kw):
    base = dict(global_rank=0, local_rank=0, world_size=1, dp_size=1, pp_size=1, ep_size=1, dp_rank=0,
                pp_rank=0, ep_rank=0, is_pp_first_stage=True, is_pp_last_stage=True, prev_pp_rank=-1,
                next_pp_rank=-1, pp_group=None, ep_group=None, shared_dp_group=None, expert_dp_group=None,
                shared_dp_group_ranks=[0], expert_dp_group_ranks=[0], data_world_size=1, data_rank=0,
                num_experts=1)
    base.update(kw)
    return SimpleNamespace(**base)


def random_batch(cfg: AppConfig, seed: int, batch: int | None = None):
    g = torch.Generator().manual_seed(seed)
    b = batch or cfg.trainer.per_device_batch_size
    ids = torch.randint(0, cfg.model.vocab_size, (b, cfg.model.max_seq_len + 1), generator=g)
    return ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
