"""The model on the native kernels against the same model on PyTorch ops (fp32 oracle)."""
import copy

import pytest
import torch

from nanotitan_b200.config import ModelConfig
from nanotitan_b200.models import ModelShardSpec, NanoTitanModel

pytestmark = pytest.mark.gpu


def _cfg(**over):
    base = dict(vocab_size=1003, d_model=128, d_head=32, n_heads=4, n_layers=2, max_seq_len=128, ffn_in=256,
                num_experts=4, top_k=2, router_alpha=0.01, moe_backend="cuda", dtype="bfloat16")
    base.update(over)
    return ModelConfig(**base)


def _oracle(model, cfg):
    ocfg = cfg.model_copy(update=dict(moe_backend="torch", dtype="float32"))
    oracle = NanoTitanModel(ocfg, ModelShardSpec.full(ocfg)).cuda()
    with torch.no_grad():
        for (k, v), (_, ov) in zip(model.state_dict().items(), oracle.state_dict().items()):
            ov.copy_(v.float())
    for block in oracle.blocks:
        if hasattr(block, "ffn"):
            block.ffn.moe_backend.aux_on_detached_tokens = True  # the semantics of the CUDA backend
    return oracle


@pytest.mark.parametrize("experts,top_k", [(1, 1), (4, 2)])
def test_forward_loss_and_gradients_match_fp32_oracle(experts, top_k, monkeypatch):
    torch.manual_seed(0)
    cfg = _cfg(num_experts=experts, top_k=top_k)
    model = NanoTitanModel(cfg, ModelShardSpec.full(cfg)).cuda()
    oracle = _oracle(model, cfg)
    ids = torch.randint(0, cfg.vocab_size, (3, cfg.max_seq_len + 1), device="cuda")
    x, y = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
    loss, stats = model.forward_loss(x, y)
    aux = torch.stack([s.aux_loss for s in stats]).mean()
    (loss + aux).backward()
    monkeypatch.setenv("NT_DISABLE_NATIVE", "all")
    want, ostats = oracle.forward_loss(x, y)
    oaux = torch.stack([s.aux_loss for s in ostats]).mean()
    (want + oaux).backward()
    assert abs(loss.item() - want.item()) < 3e-2 * max(1.0, abs(want.item()))
    assert sum(s.tokens_per_expert.sum().item() for s in stats) == cfg.n_layers * x.numel() * top_k
    # per tensor: ||g - g_oracle|| / ||g_oracle|| <= 3 % (bf16 activations and weights against fp32).
    # With several experts a few tokens sit close enough to a routing tie that the bf16 model and the
    # fp32 oracle send them to different experts; those rows change whole gradient rows of the experts
    # of the first layers (measured: up to 4.6 % there, under 1.2 % everywhere else), hence 6 % for
    # the expert and ffn-norm tensors of a multi-expert model.
    errors = {}
    for (name, p), (_, q) in zip(model.named_parameters(), oracle.named_parameters()):
        assert p.grad is not None, name
        errors[name] = ((p.grad.float() - q.grad).norm() / (q.grad.norm() + 1e-12)).item()
    def bound(name):
        return 0.06 if experts > 1 and (".ffn.experts." in name or ".ffn_norm." in name) else 0.03

    bad = {k: round(v, 4) for k, v in errors.items() if v > bound(k)}
    assert not bad, f"relative gradient errors above 3 %: {bad} (all: { {k: round(v, 4) for k, v in errors.items()} })"


def test_training_reduces_loss_and_uses_native_kernels():
    from nanotitan_b200.ops.adamw import FusedAdamW
    from nanotitan_b200.ops.ext import get_ext

    torch.manual_seed(1)
    cfg = _cfg()
    model = NanoTitanModel(cfg, ModelShardSpec.full(cfg)).cuda()
    opt = FusedAdamW(list(model.parameters()), lr=3e-3)
    ids = torch.randint(0, cfg.vocab_size, (4, cfg.max_seq_len + 1), device="cuda")
    x, y = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
    before = get_ext().launch_count()
    losses = []
    for _ in range(8):
        opt.zero_grad()
        loss, stats = model.forward_loss(x, y)
        (loss + torch.stack([s.aux_loss for s in stats]).mean()).backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0]
    assert get_ext().launch_count() - before > 100
    assert get_ext().read_status(True)[0] == 0


def test_two_identical_steps_are_bitwise_identical():
    torch.manual_seed(2)
    cfg = _cfg()
    model = NanoTitanModel(cfg, ModelShardSpec.full(cfg)).cuda()
    ids = torch.randint(0, cfg.vocab_size, (2, cfg.max_seq_len + 1), device="cuda")
    x, y = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
    grads = []
    for _ in range(2):
        model.zero_grad(set_to_none=True)
        loss, _ = model.forward_loss(x, y)
        loss.backward()
        grads.append([p.grad.clone() for p in model.parameters()])
    for a, b in zip(*grads):
        assert torch.equal(a, b)


def test_pipeline_step_api_on_one_gpu():
    from tests.helpers import fake_dims, random_batch, tiny_app_cfg
    from nanotitan_b200.ops.adamw import FusedAdamW
    from nanotitan_b200.parallel import PipelineParallel
    from nanotitan_b200.parallel.reducer import ReducerV1

    cfg = tiny_app_cfg(vocab_size=503, d_model=64, d_head=32, n_heads=2, max_seq_len=64, ffn_in=128,
                       moe_backend="cuda", dtype="bfloat16", batch=4, microbatches=2)
    torch.manual_seed(3)
    model = NanoTitanModel(cfg.model, ModelShardSpec.full(cfg.model)).cuda()
    groups = model.parameter_sync_groups()
    reducers = {k: ReducerV1(v, 1, None, 1) for k, v in groups.items()}
    opt = FusedAdamW(list(model.parameters()), lr=3e-3)
    opt.bind_reducers(reducers)
    step = PipelineParallel(cfg, fake_dims(num_experts=4), reducers)
    first = step.train_step(model, random_batch(cfg, 0), opt)["train/ce_loss"].value
    for _ in range(6):
        last = step.train_step(model, random_batch(cfg, 0), opt)["train/ce_loss"].value
    assert last < first
