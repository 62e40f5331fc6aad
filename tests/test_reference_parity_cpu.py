"""Semantic parity with the reference's own model code on CPU, in fp32: both models are built from the
reference's `state_dict()` (same keys, same shapes) and must produce the same logits, the same
load-balancing statistics and the same parameter gradients.  Runs the reference from baseline/_ref
(skipped when it is not installed); nothing here needs a GPU or a process group."""
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"

pytestmark = pytest.mark.skipif(not (REF / "model" / "model.py").exists(), reason="reference not installed under baseline/_ref")

MODEL = dict(vocab_size=211, d_model=64, d_head=16, n_heads=4, n_layers=3, max_seq_len=32, ffn_in=96, router_alpha=0.01,
             moe_backend="torch", dtype="float32")


def _reference_model(experts, top_k):
    sys.path.insert(0, str(ROOT / "baseline"))
    import ref_harness

    ref_harness._alias_src()
    from src.config import ModelConfig as RefModelConfig
    from src.model.model import NanoTitanModel as RefModel
    from src.model.utils import ModelShardSpec as RefSpec

    cfg = RefModelConfig(**dict(MODEL, num_experts=experts, top_k=top_k))
    cfg.dtype = torch.float32
    cfg.moe_router_dtype = torch.float32
    spec = RefSpec(layer_start=0, layer_end=cfg.n_layers, has_token_embed=True, has_pos_embed=True, has_unembed_head=True,
                   per_rank_expert=experts, start_expert_id=0, end_expert_id=experts, ep_size=1, ep_group=None)
    torch.manual_seed(5)
    return RefModel.from_specs(cfg, spec)


def _our_model(experts, top_k):
    from nanotitan_b200.config import ModelConfig
    from nanotitan_b200.models import ModelShardSpec, NanoTitanModel

    cfg = ModelConfig(**dict(MODEL, num_experts=experts, top_k=top_k))
    return NanoTitanModel(cfg, ModelShardSpec.full(cfg))


@pytest.mark.parametrize("experts,top_k", [(1, 1), (4, 2)])
def test_same_weights_give_the_same_logits_statistics_and_gradients(experts, top_k):
    ref = _reference_model(experts, top_k)
    ours = _our_model(experts, top_k)
    state = ref.state_dict()
    assert list(state) == list(ours.state_dict()), "state-dict keys / order differ from the reference"
    for key, value in state.items():
        assert ours.state_dict()[key].shape == value.shape, key
    ours.load_state_dict(state)

    torch.manual_seed(9)
    ids = torch.randint(0, MODEL["vocab_size"], (3, MODEL["max_seq_len"]))
    targets = torch.randint(0, MODEL["vocab_size"], (3, MODEL["max_seq_len"]))
    ref_logits, ref_stats = ref(ids)
    our_logits, our_stats = ours(ids)
    torch.testing.assert_close(our_logits, ref_logits, rtol=1e-4, atol=1e-4)
    for a, b in zip(our_stats, ref_stats):
        assert torch.equal(a.tokens_per_expert.long(), b.tokens_per_expert.long())
        torch.testing.assert_close(a.aux_loss, b.aux_loss, rtol=1e-5, atol=1e-6)

    def total(logits, stats):
        ce = torch.nn.functional.cross_entropy(logits.reshape(-1, logits.size(-1)), targets.reshape(-1))
        return ce + torch.stack([s.aux_loss for s in stats]).mean()

    total(ref_logits, ref_stats).backward()
    total(our_logits, our_stats).backward()
    mine = dict(ours.named_parameters())
    for name, p in ref.named_parameters():
        assert mine[name].grad is not None, name
        torch.testing.assert_close(mine[name].grad, p.grad, rtol=2e-4, atol=2e-5, msg=lambda m, n=name: f"{n}: {m}")


def test_training_trajectories_agree_over_twenty_steps():
    """Reference model + its optimizer (torch AdamW, weight decay 0.1) against this model + FusedAdamW
    (flat buckets, fp32 master weights), same weights and batches: the loss curves coincide."""
    from nanotitan_b200.ops.adamw import FusedAdamW

    ref = _reference_model(4, 2)
    ours = _our_model(4, 2)
    ours.load_state_dict(ref.state_dict())
    ref_opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, weight_decay=0.1)
    our_opt = FusedAdamW(ours.parameters(), lr=1e-3, weight_decay=0.1)

    def loss_of(model, ids, targets):
        logits, stats = model(ids)
        ce = torch.nn.functional.cross_entropy(logits.reshape(-1, logits.size(-1)), targets.reshape(-1))
        return ce + torch.stack([s.aux_loss for s in stats]).mean(), ce

    gen = torch.Generator().manual_seed(21)
    curve_ref, curve_ours = [], []
    for _ in range(20):
        ids = torch.randint(0, MODEL["vocab_size"], (4, MODEL["max_seq_len"]), generator=gen)
        targets = torch.roll(ids, -1, dims=1)
        for model, opt, curve in ((ref, ref_opt, curve_ref), (ours, our_opt, curve_ours)):
            opt.zero_grad()
            total, ce = loss_of(model, ids, targets)
            total.backward()
            opt.step()
            curve.append(ce.item())
    assert curve_ref[-1] < curve_ref[0], "the reference did not learn; the comparison would be empty"
    for step, (a, b) in enumerate(zip(curve_ours, curve_ref)):
        assert abs(a - b) < 2e-3 * max(1.0, abs(b)), f"step {step}: ours {a} reference {b}"
