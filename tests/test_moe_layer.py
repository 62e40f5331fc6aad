"""Model / MoE layer API (mirrors the reference's tests/test_moe_layer.py and adds oracles)."""
import pytest
import torch

from nanotitan_b200.models.feed_fwd import MoE
from nanotitan_b200.models.model import NanoTitanModel
from nanotitan_b200.models.utils import MoELayerStats
from nanotitan_b200.ops import reference as ref
from tests.helpers import full_spec, tiny_model_cfg


def test_moe_output_shape_and_stats():
    cfg = tiny_model_cfg(d_model=8, ffn_in=16)
    moe = MoE(cfg, full_spec(cfg, has_token_embed=False, has_pos_embed=False, has_unembed_head=False))
    x = torch.randn(2, 4, 8)
    y, stats = moe(x)
    assert y.shape == x.shape
    assert stats.tokens_per_expert.sum().item() == 2 * 4 * cfg.top_k
    assert stats.aux_loss.ndim == 0


def test_moe_matches_dense_loop_oracle():
    """Vectorised pack/combine equals a token-by-token evaluation of the same experts."""
    torch.manual_seed(0)
    cfg = tiny_model_cfg(d_model=8, ffn_in=16, num_experts=3, top_k=2)
    moe = MoE(cfg, full_spec(cfg))
    x = torch.randn(1, 5, 8)
    y, _ = moe(x)
    flat = x.reshape(-1, 8)
    gates, top_e, _ = ref.router_topk(flat, moe.router.weight, 2)
    want = torch.zeros_like(flat)
    ex = moe.experts
    for t in range(flat.shape[0]):
        for j in range(2):
            e = top_e[t, j].item()
            h = torch.nn.functional.silu(flat[t] @ ex.W_gate[e]) * (flat[t] @ ex.W_val[e])
            want[t] += gates[t, j] * (h @ ex.W_out[e])
    torch.testing.assert_close(y.reshape(-1, 8), want, rtol=1e-5, atol=1e-6)


def test_aux_loss_formula():
    cfg = tiny_model_cfg(num_experts=4)
    counts = torch.tensor([4, 0, 2, 2])
    probs = torch.tensor([[0.7, 0.1, 0.1, 0.1], [0.1, 0.1, 0.4, 0.4]])
    stats = MoELayerStats(counts, probs, cfg)
    frac = counts.float() / 8
    want = 0.01 * 4 * (frac * probs.mean(0)).sum()
    torch.testing.assert_close(stats.aux_loss, want)
    # a pre-averaged [E] vector is accepted too
    torch.testing.assert_close(MoELayerStats(counts, probs.mean(0), cfg).aux_loss, want)


def test_model_active_parameter_count_uses_top_k_experts():
    cfg = tiny_model_cfg(vocab_size=1, d_head=1, n_heads=1, n_layers=1, max_seq_len=1, d_model=8, ffn_in=16)
    spec = full_spec(cfg, has_token_embed=False, has_pos_embed=False, has_unembed_head=False)
    model = NanoTitanModel(cfg, spec)
    attention = 4 * cfg.d_model * cfg.d_head * cfg.n_heads
    norms = 4 * cfg.d_model
    router = cfg.d_model * cfg.num_experts
    expert = 3 * cfg.d_model * cfg.ffn_in
    assert model.total_parameter_count() == sum(p.numel() for p in model.parameters())
    assert model.active_parameter_count() == cfg.n_layers * (attention + norms + router + cfg.top_k * expert)


def test_parameter_sync_groups_handle_pipeline_boundary_blocks():
    cfg = tiny_model_cfg()
    model = NanoTitanModel(cfg, full_spec(cfg))
    groups = model.parameter_sync_groups()
    shared = {id(p) for p in groups["shared"]}
    expert = {id(p) for p in groups["expert"]}
    assert shared and expert and shared.isdisjoint(expert)
    assert shared | expert == {id(p) for p in model.parameters() if p.requires_grad}


def test_state_dict_layout_matches_reference_keys():
    cfg = tiny_model_cfg(n_layers=1)
    keys = list(NanoTitanModel(cfg, full_spec(cfg)).state_dict())
    assert keys == [
        "blocks.0.token_embed.token_embed.weight", "blocks.0.position_embed.pos_embed",
        "blocks.1.attn.W_Q", "blocks.1.attn.W_K", "blocks.1.attn.W_V", "blocks.1.attn.W_O",
        "blocks.1.attn.mask", "blocks.1.ffn.experts.W_gate", "blocks.1.ffn.experts.W_val",
        "blocks.1.ffn.experts.W_out", "blocks.1.ffn.router.weight", "blocks.1.attn_norm.gamma",
        "blocks.1.attn_norm.beta", "blocks.1.ffn_norm.gamma", "blocks.1.ffn_norm.beta",
        "blocks.2.unembed.weight",
    ]


def test_forward_matches_explicit_reference_math():
    """The op-based forward equals the reference's formulation (S x S masked softmax, separate
    residual adds, F.cross_entropy on logits)."""
    torch.manual_seed(1)
    cfg = tiny_model_cfg(num_experts=1, top_k=1)
    model = NanoTitanModel(cfg, full_spec(cfg))
    ids = torch.randint(0, cfg.vocab_size, (2, cfg.max_seq_len))
    tgt = torch.randint(0, cfg.vocab_size, (2, cfg.max_seq_len))
    logits, _ = model(ids)
    loss, _ = model.forward_loss(ids, tgt)

    emb = model.blocks[0]
    x = emb.token_embed.token_embed.weight[ids] + emb.position_embed.pos_embed[None]
    for layer in model.blocks[1:-1]:
        def ln(v, n):
            mu = v.mean(-1, keepdim=True)
            var = v.var(-1, keepdim=True, correction=0)
            return (v - mu) / torch.sqrt(var + 1e-8) * n.gamma + n.beta
        h = ln(x, layer.attn_norm)
        a = layer.attn
        q, k, v = (
            (h @ w).view(2, -1, cfg.n_heads, cfg.d_head).transpose(1, 2) for w in (a.W_Q, a.W_K, a.W_V)
        )
        s = (q @ k.transpose(-1, -2)) / cfg.d_head**0.5
        s = s.masked_fill(a.mask[..., : s.shape[-2], : s.shape[-1]] == 0, float("-inf"))
        ctx = (s.softmax(-1) @ v).transpose(1, 2).reshape(2, -1, cfg.n_heads * cfg.d_head)
        x = ctx @ a.W_O + x
        h = ln(x, layer.ffn_norm)
        ex = layer.ffn.experts
        x = (torch.nn.functional.silu(h @ ex.W_gate[0]) * (h @ ex.W_val[0])) @ ex.W_out[0] + x
    want = x @ model.blocks[-1].unembed.weight.t()
    torch.testing.assert_close(logits, want, rtol=1e-4, atol=1e-5)
    want_loss = torch.nn.functional.cross_entropy(want.view(-1, cfg.vocab_size), tgt.view(-1))
    torch.testing.assert_close(loss, want_loss, rtol=1e-5, atol=1e-6)


def test_cuda_backend_on_cpu_raises_clearly():
    cfg = tiny_model_cfg(moe_backend="cuda")
    moe = MoE(cfg, full_spec(cfg))
    with pytest.raises(RuntimeError, match="GPU"):
        moe(torch.randn(1, 2, cfg.d_model))
