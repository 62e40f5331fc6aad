"""The autoregressive transformer LM whose every FFN is an MoE layer.

Module tree, parameter names, shapes, buffers and initialisers follow the reference
(src/model/model.py:19-269) so `state_dict()` is interchangeable and the same seed
gives the same initial weights: pre-LN layers `x = attn(ln(x)) + x; x = moe(ln(x)) + x`,
hand-rolled LayerNorm (biased variance, eps 1e-8), fixed sinusoidal positions held as
a buffer, four bias-free `[d, H*Dh]` attention matrices, an untied bias-free unembed
and no final norm.  The math itself runs through `nanotitan_b200.ops`: on a GPU that
means the fused sm_100a kernels (flash attention instead of an S x S score tensor,
residual adds folded into GEMM epilogues, unembed fused with the loss).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from nanotitan_b200 import ops
from nanotitan_b200.models.feed_fwd import MoE
from nanotitan_b200.models.utils import ModelShardSpec, MoELayerStats
from nanotitan_b200.utils import resolve_dtype


def _parameter_count(module: nn.Module) -> int:
    return sum(p.numel() for p in module.parameters())


class TokenEmbed(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.token_embed = nn.Embedding(cfg.vocab_size, cfg.d_model, dtype=resolve_dtype(cfg.dtype))

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        return self.token_embed(input_ids)

    def project(self, hidden_states: torch.Tensor) -> torch.Tensor:
        """Tied-unembedding helper: hidden [B,S,d] -> logits [B,S,V] with the embedding matrix."""
        return hidden_states @ self.token_embed.weight.t()


class PositionEmbed(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.max_seq_len = cfg.max_seq_len
        self.register_buffer("pos_embed", self._sinusoids(cfg))

    @staticmethod
    def _sinusoids(cfg) -> torch.Tensor:
        pos = torch.arange(cfg.max_seq_len).unsqueeze(1)
        freq = torch.exp(torch.arange(0, cfg.d_model, 2) * (-math.log(10000.0) / cfg.d_model))
        table = torch.zeros(cfg.max_seq_len, cfg.d_model, dtype=resolve_dtype(cfg.dtype))
        table[:, 0::2] = torch.sin(pos * freq)
        table[:, 1::2] = torch.cos(pos * freq)
        return table

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        seq_len = x.shape[1]
        if seq_len > self.max_seq_len:
            raise ValueError(
                f"Sequence length {seq_len} exceeds configured max_seq_len={self.max_seq_len}"
            )
        return self.pos_embed[:seq_len].unsqueeze(0)


class EmbeddingBlock(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.cfg = cfg
        self.token_embed = TokenEmbed(cfg)
        self.position_embed = PositionEmbed(cfg)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.token_embed(x) + self.position_embed(x)

    def active_parameter_count(self) -> int:
        return _parameter_count(self.token_embed)


class Unembed(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.cfg = cfg
        self.unembed = nn.Linear(cfg.d_model, cfg.vocab_size, bias=False, dtype=resolve_dtype(cfg.dtype))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.unembed(x)

    def loss(self, x: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """Mean next-token cross-entropy without materialising fp32 logits."""
        return ops.linear_cross_entropy(
            x.reshape(-1, x.shape[-1]), self.unembed.weight, targets.reshape(-1)
        )

    def active_parameter_count(self) -> int:
        return _parameter_count(self.unembed)


class LayerNorm(nn.Module):
    EPS = 1e-8

    def __init__(self, cfg):
        super().__init__()
        self.d_model = cfg.d_model
        dtype = resolve_dtype(cfg.dtype)
        self.gamma = nn.Parameter(torch.ones(self.d_model, dtype=dtype))
        self.beta = nn.Parameter(torch.zeros(self.d_model, dtype=dtype))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.layer_norm(x, self.gamma, self.beta, self.EPS)

    def forward_residual(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """(norm(x), x) with x routed through the norm's autograd node (see `ops.layer_norm_residual`)."""
        return ops.layer_norm_residual(x, self.gamma, self.beta, self.EPS)


class MultiHeadAttention(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.cfg = cfg
        dtype = resolve_dtype(cfg.dtype)
        inner = cfg.d_head * cfg.n_heads
        self.W_Q = nn.Parameter(torch.empty(cfg.d_model, inner, dtype=dtype))
        self.W_K = nn.Parameter(torch.empty(cfg.d_model, inner, dtype=dtype))
        self.W_V = nn.Parameter(torch.empty(cfg.d_model, inner, dtype=dtype))
        self.W_O = nn.Parameter(torch.empty(inner, cfg.d_model, dtype=dtype))
        for w in (self.W_Q, self.W_K, self.W_V, self.W_O):
            nn.init.xavier_uniform_(w)
        # Kept only so the state dict carries the same keys as the reference; the causal
        # structure is computed from indices inside the attention kernel.
        mask = torch.tril(torch.ones(cfg.max_seq_len, cfg.max_seq_len, dtype=torch.bool))
        self.register_buffer("mask", mask[None, None, :, :])

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        batch, seq, d_model = x.shape
        heads, d_head = self.cfg.n_heads, self.cfg.d_head
        ctx = ops.qkv_attention(x, self.W_Q, self.W_K, self.W_V, heads, d_head, 1.0 / math.sqrt(d_head))
        res = None if residual is None else residual.reshape(-1, d_model)
        out = ops.linear(ctx.reshape(-1, heads * d_head), self.W_O, res)
        return out.view(batch, seq, d_model)


class TransformerLayer(nn.Module):
    def __init__(self, cfg, spec: ModelShardSpec):
        super().__init__()
        self.cfg = cfg
        self.attn = MultiHeadAttention(cfg)
        self.ffn = MoE(cfg, spec)
        self.attn_norm = LayerNorm(cfg)
        self.ffn_norm = LayerNorm(cfg)

    def active_parameter_count(self) -> int:
        return (
            _parameter_count(self.attn)
            + _parameter_count(self.attn_norm)
            + _parameter_count(self.ffn_norm)
            + self.ffn.active_parameter_count()
        )

    def forward(self, x: torch.Tensor) -> tuple[torch.Tensor, MoELayerStats]:
        h, x = self.attn_norm.forward_residual(x)
        x = self.attn(h, residual=x)
        h, x = self.ffn_norm.forward_residual(x)
        x, layer_stats = self.ffn(h, residual=x)
        return x, layer_stats


class NanoTitanModel(nn.Module):
    """`blocks` = [EmbeddingBlock?] + layers[layer_start:layer_end] + [Unembed?] for one PP stage."""

    def __init__(self, cfg, spec: ModelShardSpec):
        super().__init__()
        self.cfg = cfg
        self.spec = spec
        self.blocks = nn.ModuleList()
        if spec.has_token_embed and spec.has_pos_embed:
            self.blocks.append(EmbeddingBlock(cfg))
        for _ in range(spec.layer_start, spec.layer_end):
            self.blocks.append(TransformerLayer(cfg, spec))
        if spec.has_unembed_head:
            self.blocks.append(Unembed(cfg))

    @classmethod
    def from_specs(cls, cfg, spec: ModelShardSpec) -> "NanoTitanModel":
        return cls(cfg, spec)

    def total_parameter_count(self) -> int:
        return _parameter_count(self)

    def active_parameter_count(self):
        return sum(block.active_parameter_count() for block in self.blocks)

    def parameter_sync_groups(self) -> dict:
        """Split trainable parameters into expert shards (reduced over dp ranks) and the
        rest (reduced over dp*ep ranks)."""
        expert = tuple(
            p
            for block in self.blocks
            if isinstance(block, TransformerLayer)
            for p in block.ffn.experts.parameters()
            if p.requires_grad
        )
        expert_ids = {id(p) for p in expert}
        shared = tuple(
            p for p in self.parameters() if p.requires_grad and id(p) not in expert_ids
        )
        return {"shared": shared, "expert": expert}

    def forward(self, x: torch.Tensor) -> tuple[torch.Tensor, list[MoELayerStats]]:
        stats: list[MoELayerStats] = []
        for block in self.blocks:
            if isinstance(block, TransformerLayer):
                x, layer_stats = block(x)
                stats.append(layer_stats)
            else:
                x = block(x)
        return x, stats

    def forward_loss(self, x: torch.Tensor, targets: torch.Tensor):
        """Last-stage forward that ends in the fused unembed + cross-entropy.

        Returns (loss, stats).  Equivalent to `F.cross_entropy(self(x)[0], targets)`.
        """
        assert self.spec.has_unembed_head, "forward_loss needs the unembed head on this stage"
        stats: list[MoELayerStats] = []
        for block in self.blocks:
            if isinstance(block, TransformerLayer):
                x, layer_stats = block(x)
                stats.append(layer_stats)
            elif isinstance(block, Unembed):
                return block.loss(x, targets), stats
            else:
                x = block(x)
        raise AssertionError("unreachable")
