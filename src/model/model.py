from nanotitan_b200.models.model import *  # noqa: F401,F403
from nanotitan_b200.models.model import EmbeddingBlock, LayerNorm, MultiHeadAttention, NanoTitanModel, PositionEmbed, TokenEmbed, TransformerLayer, Unembed  # noqa: F401
