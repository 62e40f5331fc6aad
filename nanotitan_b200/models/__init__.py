from nanotitan_b200.models.model import NanoTitanModel
from nanotitan_b200.models.utils import ModelShardSpec, MoELayerStats, get_model_shard_specs

__all__ = ["NanoTitanModel", "ModelShardSpec", "MoELayerStats", "get_model_shard_specs"]
