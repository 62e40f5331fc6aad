from nanotitan_b200.models.utils import ModelShardSpec, MoELayerStats, get_layer_bounds, get_logical_expert_bounds, get_model_shard_specs  # noqa: F401
