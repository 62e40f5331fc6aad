from nanotitan_b200.models.feed_fwd import FFN, ExpertFFN, MoE  # noqa: F401
