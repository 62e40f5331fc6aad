from nanotitan_b200.optim import setup_optimizer  # noqa: F401
