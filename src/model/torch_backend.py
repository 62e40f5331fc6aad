from nanotitan_b200.models.torch_backend import TorchMoEBackend  # noqa: F401
