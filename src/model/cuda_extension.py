from nanotitan_b200.models.cuda_extension import get_cuda_extension  # noqa: F401
