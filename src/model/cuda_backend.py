from nanotitan_b200.models.cuda_backend import CUDAMoEBackend  # noqa: F401
