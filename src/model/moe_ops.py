from nanotitan_b200.models.moe_ops import (  # noqa: F401
    CombineTokensFN, GroupedGEMM_FN, PackTokensFN, TorchBackendAll2ALL, combine_tokens_fn, grouped_gemm_fn, pack_tokens_fn,
    torch_backend_all_to_all,
)
