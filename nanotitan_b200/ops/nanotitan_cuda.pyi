"""Type stub of the `nanotitan_cuda` extension, generated from the signatures pybind11 records
(`python -m nanotitan_b200.ops.ext --stub` rewrites it).  The module itself is built from nanotitan_b200/csrc
and loaded by `nanotitan_b200.ops.ext.get_ext()`."""
from __future__ import annotations

import torch

Tensor = torch.Tensor

class TokenWindowLoader:
    def __init__(self, path: str, seq_len: int, batch: int, depth: int, threads: int) -> None: ...
    batches_in_epoch: int
    def next(self, timeout_ms: int) -> int: ...
    num_sequences: int
    def release(self, arg0: int) -> None: ...
    def set_ring(self, arg0: Tensor, arg1: int) -> None: ...
    slot_elements: int
    def start(self, arg0: Tensor) -> None: ...
    def stop(self) -> None: ...

def adamw_step(param: Tensor, grad: Tensor, master: Tensor, m: Tensor, v: Tensor, step: int, lr: float, beta1: float, beta2: float, eps: float, wd: float, grad_scale: float, want_sq: bool, bc_dev: Tensor | None = None) -> Tensor:
    ...

def assign_slots(arg0: Tensor, arg1: Tensor) -> list[Tensor]:
    ...

def bounded_wait_probe(arg0: float) -> int:
    """Let a bounded device wait run out; returns the number of threads that gave up"""

def bucket_allreduce(arg0: Tensor, arg1: int, arg2: Tensor, arg3: int, arg4: Tensor, arg5: Tensor | None, arg6: Tensor | None, arg7: Tensor | None, arg8: Tensor, arg9: Tensor, arg10: Tensor, arg11: int, arg12: int, arg13: int, arg14: Tensor, arg15: int, arg16: Tensor | None, arg17: float, arg18: float, arg19: float, arg20: float, arg21: float, arg22: int, arg23: float) -> None:
    """Fused bucket all-reduce (+ AdamW) over peer / multicast memory"""

def bwd_grouped_gemm_dW_kernel(arg0: Tensor, arg1: Tensor, arg2: Tensor) -> Tensor:
    ...

def bwd_grouped_gemm_dX_kernel(arg0: Tensor, arg1: Tensor, arg2: Tensor) -> Tensor:
    ...

def combine_bwd(arg0: Tensor, arg1: Tensor, arg2: Tensor, arg3: Tensor) -> list[Tensor]:
    ...

def combine_fwd(arg0: Tensor, arg1: Tensor, arg2: Tensor, arg3: Tensor | None, arg4: int, arg5: Tensor | None, arg6: bool) -> Tensor:
    ...

def combine_kernel_backward(arg0: Tensor, arg1: Tensor, arg2: Tensor, arg3: Tensor, arg4: int) -> list[Tensor]:
    """Backward of combine"""

def combine_tokens_kernel(arg0: Tensor, arg1: Tensor, arg2: Tensor, arg3: int, arg4: int) -> Tensor:
    """Gate-weighted combine of expert rows (fp32 out)"""

def copy_rows_prefix(arg0: Tensor, arg1: Tensor, arg2: Tensor) -> None:
    ...

def copy_scalar(arg0: Tensor, arg1: Tensor, arg2: int) -> None:
    """Element-wise copy of n elements"""

def copy_vector(arg0: Tensor, arg1: Tensor) -> None:
    """16-byte vector copy"""

def count_expert_kernel(arg0: Tensor, arg1: Tensor, arg2: int, arg3: int) -> Tensor:
    """Histogram of expert ids"""

def cross_entropy_fwd_bwd(arg0: Tensor, arg1: Tensor, arg2: int, arg3: float, arg4: bool) -> Tensor:
    ...

def ep_allgather_counts(arg0: Tensor, arg1: Tensor, arg2: Tensor, arg3: Tensor, arg4: int, arg5: int, arg6: Tensor, arg7: int, arg8: float) -> None:
    """All-gather per-expert counts through peer stores"""

def ep_dispatch(arg0: Tensor, arg1: Tensor, arg2: Tensor, arg3: Tensor, arg4: Tensor, arg5: Tensor, arg6: Tensor, arg7: Tensor, arg8: Tensor, arg9: int, arg10: int, arg11: Tensor, arg12: Tensor, arg13: Tensor, arg14: int, arg15: int, arg16: Tensor, arg17: float, arg18: int) -> list[Tensor]:
    """Fused count exchange + pack + push of token rows into the expert ranks' staging buffers"""

def ep_push_rows(arg0: Tensor, arg1: Tensor, arg2: int, arg3: Tensor, arg4: int, arg5: int, arg6: bool, arg7: Tensor, arg8: Tensor, arg9: Tensor, arg10: int, arg11: int, arg12: Tensor, arg13: int, arg14: float, arg15: int) -> None:
    """Push rows into peers' staging buffers (expert-parallel dispatch / return)"""

def flash_bwd(dout: Tensor, q: Tensor, k: Tensor, v: Tensor, out: Tensor, lse: Tensor, scale: float, grads: list[Tensor] = []) -> list[Tensor]:
    """Causal flash attention backward -> (dq, dk, dv)"""

def flash_fwd(arg0: Tensor, arg1: Tensor, arg2: Tensor, arg3: float) -> list[Tensor]:
    """Causal flash attention forward -> (out, lse)"""

def gemm_kernel(A: Tensor, B: Tensor, implementation: str = 'tiled') -> Tensor:
    ...

def gemm_tc(A: Tensor, a_mn: bool, Bs: list[Tensor], b_mn: bool, b_split: int, Cs: list[Tensor], mode: int = 0, offsets: Tensor | None = None, epilogue: int = 0, accumulate: bool = False, aux: Tensor | None = None, aux_out: Tensor | None = None, force_bn: int = 0) -> None:
    ...

def grouped_gemm_kernel(arg0: Tensor, arg1: Tensor, arg2: Tensor) -> Tensor:
    """out[r] = X[r] . W[e(r)]"""

def launch_count() -> int:
    """Kernels of this library launched by this process"""

def launch_counts() -> dict[str, int]:
    """Kernel launches of this process by host entry point"""

def layer_norm_bwd(dy: Tensor, x: Tensor, gamma: Tensor, mean: Tensor, rstd: Tensor, dres: Tensor | None = None, dgamma_out: Tensor | None = None, dbeta_out: Tensor | None = None) -> list[Tensor]:
    ...

def layer_norm_fwd(arg0: Tensor, arg1: Tensor, arg2: Tensor, arg3: float) -> list[Tensor]:
    ...

def naive_gemm_kernel(arg0: Tensor, arg1: Tensor) -> Tensor:
    ...

def pack_bwd(arg0: Tensor, arg1: Tensor, arg2: Tensor | None, arg3: int) -> Tensor:
    ...

def pack_fwd(arg0: Tensor, arg1: Tensor, arg2: Tensor, arg3: Tensor) -> list[Tensor]:
    ...

def pack_kernel_backward(arg0: Tensor, arg1: Tensor, arg2: Tensor, arg3: Tensor, arg4: Tensor) -> list[Tensor]:
    """Backward of pack"""

def pack_tokens_kernel(arg0: Tensor, arg1: Tensor, arg2: Tensor, arg3: Tensor) -> list[Tensor]:
    """Pack token rows into expert-major order"""

def peer_copy_scalar(arg0: Tensor, arg1: Tensor) -> None:
    """GPU-to-GPU copy over NVLink"""

def random_op(arg0: Tensor, arg1: int) -> Tensor:
    """Zero vector of length x with t's options"""

def read_status(clear: bool = True) -> list[int]:
    """[code, kernel, detail, count] of the device status word"""

def router_bwd(arg0: Tensor, arg1: Tensor, arg2: Tensor, arg3: Tensor | None, arg4: Tensor | None, arg5: Tensor | None, arg6: Tensor) -> list[Tensor]:
    ...

def router_from_logits(arg0: Tensor, arg1: int) -> list[Tensor]:
    """router_topk's outputs from fp32 logits [T, E]"""

def router_topk(arg0: Tensor, arg1: Tensor, arg2: int) -> list[Tensor]:
    ...

def status_word_tensor() -> Tensor:
    ...

def symm_heap_alloc(heap: int, bytes: int, multicast: bool) -> tuple[Tensor, list[int], int, int]:
    """Collective allocation -> (byte tensor over this rank's piece, every rank's address, multicast address, id)"""

def symm_heap_close(arg0: int) -> None:
    ...

def symm_heap_free(arg0: int, arg1: int) -> None:
    ...

def symm_heap_open(job: str, rank: int, world: int, device: int, timeout_ms: int) -> int:
    """Open this rank's end of a symmetric heap (collective over the ranks of one machine)"""

def tiled_gemm_kernel(arg0: Tensor, arg1: Tensor) -> Tensor:
    ...

