"""TOML -> pydantic configuration tree.

The key names, defaults and validators follow the reference schema
(src/config.py:19-153) so every reference TOML loads unchanged; unknown keys are
rejected everywhere.  Two optional tables are additions of this framework:
``[checkpoint]`` (sharded save / resume) and ``[fault]`` (process-group timeout,
heartbeat), and ``runtime.cuda_graph`` is an added key.  Tables appear below in the
order a config file usually lists them; every key says what it controls.
"""
from __future__ import annotations

import tomllib
from pathlib import Path
from typing import Any, Literal

from pydantic import BaseModel, ConfigDict, Field, NonNegativeInt, PositiveInt, model_validator

DTypeName = Literal["float16", "float32", "bfloat16"]


class _Strict(BaseModel):
    """Base for every table: extra keys are an error, torch dtypes may be assigned later."""

    model_config = ConfigDict(extra="forbid", arbitrary_types_allowed=True)


# --------------------------------------------------------------------------- [model]
class TokenEmbeddingConfig(_Strict):
    """[model.token_embedding]: no keys yet; the table may be present and empty."""


class PositionalEmbeddingConfig(_Strict):
    """[model.positional_embedding]: no keys yet (positions are fixed sinusoids)."""


class ModelConfig(_Strict):
    vocab_size: PositiveInt        # rows of the embedding and of the (untied) unembedding
    d_model: PositiveInt           # residual width
    d_head: PositiveInt            # per-head width; n_heads * d_head is the attention width
    n_heads: PositiveInt
    n_layers: PositiveInt          # transformer layers, each attention + MoE feed-forward
    max_seq_len: PositiveInt       # tokens per sample and length of the position table
    ffn_in: PositiveInt            # hidden width of one expert
    num_experts: PositiveInt       # experts per layer; 1 = a dense SwiGLU feed-forward
    top_k: PositiveInt             # experts per token
    token_embedding: TokenEmbeddingConfig = Field(default_factory=TokenEmbeddingConfig)
    positional_embedding: PositionalEmbeddingConfig = Field(default_factory=PositionalEmbeddingConfig)
    moe_backend: str = "torch"     # "torch" (portable modules) or "cuda" (this library's kernels)
    dtype: DTypeName = "float32"   # parameter / activation dtype
    moe_router_dtype: DTypeName = "float32"
    router_alpha: float            # weight of the load-balancing loss

    @model_validator(mode="after")
    def _even_width(self) -> "ModelConfig":
        if self.d_model % 2 != 0:
            raise ValueError("model.d_model must be even when using sinusoidal positional embeddings")
        return self


# --------------------------------------------------------------------------- [trainer] [data] [optim]
class TrainerConfig(_Strict):
    device_id: NonNegativeInt          # kept for the reference's files; ranks take LOCAL_RANK
    eval_every_step: int               # -1: never; 0: validate after every step; n: after every n-th step
    per_device_batch_size: PositiveInt
    seed: NonNegativeInt               # the reference insists on seed > 0 (src/config.py:121); 0 is a valid seed here


class DataConfig(_Strict):
    num_workers: PositiveInt           # loader threads (packed token files) or DataLoader workers
    train_tokens_path: str             # flat uint16 token stream
    val_tokens_path: str


class OptimizerConfig(_Strict):
    type: str                          # "adam": AdamW, weight decay 0.1
    lr: float


# --------------------------------------------------------------------------- [runtime]
class RuntimeConfig(_Strict):
    """Parallel layout of one run (reference: src/config.py:42-57)."""

    name: str
    reducer: str = "v0"                # informational only, never branched on
    bucket_size: int = 25              # MiB per gradient bucket
    num_microbatches: int = 1          # GPipe microbatches per step
    dp_size: int = 1
    pp_size: int = 1
    ep_size: int = 1
    num_expert: PositiveInt = 1        # mirrored from model.num_experts by AppConfig
    # Capture the whole optimizer step in a CUDA graph after two ordinary steps (GPU, pp_size 1);
    # the environment variable NT_CUDA_GRAPH=0/1 overrides it.  No counterpart in the reference.
    cuda_graph: bool = True


# --------------------------------------------------------------------------- optional tables
class ProfilerConfig(_Strict):
    enabled: bool = False
    wait_steps: NonNegativeInt = 2     # idle steps before the warm-up
    warmup_steps: NonNegativeInt = 2   # traced but discarded
    active_steps: NonNegativeInt = 6   # recorded
    record_shapes: bool = True
    profile_memory: bool = True
    with_stack: bool = False
    with_flops: bool = False

    @model_validator(mode="after")
    def _active_steps_positive(self) -> "ProfilerConfig":
        if self.enabled and self.active_steps == 0:
            raise ValueError("profiler.active_steps must be positive when profiler.enabled=true")
        return self


class HardwareConfig(_Strict):
    peak_flops_tflops_per_gpu: float = 0.0   # > 0 turns on the MFU metric


class CheckpointConfig(_Strict):
    """Sharded checkpointing (no counterpart in the reference, which never saves)."""

    dir: str = ""
    every_steps: NonNegativeInt = 0    # 0 disables periodic saves
    resume: bool = False
    # also store the optimizer state per parameter, so that `consolidate --with-optimizer` + `--init-from` can
    # continue the run on another dp x pp x ep layout (costs a gather of the sharded state at every save)
    portable_optimizer: bool = False
    # copy the state to host memory, then serialise and write it from a background thread while training goes on
    async_save: bool = False


class FaultConfig(_Strict):
    """Host-side failure detection (no counterpart in the reference)."""

    pg_timeout_s: float = 600.0        # process-group timeout: ends a collective a lost peer never joins
    heartbeat_dir: str = ""            # "" disables heartbeats
    heartbeat_stale_s: float = 120.0   # a peer silent for longer counts as lost


# --------------------------------------------------------------------------- the file
class AppConfig(_Strict):
    run_name: str
    max_steps: PositiveInt
    model: ModelConfig
    trainer: TrainerConfig
    data: DataConfig
    optim: OptimizerConfig
    runtime: RuntimeConfig
    profiler: ProfilerConfig = Field(default_factory=ProfilerConfig)
    hardware: HardwareConfig = Field(default_factory=HardwareConfig)
    checkpoint: CheckpointConfig = Field(default_factory=CheckpointConfig)
    fault: FaultConfig = Field(default_factory=FaultConfig)
    track_backward_time: bool = False  # accepted for the reference's files; time/backward_time is always reported

    @model_validator(mode="before")
    @classmethod
    def _mirror_expert_count(cls, raw: Any) -> Any:
        """runtime.num_expert always equals model.num_experts (src/config.py:138-153)."""
        if not isinstance(raw, dict):
            return raw
        model, runtime = raw.get("model"), raw.get("runtime")
        if not isinstance(model, dict) or not isinstance(runtime, dict):
            return raw
        out = dict(raw)
        out["runtime"] = {**runtime, "num_expert": model.get("num_experts")}
        return out


def resolve_config_path(path: str | Path) -> Path:
    """Return ``path`` if it exists, else ``configs/<path>`` (src/config.py:156-165)."""
    direct = Path(path)
    if direct.exists():
        return direct
    fallback = Path("configs") / direct
    if fallback.exists():
        return fallback
    raise FileNotFoundError(f"Could not find config file at '{path}' or '{fallback}'")


def load_config(path: str | Path) -> AppConfig:
    with resolve_config_path(path).open("rb") as fh:
        return AppConfig.model_validate(tomllib.load(fh))
