"""Engine-level options.

`EngineArgs` keeps the names and meanings of the reference's command-line struct
(core/src/common/config.rs:11-87) for the options that this engine has; swap space,
paddings, quantization, tp/pp and chat templates have no counterpart here.
`CacheConfig` and `SchedulerConfig` follow core/src/common/config.rs:231-314.
"""
from __future__ import annotations

import argparse
from dataclasses import dataclass
from typing import Optional

from .model_config import ConfigError

DTYPES = ("bfloat16", "float32")


def canonical_dtype(name: Optional[str]) -> Optional[str]:
    if name is None:
        return None
    n = str(name).replace("torch.", "")
    if n in ("bfloat16", "bf16"):
        return "bfloat16"
    if n in ("float32", "float", "fp32", "f32"):
        return "float32"
    raise ConfigError(f"dtype {name!r} is not supported by this engine (choose from {', '.join(DTYPES)})")


@dataclass
class CacheConfig:
    block_size: int = 16
    gpu_memory_utilization: float = 0.9
    num_gpu_blocks: Optional[int] = None     # override of the memory-derived page count

    def __post_init__(self):
        if self.block_size <= 0 or self.block_size & (self.block_size - 1):
            raise ConfigError(f"block_size must be a power of two, got {self.block_size}")
        if not (0.0 < self.gpu_memory_utilization <= 1.0):
            # core/src/common/config.rs:245-250
            raise ConfigError(f"gpu_memory_utilization must be in (0, 1], got {self.gpu_memory_utilization}")
        if self.num_gpu_blocks is not None and self.num_gpu_blocks <= 0:
            raise ConfigError("num_gpu_blocks must be positive")


@dataclass
class SchedulerConfig:
    max_num_batched_tokens: int
    max_num_seqs: int
    max_model_len: int

    @staticmethod
    def new(max_num_batched_tokens: Optional[int], max_num_seqs: int, max_model_len: int) -> "SchedulerConfig":
        # The reference defaults to max(max_model_len, 2048) because it runs a prompt in one piece
        # (core/src/common/config.rs:301-307).  Prompts are cut into portions here, so the budget of a step need
        # not cover a whole prompt: 8,192 tokens at most keep the activations of a step small whatever the
        # model's context length is.
        if max_num_batched_tokens is None:
            max_num_batched_tokens = min(max(max_model_len, 2048), 8192)
        if max_num_batched_tokens <= 0 or max_num_seqs <= 0:
            raise ConfigError("max_num_batched_tokens and max_num_seqs must be positive")
        return SchedulerConfig(max_num_batched_tokens, max_num_seqs, max_model_len)


@dataclass
class EngineArgs:
    model: str
    max_num_batched_tokens: Optional[int] = None
    max_num_seqs: int = 256
    max_model_len: Optional[int] = None
    block_size: int = 16
    seed: int = 0
    gpu_memory_utilization: float = 0.9
    dtype: Optional[str] = None
    num_gpu_blocks: Optional[int] = None
    enforce_eager: bool = False
    no_async_scheduling: bool = False

    @staticmethod
    def add_cli_args(p: argparse.ArgumentParser) -> argparse.ArgumentParser:
        p.add_argument("--model", required=True, help="path of the model folder (config.json + safetensors)")
        p.add_argument("--max-num-batched-tokens", type=int, default=None,
                       help="maximum number of batched tokens per iteration")
        p.add_argument("--max-num-seqs", type=int, default=256, help="maximum number of sequences per iteration")
        p.add_argument("--max-model-len", type=int, default=None,
                       help="model context length. If unspecified, will be automatically derived from the model")
        p.add_argument("--block-size", type=int, default=16, help="token block size")
        p.add_argument("--seed", type=int, default=0, help="random seed")
        p.add_argument("--gpu-memory-utilization", type=float, default=0.9,
                       help="the percentage of GPU memory to be used for the model executor")
        p.add_argument("--dtype", default=None, help="the datatype to use for model (bfloat16 or float32)")
        p.add_argument("--num-gpu-blocks", type=int, default=None,
                       help="number of cache pages, instead of deriving it from free memory")
        p.add_argument("--enforce-eager", action="store_true", help="never replay decode steps as CUDA graphs")
        p.add_argument("--no-async-scheduling", action="store_true",
                       help="read every batch's tokens before the next batch is scheduled")
        return p

    @staticmethod
    def from_cli_args(ns: argparse.Namespace) -> "EngineArgs":
        return EngineArgs(model=ns.model, max_num_batched_tokens=ns.max_num_batched_tokens,
                          max_num_seqs=ns.max_num_seqs, max_model_len=ns.max_model_len, block_size=ns.block_size,
                          seed=ns.seed, gpu_memory_utilization=ns.gpu_memory_utilization, dtype=ns.dtype,
                          num_gpu_blocks=ns.num_gpu_blocks, enforce_eager=ns.enforce_eager,
                          no_async_scheduling=ns.no_async_scheduling)


def resolve_max_model_len(user_value: Optional[int], derived: int) -> int:
    """core/src/common/config.rs:146-157: a user value above the model's own limit is an error."""
    if user_value is None:
        return derived
    if user_value <= 0:
        raise ConfigError("max_model_len must be positive")
    if user_value > derived:
        raise ConfigError(f"User-specified max_model_len ({user_value}) is greater than the derived max_model_len "
                          f"({derived}) in the model's config.json")
    return user_value
