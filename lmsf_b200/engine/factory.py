"""From a model folder to a model on the device (the role of ModelFactory::load_model,
core/src/model_executor/models/model_factory.rs:116-267)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import models  # noqa: F401  (registers the architectures)
from ..config.engine_config import canonical_dtype
from ..config.registry import load_model_config
from ..parts.decoder import DecoderModel
from ..weights.loader import load_weights
from ..weights.random_init import init_random_on_device

TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def resolve_dtype(requested: Optional[str], config) -> torch.dtype:
    """--dtype wins; else the config's torch_dtype (float16 checkpoints run as bfloat16)."""
    name = canonical_dtype(requested) if requested else None
    if name is None:
        td = getattr(config, "torch_dtype", "bfloat16")
        name = "float32" if td in ("float32", "float") else "bfloat16"
    return TORCH_DTYPES[name]


def build_model(model_dir: str, dtype: Optional[str] = None, device="cuda:0", load_format: str = "auto",
                seed: int = 0) -> Tuple[DecoderModel, object, torch.dtype]:
    """load_format "auto": weights from the folder's safetensors; "dummy": random weights made on the
    device from config.json alone."""
    if not torch.cuda.is_available():
        raise RuntimeError("lmsf_b200 needs a CUDA device (sm_100a); none is visible and there is no CPU path")
    device = torch.device(device)
    arch, cfg = load_model_config(model_dir)
    tdt = resolve_dtype(dtype, cfg)
    model = DecoderModel(arch.build_spec(cfg))
    if load_format == "dummy":
        init_random_on_device(model, seed, tdt, device)
    elif load_format == "auto":
        load_weights(model, model_dir, tdt, device)
    else:
        raise ValueError(f"unknown load_format {load_format!r} (auto, dummy)")
    model.prepare(tdt, device)
    return model, cfg, tdt
