"""Random weights: writes a model folder (config.json, model.safetensors) from a configuration and a seed.

The reference has no such mode.  Every matrix is i.i.d. N(0, std^2), every norm weight is 1; the
values of a tensor depend on (seed, tensor name) only, not on the order of generation.  Values are
drawn in float32 and rounded to the stored dtype.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, List, Tuple

import torch

from ..config.registry import resolve_architecture
from ..parts.decoder import DecoderModel
from .loader import collect_requirements
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(seed: int, name: str, shape, dtype: torch.dtype, std: float, is_norm: bool) -> torch.Tensor:
    if is_norm:
        return torch.ones(shape, dtype=dtype)
    g = torch.Generator(device="cpu")
    g.manual_seed(_tensor_seed(seed, name))
    return (torch.randn(shape, generator=g, dtype=torch.float32) * std).to(dtype)


def tensor_list(model: DecoderModel) -> List[Tuple[str, Tuple[int, ...], bool]]:
    """(name, shape, is a norm-like vector) of every stored tensor of the model, once each."""
    seen, out = set(), []
    for _, _, wspec, names in collect_requirements(model):
        for name, shape in zip(names, wspec.shapes):
            if name not in seen:
                seen.add(name)
                out.append((name, tuple(shape), wspec.keep_fp32))
    return out


def write_random_model(folder: str, config: Dict[str, Any], seed: int = 0, dtype: str = "bfloat16",
                       std: float = 0.02) -> str:
    """config: the content of config.json (a dict, or a typed configuration with to_dict())."""
    cfg_dict = config.to_dict() if hasattr(config, "to_dict") else dict(config)
    arch = resolve_architecture(cfg_dict)
    typed = arch.parse_config(cfg_dict)
    model = DecoderModel(arch.build_spec(typed))
    tdt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    os.makedirs(folder, exist_ok=True)
    cfg_dict["torch_dtype"] = dtype
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg_dict, f, indent=1)
    tensors = tensor_list(model)
    info = {n: (s, is_norm) for n, s, is_norm in tensors}
    write_safetensors(os.path.join(folder, "model.safetensors"), [(n, tdt, s) for n, s, _ in tensors],
                      lambda n: random_tensor(seed, n, info[n][0], tdt, std, info[n][1]),
                      metadata={"format": "pt", "seed": str(seed)})
    return folder


def init_random_on_device(model: DecoderModel, seed: int, dtype: torch.dtype, device, std: float = 0.02) -> None:
    """Fills the model's weights on the device without a file (for measurements of large shapes, where only
    the sizes matter).  Not the same values as `write_random_model`."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    done: Dict[Tuple[str, ...], torch.Tensor] = {}
    per_part: Dict[int, Dict[str, torch.Tensor]] = {}
    parts = {}
    for part, logical, wspec, names in collect_requirements(model):
        key = tuple(names)
        t = done.get(key)
        if t is None:
            rows = sum(s[0] for s in wspec.shapes)
            shape = (rows, *wspec.shapes[0][1:])
            if wspec.keep_fp32:
                t = torch.ones(shape, dtype=dtype, device=device)
            else:
                t = torch.empty(shape, dtype=dtype, device=device)
                t.normal_(0.0, std, generator=g)
            done[key] = t
        per_part.setdefault(id(part), {})[logical] = t
        parts[id(part)] = part
    for pid, tensors in per_part.items():
        parts[pid].set_weights(tensors)
