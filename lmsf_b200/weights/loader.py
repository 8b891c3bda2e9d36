"""Loads the weights of a built model from a model folder, by tensor name.

Every part declares the tensors it needs (`Part.weight_specs`) and the model description says
under which names they are stored (`PartSpec.weights`).  All names and shapes are checked before
anything is copied, and every fault is reported in ONE error: missing tensors, tensors of the
wrong shape, and tensors of the file that no part asked for.  The reference reports the first
missing name or shape mismatch it meets (core/src/model_executor/layers/linear.rs:285-290,
:471-476, :698-703).

Floating-point tensors are converted to the run dtype on load (the reference does the same,
core/src/model_executor/models/model_factory.rs:133-139), except those whose part asks to keep a
32-bit original (norm weights); integer tensors become int32.
"""
from __future__ import annotations

import re
from typing import Dict, List, Tuple

import torch

from ..parts.base import WeightSpec
from .safetensors_io import TensorEntry, open_model_tensors


class WeightError(ValueError):
    def __init__(self, missing, unexpected, wrong_shape, model_dir=""):
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)
        lines = [f"the weights in {model_dir!r} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: expected {tuple(e)}, found {tuple(f)}" for n, e, f in self.wrong_shape))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        super().__init__("\n".join(lines))


def _names(v) -> List[str]:
    return [v] if isinstance(v, str) else list(v)


def collect_requirements(model) -> List[Tuple[object, str, WeightSpec, List[str]]]:
    req = []
    for part, pspec in model.parts_with_specs():
        for logical, wspec in part.weight_specs().items():
            if logical not in pspec.weights:
                raise KeyError(f"part {pspec.kind!r} needs a weight {logical!r} that its description does not name")
            names = _names(pspec.weights[logical])
            if len(names) != len(wspec.shapes):
                raise KeyError(f"part {pspec.kind!r}: weight {logical!r} is made of {len(wspec.shapes)} tensors, "
                               f"{len(names)} names given")
            req.append((part, logical, wspec, names))
    return req


def check_tensors(model, entries: Dict[str, TensorEntry], model_dir: str = "") -> None:
    missing, wrong, used = [], [], set()
    for _, _, wspec, names in collect_requirements(model):
        for name, shape in zip(names, wspec.shapes):
            used.add(name)
            e = entries.get(name)
            if e is None:
                if name not in missing:
                    missing.append(name)
            elif tuple(e.shape) != tuple(shape):
                wrong.append((name, shape, e.shape))
    ignored = [re.compile(p) for p in model.spec.ignored_weights]
    unexpected = sorted(n for n in entries if n not in used and not any(p.search(n) for p in ignored))
    if missing or wrong or unexpected:
        raise WeightError(missing, unexpected, wrong, model_dir)


def target_dtype(stored: torch.dtype, run_dtype: torch.dtype, keep_fp32: bool) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if keep_fp32 and stored in (torch.float32, torch.float64):
        return torch.float32
    return run_dtype


def load_weights(model, model_dir: str, dtype: torch.dtype, device) -> None:
    entries = open_model_tensors(model_dir)
    check_tensors(model, entries, model_dir)
    done: Dict[Tuple[Tuple[str, ...], torch.dtype], torch.Tensor] = {}
    per_part: Dict[int, Dict[str, torch.Tensor]] = {}
    parts = {}
    for part, logical, wspec, names in collect_requirements(model):
        tdt = target_dtype(entries[names[0]].dtype, dtype, wspec.keep_fp32)
        key = (tuple(names), tdt)
        t = done.get(key)
        if t is None:
            pieces = [entries[n].load().to(device=device, dtype=tdt) for n in names]
            t = pieces[0].contiguous() if len(pieces) == 1 else torch.cat(pieces, dim=0)
            done[key] = t                      # tied weights share one tensor
        per_part.setdefault(id(part), {})[logical] = t
        parts[id(part)] = part
    for pid, tensors in per_part.items():
        parts[pid].set_weights(tensors)
