"""Rotary position encoding.

The reference builds a cos/sin table once per process with base 10000 whatever config.json says
(core/src/model_executor/layers/rotary_embedding.rs:8-29, :104-110; vllm/src/pos_encoding.rs:8-36)
and rotates NeoX-style in the model dtype (vllm/kernels/pos_encoding_kernels.cu:12-77).  Here the
base, the rotated width, the pairing and the frequency scaling are parameters; frequencies are
computed in float64 on the host and stored as float32, angles are position * inv_freq in float32
inside the kernel, so there is no table and no cap on positions.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch

from .. import kernels
from .base import PositionEncoding, StepContext, register_part


def rope_inverse_frequencies(rot_dim: int, theta: float, scaling_type: str = "default", factor: float = 1.0,
                             low_freq_factor: float = 1.0, high_freq_factor: float = 4.0,
                             original_max_position_embeddings: int = 8192) -> List[float]:
    """f_i = theta^(-2i/rot_dim), then by scaling type:
    linear: f_i / factor.
    llama3: wavelength 2 pi / f_i shorter than L0/high keeps f_i, longer than L0/low gives f_i / factor,
            between them an interpolation with s = (L0 / wavelength - low) / (high - low)."""
    inv = [theta ** (-(2.0 * i) / rot_dim) for i in range(rot_dim // 2)]
    if scaling_type == "default":
        return inv
    if scaling_type == "linear":
        return [f / factor for f in inv]
    if scaling_type == "llama3":
        out = []
        l0 = float(original_max_position_embeddings)
        for f in inv:
            wavelen = 2.0 * math.pi / f
            if wavelen < l0 / high_freq_factor:
                out.append(f)
            elif wavelen > l0 / low_freq_factor:
                out.append(f / factor)
            else:
                s = (l0 / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
                out.append((1.0 - s) * f / factor + s * f)
        return out
    raise ValueError(f"unknown rope scaling type {scaling_type!r}")


@register_part("position_encoding", "rotary")
class RotaryEmbedding(PositionEncoding):
    graph_safe = True

    def __init__(self, rot_dim: int, theta: float = 10000.0, is_neox: bool = True, scaling_type: str = "default",
                 factor: float = 1.0, low_freq_factor: float = 1.0, high_freq_factor: float = 4.0,
                 original_max_position_embeddings: int = 8192):
        if rot_dim <= 0 or rot_dim % 2:
            raise ValueError(f"rotary width must be a positive even number, got {rot_dim}")
        self.rot_dim = int(rot_dim)
        self.is_neox = bool(is_neox)
        self.inv_freq_host = rope_inverse_frequencies(rot_dim, float(theta), scaling_type, float(factor),
                                                      float(low_freq_factor), float(high_freq_factor),
                                                      int(original_max_position_embeddings))
        self.inv_freq: Optional[torch.Tensor] = None

    def prepare(self, dtype: torch.dtype, device: torch.device) -> None:
        self.inv_freq = torch.tensor(self.inv_freq_host, dtype=torch.float64).to(torch.float32).to(device)

    def fused_rotary(self) -> Optional[Tuple[torch.Tensor, int, bool]]:
        return self.inv_freq, self.rot_dim, self.is_neox

    def apply(self, ctx: StepContext, q, k, n_q_heads, n_kv_heads, head_dim) -> None:
        kernels.rope_cache_write(q, None, None, ctx.positions, None, None, 0, None, self.inv_freq, self.rot_dim,
                                 self.is_neox, n_q_heads, 0, head_dim)
        if k is not None:
            kernels.rope_cache_write(k, None, None, ctx.positions, None, None, 0, None, self.inv_freq, self.rot_dim,
                                     self.is_neox, n_kv_heads, 0, head_dim)


@register_part("position_encoding", "none")
class NoPositionEncoding(PositionEncoding):
    graph_safe = True

    def __init__(self):
        pass

    def apply(self, ctx, q, k, n_q_heads, n_kv_heads, head_dim) -> None:
        return None


@register_part("position_encoding", "distance_bias")
class DistanceBias(PositionEncoding):
    """Positions enter the scores, not q and k: slope[head] * (key position - query position) is added to every scaled
    score (the reference's decode kernel takes such slopes, vllm/kernels/attention/attention_kernels.cu:144-145,
    :232-234, through layers/attention.rs:58-83; no model of its Llama path sets them).  The slopes are parameters, one
    per query head.  Only the generic attention kernel takes them, so an attention part with this encoding runs on that
    kernel in bfloat16 too: right, and slow."""
    graph_safe = True

    def __init__(self, slopes):
        self.slopes_host = [float(v) for v in slopes]
        if not self.slopes_host:
            raise ValueError("a distance bias needs one slope per query head")
        self.slopes: Optional[torch.Tensor] = None

    def prepare(self, dtype, device) -> None:
        self.slopes = torch.tensor(self.slopes_host, dtype=torch.float32, device=device)

    def apply(self, ctx, q, k, n_q_heads, n_kv_heads, head_dim) -> None:
        return None

    def score_slopes(self) -> Optional[torch.Tensor]:
        return self.slopes
