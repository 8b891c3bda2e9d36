"""Gated feed-forward: (act(h Wg^T) * (h Wu^T)) Wd^T, gate and up merged into one matrix.

Reference: Mlp in core/src/model_executor/models/llama/llama.rs:223-274 with silu_and_mul_kernel
(vllm/kernels/activation_kernels.cu:26-41).  The activation is a parameter here (the reference
fixes SiLU in code although it parses `hidden_act`).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from .base import FeedForward, NormAfter, Prenormed, StepContext, WeightSpec, register_part
from . import linear
from .linear import matmul_tn, matmul_tn_residual


@register_part("feed_forward", "gated_mlp")
class GatedMLP(FeedForward):
    graph_safe = True
    takes_prenormed = True
    fuses_norm = True

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu", bias: bool = False):
        if activation not in kernels.ACT_CODES:
            raise ValueError(f"activation {activation!r} is not supported (known: {', '.join(sorted(kernels.ACT_CODES))})")
        self.hidden_size, self.intermediate_size, self.activation = int(hidden_size), int(intermediate_size), activation
        self.has_bias = bool(bias)
        self.gate_up: Optional[torch.Tensor] = None
        self.down: Optional[torch.Tensor] = None
        self.gate_up_bias: Optional[torch.Tensor] = None
        self.down_bias: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {"gate_up": WeightSpec([(self.intermediate_size, self.hidden_size)] * 2),
                 "down": WeightSpec([(self.hidden_size, self.intermediate_size)])}
        if self.has_bias:
            specs["gate_up_bias"] = WeightSpec([(self.intermediate_size,)] * 2)
            specs["down_bias"] = WeightSpec([(self.hidden_size,)])
        return specs

    def activation_width(self) -> int:
        return 3 * self.intermediate_size                    # gate, up and their product

    def forward(self, ctx: StepContext, h, then: Optional[NormAfter] = None):
        hx = h.x if isinstance(h, Prenormed) else h
        if linear.USE_SKINNY and self.gate_up_bias is None and kernels.gemm_skinny_supported(hx, self.gate_up):
            # a decode step: gate, up and the activation in one pass over the weights
            m = torch.empty((hx.shape[0], self.intermediate_size), dtype=hx.dtype, device=hx.device)
            kernels.gemm_skinny(m, hx, self.gate_up, fuse_act=self.activation,
                                prenorm=(h.sumsq, h.eps, h.width) if isinstance(h, Prenormed) else None)
            return self._down(m, then)
        gu = matmul_tn(h, self.gate_up, bias=self.gate_up_bias)
        m = torch.empty((gu.shape[0], self.intermediate_size), dtype=gu.dtype, device=gu.device)
        kernels.gated_act(m, gu, self.activation)
        return self._down(m, then)

    def _down(self, m: torch.Tensor, then: Optional[NormAfter]):
        if then is not None and self.down_bias is None:
            p = matmul_tn_residual(m, self.down, then)
            if p is not None:
                return p
        return matmul_tn(m, self.down, bias=self.down_bias)
