"""RMSNorm, alone or fused with the residual add before it.

Formula of the reference: vllm/kernels/layernorm_kernels.cu:13-68, called from
core/src/model_executor/models/llama/llama.rs:295-317, :333, :461-462.  The residual stream is
float32 here whatever the activation dtype.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import kernels
from .base import Norm, WeightSpec, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, hidden_size: int, eps: float):
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec([(self.hidden_size,)], keep_fp32=True)}

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = torch.empty_like(x)
        kernels.add_rmsnorm(h, x, None, self.weight, self.eps, 0)
        return h

    def forward_residual(self, x: torch.Tensor, res: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
        h = torch.empty_like(x)
        if res is None:
            res = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            kernels.add_rmsnorm(h, x, res, self.weight, self.eps, 1)
        else:
            kernels.add_rmsnorm(h, x, res, self.weight, self.eps, 2)
        return h, res
