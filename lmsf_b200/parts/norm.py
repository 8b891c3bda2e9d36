"""RMSNorm, alone or fused with the residual add before it.

Formula of the reference: vllm/kernels/layernorm_kernels.cu:13-68, called from
core/src/model_executor/models/llama/llama.rs:295-317, :333, :461-462.  The residual stream is
float32 here whatever the activation dtype.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple, Union

import torch

from .. import kernels
from .base import Norm, Prenormed, WeightSpec, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    graph_safe = True
    splittable = True

    def __init__(self, hidden_size: int, eps: float, weight_offset: float = 0.0):
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)
        # architectures that scale by (1 + w) store w: the offset is folded into the weight when it is set, as the
        # reference's loader does (vllm/src/rms_norm.rs:45-56); 0 for Llama
        self.weight_offset = float(weight_offset)
        self.weight: Optional[torch.Tensor] = None

    def set_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        super().set_weights(tensors)
        if self.weight_offset and "weight" in tensors:
            self.weight = (tensors["weight"].float() + self.weight_offset).to(tensors["weight"].dtype)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec([(self.hidden_size,)], keep_fp32=True)}

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = torch.empty_like(x)
        kernels.add_rmsnorm(h, x, None, self.weight, self.eps, 0)
        return h

    def forward_residual(self, x: Union[torch.Tensor, Prenormed], res: Optional[torch.Tensor]
                         ) -> Tuple[Union[torch.Tensor, Prenormed], torch.Tensor]:
        if isinstance(x, Prenormed):
            if x.norm is not self or x.res is not res:
                raise ValueError("a Prenormed activation was prepared for another norm or residual stream")
            return x, res
        h = torch.empty_like(x)
        if res is None:
            res = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            kernels.add_rmsnorm(h, x, res, self.weight, self.eps, 1)
        else:
            kernels.add_rmsnorm(h, x, res, self.weight, self.eps, 2)
        return h, res

    def finish(self, p: Prenormed) -> torch.Tensor:
        """The ordinary output of the norm from a `Prenormed`, for a product that cannot take one."""
        h = torch.empty_like(p.x)
        kernels.finish_rmsnorm(h, p.res, p.sumsq, self.weight, self.eps)
        return h
