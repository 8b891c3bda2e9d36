"""Token embedding: x[t] = E[id_t] (core/src/model_executor/layers/vocab_parallel_embedding.rs:5-38)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from .base import Part, StepContext, WeightSpec, register_part


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, scale: float = 1.0):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.scale = float(scale)      # every embedding is multiplied by it (1 for Llama; sqrt(width) elsewhere)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec([(self.vocab_size, self.hidden_size)])}

    def forward(self, ctx: StepContext) -> torch.Tensor:
        x = torch.empty((ctx.n_tokens, self.hidden_size), dtype=self.weight.dtype, device=self.weight.device)
        kernels.embedding(x, self.weight, ctx.token_ids, ctx.error_flag, scale=self.scale)
        return x
