"""Arrangements of parts inside one layer.

`pre_norm` is the reference's Block (core/src/model_executor/models/llama/llama.rs:276-385): norm,
mixer, norm, feed-forward, where each residual add is deferred into the following norm
(llama.rs:295-317, :333) and the layer hands (branch output, residual) to the next one.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .base import Block, LayerCache, Part, StepContext, register_part


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    ROLES = {"mixer_norm": "norm", "mixer": "mixer", "ffn_norm": "norm", "feed_forward": "feed_forward"}

    def __init__(self, parts: Dict[str, Part]):
        super().__init__(parts)
        self.mixer_norm, self._mixer = parts["mixer_norm"], parts["mixer"]
        self.ffn_norm, self.feed_forward = parts["ffn_norm"], parts["feed_forward"]

    def forward(self, ctx: StepContext, x: torch.Tensor, res: Optional[torch.Tensor], cache: LayerCache
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        h, res = self.mixer_norm.forward_residual(x, res)
        a = self._mixer.forward(ctx, h, cache)
        h, res = self.ffn_norm.forward_residual(a, res)
        return self.feed_forward.forward(ctx, h), res
