"""Arrangements of parts inside one layer.

`pre_norm` is the reference's Block (core/src/model_executor/models/llama/llama.rs:276-385): norm,
mixer, norm, feed-forward, where each residual add is deferred into the following norm
(llama.rs:295-317, :333) and the layer hands (branch output, residual) to the next one.
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import torch

from .. import kernels
from .base import Block, LayerCache, Norm, NormAfter, Part, StepContext, register_part

# A step of a few tokens in bfloat16: a norm between two weight-streaming products is done by those products
# (the one before adds to the residual stream and leaves sums of squares, the one after divides).  LMSF_FUSE_NORMS=0:
# every norm is a kernel of its own.
FUSE_NORMS = os.environ.get("LMSF_FUSE_NORMS", "1") != "0"


def norm_after(ctx: StepContext, producer: Part, norm: Norm, consumer: Part, res: Optional[torch.Tensor]) -> Optional[NormAfter]:
    """The offer to `producer` to take `norm` into its last product, if everybody involved is able to on this step."""
    if (FUSE_NORMS and res is not None and getattr(producer, "fuses_norm", False)
            and getattr(consumer, "takes_prenormed", False) and getattr(norm, "splittable", False)
            and ctx.dtype == torch.bfloat16 and ctx.n_tokens <= kernels.SKINNY_MAX_M):
        return NormAfter(norm, res)
    return None


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    ROLES = {"mixer_norm": "norm", "mixer": "mixer", "ffn_norm": "norm", "feed_forward": "feed_forward"}

    def __init__(self, parts: Dict[str, Part]):
        super().__init__(parts)
        self.mixer_norm, self._mixer = parts["mixer_norm"], parts["mixer"]
        self.ffn_norm, self.feed_forward = parts["ffn_norm"], parts["feed_forward"]

    fuses_next_norm = True

    def entry(self) -> Optional[Tuple[Norm, Part]]:
        return self.mixer_norm, self._mixer

    def forward(self, ctx: StepContext, x, res: Optional[torch.Tensor], cache: LayerCache,
                next_entry: Optional[Tuple[Norm, Part]] = None):
        h, res = self.mixer_norm.forward_residual(x, res)
        then = norm_after(ctx, self._mixer, self.ffn_norm, self.feed_forward, res)
        a = self._mixer.forward(ctx, h, cache, then=then) if then is not None else self._mixer.forward(ctx, h, cache)
        h, res = self.ffn_norm.forward_residual(a, res)
        then = norm_after(ctx, self.feed_forward, next_entry[0], next_entry[1], res) if next_entry is not None else None
        out = self.feed_forward.forward(ctx, h, then=then) if then is not None else self.feed_forward.forward(ctx, h)
        return out, res
