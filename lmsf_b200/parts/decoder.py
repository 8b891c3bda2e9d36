"""A decoder put together from a `ModelSpec`: embedding, blocks run in the order the spec lists,
final norm over the rows whose logits are wanted, output head.

The reference's counterpart is Llama::do_forward (core/src/model_executor/models/llama/llama.rs:397-476);
it takes the hidden state at one padded column (llama.rs:466), here the wanted rows are gathered
before the final norm so that the head runs on them alone.
"""
from __future__ import annotations

from typing import Iterator, List, Optional, Tuple

import torch

from .. import kernels
from ..utils.tracing import span
from .base import (Block, KVCacheSpec, LayerCache, ModelSpec, Part, PartSpec, StateSpec, StepContext, build_part,
                   part_class, with_nested)


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = build_part("embedding", spec.embedding)
        self.blocks: List[Block] = []
        self._owned: List[Tuple[Part, PartSpec]] = list(with_nested(self.embedding, spec.embedding))
        for ls in spec.layers:
            cls = part_class("block", ls.block)
            missing = [r for r in cls.ROLES if r not in ls.parts]
            if missing:
                raise ValueError(f"block {ls.block!r} needs the parts {sorted(cls.ROLES)}; missing {missing}")
            parts = {}
            for role, family in cls.ROLES.items():
                parts[role] = build_part(family, ls.parts[role])
                self._owned += list(with_nested(parts[role], ls.parts[role]))
            self.blocks.append(cls(parts, **ls.block_params))
        self.final_norm = build_part("norm", spec.final_norm)
        self.lm_head = build_part("linear", spec.lm_head)
        self._owned += [*with_nested(self.final_norm, spec.final_norm), *with_nested(self.lm_head, spec.lm_head)]
        self.calls = list(spec.order)
        for j, call in enumerate(self.calls):
            if not (0 <= call.layer < len(self.blocks)):
                raise ValueError(f"order[{j}] names layer {call.layer}, the model has {len(self.blocks)}")
            if call.cache_of is not None:
                if not (0 <= call.cache_of < j) or self.calls[call.cache_of].cache_of is not None:
                    raise ValueError(f"order[{j}].cache_of must name an earlier entry that owns its cache")
                a, b = self.call_cache_spec(j), self.call_cache_spec(call.cache_of)
                if a is None or b is None or (a.num_kv_heads, a.head_dim) != (b.num_kv_heads, b.head_dim):
                    raise ValueError(f"order[{j}] cannot read the cache of order[{call.cache_of}]: "
                                     f"their key/value shapes differ")

    # ---- what the loader and the cache need to know
    def parts_with_specs(self) -> Iterator[Tuple[Part, PartSpec]]:
        return iter(self._owned)

    def call_cache_spec(self, j: int) -> Optional[KVCacheSpec]:
        m = self.blocks[self.calls[j].layer].mixer
        return m.cache_spec() if m is not None else None

    def call_state_spec(self, j: int) -> Optional[StateSpec]:
        m = self.blocks[self.calls[j].layer].mixer
        return m.state_spec() if m is not None else None

    def prepare(self, dtype: torch.dtype, device: torch.device) -> None:
        for part, _ in self._owned:
            part.prepare(dtype, device)

    # ---- the forward pass of one step
    def forward(self, ctx: StepContext, caches: List[LayerCache], logit_rows: Optional[torch.Tensor]) -> torch.Tensor:
        """logits float32 [len(logit_rows), vocab]; logit_rows: int32 indices into the step's tokens."""
        x = self.embedding.forward(ctx)
        res = None
        for j, call in enumerate(self.calls):
            block = self.blocks[call.layer]
            # a block that can take the next block's first norm into its last product is told that norm and its reader
            entry = self.blocks[self.calls[j + 1].layer].entry() if block.fuses_next_norm and j + 1 < len(self.calls) else None
            with span(f"layer {call.layer}"):
                if entry is not None:
                    x, res = block.forward(ctx, x, res, caches[j], next_entry=entry)
                else:
                    x, res = block.forward(ctx, x, res, caches[j])
        n_rows = 0 if logit_rows is None else logit_rows.numel()
        if n_rows == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=x.device)
        xs = torch.empty((n_rows, x.shape[1]), dtype=x.dtype, device=x.device)
        kernels.embedding(xs, x, logit_rows)                     # a row gather
        if res is None:
            h = self.final_norm.forward(xs)
        else:
            rs = torch.empty((n_rows, res.shape[1]), dtype=res.dtype, device=res.device)
            kernels.embedding(rs, res, logit_rows)
            h, _ = self.final_norm.forward_residual(xs, rs)
        return self.lm_head.forward(h)
