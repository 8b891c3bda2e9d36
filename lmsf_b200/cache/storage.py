"""Device side of the cache: the page tensors of every group of layers and the state slots.

The reference allocates one (K, V) pair of tensors per layer (core/src/worker/cache_engine.rs:107-160)
with a layout made for its decode kernel.  Here every group of layers has ONE tensor
[call, page, 2 (k, v), kv_head, slot, head_dim]: a page number addresses the same page in every
layer of its group, and one (page, kv_head) holds block_size * head_dim contiguous values.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from ..parts.base import KVCacheSpec, LayerCache, StateSpec
from .manager import CacheManager, GroupSpec


@dataclass
class GroupLayout:
    spec: KVCacheSpec
    calls: List[int]                 # entries of the run order that own a cache in this group

    def page_bytes(self, block_size: int, dtype: torch.dtype) -> int:
        """Bytes of one page over all layers of the group (cf. core/src/worker/cache_engine.rs:88-105)."""
        return len(self.calls) * 2 * self.spec.num_kv_heads * self.spec.head_dim * block_size * \
            torch.empty(0, dtype=dtype).element_size()


def plan_groups(model) -> Tuple[List[GroupLayout], Dict[int, Tuple[int, int]]]:
    """Groups the cache-owning calls of a model by what they need.  Returns the groups and, for every
    call that touches a cache, (group index, index of its tensor inside the group)."""
    groups: List[GroupLayout] = []
    where: Dict[int, Tuple[int, int]] = {}
    for j, call in enumerate(model.calls):
        spec = model.call_cache_spec(j)
        if spec is None:
            continue
        if call.cache_of is not None:
            where[j] = where[call.cache_of]
            continue
        for g, gl in enumerate(groups):
            if gl.spec == spec:
                gl.calls.append(j)
                where[j] = (g, len(gl.calls) - 1)
                break
        else:
            groups.append(GroupLayout(spec, [j]))
            where[j] = (len(groups) - 1, 0)
    return groups, where


def split_pages(groups: List[GroupLayout], block_size: int, dtype: torch.dtype, budget_bytes: int,
                max_model_len: int) -> List[int]:
    """Page counts per group for a byte budget: in proportion to what one request of full length holds."""
    if not groups:
        return []
    need = []
    for gl in groups:
        toks = max_model_len if gl.spec.window is None else min(max_model_len, gl.spec.window + 2 * block_size)
        need.append((toks + block_size - 1) // block_size)
    bytes_per_request = sum(n * gl.page_bytes(block_size, dtype) for n, gl in zip(need, groups))
    scale = budget_bytes / max(1, bytes_per_request)
    return [max(1, int(n * scale)) for n in need]


class CacheStorage:
    def __init__(self, model, block_size: int, num_blocks: List[int], num_state_slots: int, dtype: torch.dtype,
                 device: torch.device):
        self.block_size = block_size
        self.groups, where = plan_groups(model)
        if len(num_blocks) != len(self.groups):
            raise ValueError(f"the model has {len(self.groups)} cache groups, {len(num_blocks)} page counts given")
        self.num_blocks = list(num_blocks)
        self.num_state_slots = num_state_slots
        # one page more than the pool knows: the "null page" that stand-in requests of a padded batch write to
        self.tensors = [torch.zeros((len(gl.calls), n + 1, 2, gl.spec.num_kv_heads, block_size, gl.spec.head_dim),
                                    dtype=dtype, device=device) for gl, n in zip(self.groups, num_blocks)]
        self.null_pages = list(num_blocks)
        self.layer_caches: List[LayerCache] = []
        self.state_tensors: List[Optional[torch.Tensor]] = []
        for j, call in enumerate(model.calls):
            lc = LayerCache(owner=call.cache_of is None)
            if j in where:
                g, i = where[j]
                lc.kv, lc.group = self.tensors[g][i], g
            st: Optional[StateSpec] = model.call_state_spec(j)
            if st is not None:
                # one slot more than the manager hands out: the "null slot" of a padded batch's stand-in requests
                lc.state = torch.zeros((num_state_slots + 1, *st.shape), dtype=st.dtype, device=device)
            self.state_tensors.append(lc.state)
            self.layer_caches.append(lc)

    def make_manager(self) -> CacheManager:
        return CacheManager([GroupSpec(gl.spec.window) for gl in self.groups], self.num_blocks, self.block_size,
                            self.num_state_slots)

    def zero_state_slots(self, slots: List[int]) -> None:
        if not slots:
            return
        for st in self.state_tensors:
            if st is not None:
                for s in slots:
                    st[s].zero_()
