"""Grouped-query attention over the paged cache.

The reference's CausalSelfAttention (core/src/model_executor/models/llama/llama.rs:45-221) projects
q, k, v with one merged matrix, rotates q and k, scatters k and v into pages
(core/src/model_executor/layers/attention.rs:185-207) and then runs a dense prompt attention on
the fresh k, v or a paged decode kernel (attention.rs:209-294).  Here one step may hold prompt
portions and decoded tokens together: k and v always go to pages first and every query reads all
its keys from pages, so a portion that starts in the middle of a prompt needs nothing special.
"""
from __future__ import annotations

import math
import os
import warnings
from typing import Dict, Optional

import torch

from .. import kernels
from .base import (KVCacheSpec, LayerCache, Mixer, NormAfter, PositionEncoding, Prenormed, StepContext, WeightSpec,
                   register_part)
from . import linear
from .linear import matmul_tn, matmul_tn_residual


SPLITS_PER_REQUEST = os.environ.get("LMSF_DECODE_ITEMS", "1") != "0"   # decode batches of very different lengths: splits per request
USE_TC_PREFILL = True     # head sizes 64 and 128: prompt portions run on the tcgen05 kernel (csrc/attention_tc.cu)
FUSE_QKV_ROPE = True      # up to 16 single tokens: rotary encoding and cache write in the q/k/v product's epilogue


@register_part("mixer", "paged_attention")
class PagedAttention(Mixer):
    graph_safe = True      # launch geometry depends on the batch's size only: a decode step can be replayed
    takes_prenormed = True
    fuses_norm = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position_encoding: Optional[PositionEncoding] = None, window: Optional[int] = None,
                 scale: Optional[float] = None, bias: bool = False, softcap: Optional[float] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads cannot be grouped over {num_kv_heads} kv heads")
        if head_dim % 16 or not (16 <= head_dim <= 256):
            raise ValueError(f"head_dim {head_dim} is not supported: the attention kernels take multiples of 16 "
                             f"from 16 to 256")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.position_encoding = position_encoding
        self.window = int(window) if window else None
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        # scores capped smoothly, softcap * tanh(score / softcap), before the softmax (not a Llama constant).  Only the
        # generic kernel takes it: a part built with a cap runs on that kernel in bfloat16 too, which is right and slow
        self.softcap = float(softcap) if softcap else 0.0
        self.q_size = num_heads * head_dim
        self.kv_size = num_kv_heads * head_dim
        self.has_bias = bool(bias)
        self.qkv: Optional[torch.Tensor] = None
        self.o: Optional[torch.Tensor] = None
        self.qkv_bias: Optional[torch.Tensor] = None
        self.o_bias: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {"qkv": WeightSpec([(self.q_size, self.hidden_size), (self.kv_size, self.hidden_size),
                                    (self.kv_size, self.hidden_size)]),
                 "o": WeightSpec([(self.hidden_size, self.q_size)])}
        if self.has_bias:
            specs["qkv_bias"] = WeightSpec([(self.q_size,), (self.kv_size,), (self.kv_size,)])
            specs["o_bias"] = WeightSpec([(self.hidden_size,)])
        return specs

    def cache_spec(self) -> Optional[KVCacheSpec]:
        return KVCacheSpec(self.num_kv_heads, self.head_dim, self.window)

    def activation_width(self) -> int:
        return 2 * self.q_size + 2 * self.kv_size           # q, k, v and the attention's output

    def prepare(self, dtype, device) -> None:
        if self.position_encoding is not None:
            self.position_encoding.prepare(dtype, device)
        if dtype == torch.bfloat16 and not kernels.mma_attention_supported(dtype, self.head_dim):
            # right but slow: said once, so that nobody wonders where the time goes
            warnings.warn(f"head_dim {self.head_dim} is beyond the tensor-core attention kernels "
                          f"(up to {kernels.MMA_MAX_HEAD_DIM}); bfloat16 attention runs on the generic kernel",
                          RuntimeWarning, stacklevel=2)
        elif dtype == torch.bfloat16 and (self.softcap or self._slopes() is not None):
            warnings.warn("a cap on the attention scores, or a bias on them, is taken by the generic kernel only; "
                          "bfloat16 attention runs on it", RuntimeWarning, stacklevel=2)
        slopes = self._slopes()
        if slopes is not None and slopes.numel() != self.num_heads:
            raise ValueError(f"{slopes.numel()} slopes for {self.num_heads} query heads")

    def _slopes(self) -> Optional[torch.Tensor]:
        return self.position_encoding.score_slopes() if self.position_encoding is not None else None

    def forward(self, ctx: StepContext, h, cache: LayerCache, then: Optional[NormAfter] = None):
        group = ctx.groups[cache.group]
        fused = self.position_encoding.fused_rotary() if self.position_encoding is not None else None
        hx = h.x if isinstance(h, Prenormed) else h
        if (FUSE_QKV_ROPE and cache.owner and linear.USE_SKINNY and self.qkv_bias is None and (fused is not None or self.position_encoding is None)
                and kernels.gemm_skinny_qkv_rope_supported(hx, self.qkv, self.head_dim, fused[1] if fused else 0,
                                                           fused[2] if fused else True)):
            # a few single tokens (a decode step): projection, rotation and cache write in one kernel
            inv_freq, rot_dim, is_neox = fused if fused is not None else (None, 0, True)
            q = torch.empty((ctx.n_tokens, self.q_size), dtype=hx.dtype, device=hx.device)
            kernels.gemm_skinny_qkv_rope(q, hx, self.qkv, ctx.positions, ctx.token_seq, group.block_table, group.block_size,
                                         cache.kv, inv_freq, rot_dim, is_neox, self.num_heads, self.num_kv_heads,
                                         self.head_dim, ctx.error_flag,
                                         prenorm=(h.sumsq, h.eps, h.width) if isinstance(h, Prenormed) else None)
            out = torch.empty((ctx.n_tokens, self.q_size), dtype=hx.dtype, device=hx.device)
            self.attend(ctx, out, q, cache.kv, group)
            return self._project_out(out, then)
        if cache.owner:
            qkv = matmul_tn(h, self.qkv, bias=self.qkv_bias)
            q = qkv[:, :self.q_size]
            k = qkv[:, self.q_size:self.q_size + self.kv_size]
            v = qkv[:, self.q_size + self.kv_size:]
        else:  # keys and values are another call's: only the queries are needed
            q = matmul_tn(h, self.qkv[:self.q_size], bias=None if self.qkv_bias is None else self.qkv_bias[:self.q_size])
            k = v = None
        if self.position_encoding is not None and fused is None:
            self.position_encoding.apply(ctx, q, k, self.num_heads, self.num_kv_heads, self.head_dim)
        inv_freq, rot_dim, is_neox = fused if fused is not None else (None, 0, True)
        if fused is not None or cache.owner:
            kernels.rope_cache_write(q, k, v, ctx.positions, ctx.token_seq, group.block_table, group.block_size,
                                     cache.kv if cache.owner else None, inv_freq, rot_dim, is_neox, self.num_heads,
                                     self.num_kv_heads, self.head_dim, ctx.error_flag)
        out = torch.empty((ctx.n_tokens, self.q_size), dtype=q.dtype, device=q.device)
        self.attend(ctx, out, q, cache.kv, group)
        return self._project_out(out, then)

    def _project_out(self, out: torch.Tensor, then: Optional[NormAfter]):
        if then is not None and self.o_bias is None:
            p = matmul_tn_residual(out, self.o, then)
            if p is not None:
                return p
        return matmul_tn(out, self.o, bias=self.o_bias)

    def attend(self, ctx: StepContext, out: torch.Tensor, q: torch.Tensor, kv: torch.Tensor, group) -> None:
        """bfloat16 with a head size up to 128: single tokens go to the split-key decode kernel, longer portions
        to a tiled prefill kernel (tcgen05 with accumulators in tensor memory for head sizes 64 and 128,
        mma.sync otherwise).  Everything else, float32 included, runs on the
        generic kernel, which is also their plain twin."""
        slopes = self._slopes()
        if kernels.mma_attention_supported(q.dtype, self.head_dim) and not self.softcap and slopes is None and \
                not ctx.extras.get("force_generic_attention"):
            if ctx.n_decode_seqs:
                max_ctx = ctx.extras.get("decode_max_ctx")
                if max_ctx is None:
                    max_ctx = ctx.extras["decode_max_ctx"] = max(c for c, n in zip(ctx.ctx_lens, ctx.q_lens) if n == 1)
                visible = min(max_ctx, self.window) if self.window else max_ctx
                # the mean matters to the plan only where it is far below the longest context (a graph names its class)
                mean_ctx = ctx.extras.get("decode_mean_ctx")
                if mean_ctx is None:
                    lens = [c for c, n in zip(ctx.ctx_lens, ctx.q_lens) if n == 1]
                    mean_ctx = ctx.extras["decode_mean_ctx"] = sum(lens) / len(lens)
                mean_visible = min(mean_ctx, visible)
                group_size = self.num_heads // self.num_kv_heads
                all_decode = ctx.n_decode_seqs == ctx.n_seqs
                if SPLITS_PER_REQUEST and ctx.n_decode_seqs >= 2 and mean_visible * 4 <= visible:
                    # Requests that differ much in length (a mean of a quarter of the longest and less): splits per
                    # request, from a list of work items that a kernel makes from the step's context lengths (once a
                    # step, for all layers of this geometry).  Measured, 8 layers of the 8B shape: one request at
                    # 30,000 tokens beside 63 at 500: 1.64 ms a step against 2.11 ms with one number of splits for all;
                    # one at 2,300 beside 63 at 1,200: 1.54 against 1.50 (the list's launch starts after the kernel
                    # before it and adds up through global memory), hence the threshold.
                    widths = kernels.decode_widths(self.head_dim, group_size)
                    pairs = ctx.n_decode_seqs * self.num_kv_heads * ((group_size + 15) // 16)
                    warps, slots = widths[0][0], widths[0][2][0]
                    if len(widths) > 1 and pairs > slots:
                        warps, slots = widths[1][0], widths[1][2][0]
                    key = ("decode_items", self.num_kv_heads, group_size, slots, self.window or 0)
                    items = ctx.extras.get(key)
                    if items is None:
                        capacity = kernels.decode_items_capacity(ctx.n_decode_seqs, self.num_kv_heads, group_size, slots)
                        items = ctx.extras[key] = torch.empty((capacity, 4), dtype=torch.int32, device=q.device)
                        kernels.decode_build_items(items, ctx.ctx_len, None if all_decode else ctx.decode_seq_ids,
                                                   ctx.n_decode_seqs, self.window or 0, self.num_heads, self.num_kv_heads,
                                                   self.head_dim, slots)
                    need = kernels.attention_decode_items_scratch_floats(items.shape[0], self.num_heads, self.head_dim)
                    scratch = ctx.extras.get("decode_items_scratch")
                    if scratch is None or scratch.numel() < need:
                        scratch = ctx.extras["decode_items_scratch"] = torch.zeros(need, dtype=torch.float32, device=q.device)
                    kernels.attention_decode_items(out, q, kv, group.block_table, group.block_size, items, ctx.cu_q,
                                                   ctx.ctx_len, self.scale, self.window or 0, self.num_heads,
                                                   self.num_kv_heads, self.head_dim, warps, scratch)
                    splits = None
                else:
                    splits, warps = kernels.decode_plan(ctx.n_decode_seqs, self.num_kv_heads, group_size, visible,
                                                        self.head_dim, kernels.decode_widths(self.head_dim, group_size),
                                                        mean_ctx=mean_visible if mean_visible * 4 <= visible * 3 else None)
                if splits is not None:
                    need = kernels.attention_decode_scratch_floats(ctx.n_seqs, self.num_heads, splits, self.head_dim)
                    scratch = ctx.extras.get("decode_scratch")
                    if need and (scratch is None or scratch.numel() < need):
                        scratch = ctx.extras["decode_scratch"] = torch.zeros(need, dtype=torch.float32, device=q.device)
                    kernels.attention_decode(out, q, kv, group.block_table, group.block_size,
                                             None if all_decode else ctx.decode_seq_ids, ctx.n_decode_seqs, ctx.cu_q,
                                             ctx.ctx_len, self.scale, self.window or 0, self.num_heads,
                                             self.num_kv_heads, self.head_dim, splits, scratch if need else None, warps)
            if ctx.n_q_tiles and USE_TC_PREFILL and kernels.tc_attention_supported(q.dtype, self.head_dim):
                kernels.attention_prefill_tc(out, q, kv, group.block_table, group.block_size, ctx.q_tile128_seq,
                                             ctx.q_tile128_q0, ctx.n_q_tiles128, ctx.cu_q, ctx.ctx_len, self.scale,
                                             self.window or 0, self.num_heads, self.num_kv_heads, self.head_dim,
                                             ctx.error_flag)
            elif ctx.n_q_tiles:
                kernels.attention_prefill(out, q, kv, group.block_table, group.block_size, ctx.q_tile_seq,
                                          ctx.q_tile_q0, ctx.n_q_tiles, ctx.cu_q, ctx.ctx_len, self.scale,
                                          self.window or 0, self.num_heads, self.num_kv_heads, self.head_dim)
            return
        kernels.attention_generic(out, q, kv, group.block_table, group.block_size, ctx.token_seq, ctx.positions,
                                  self.scale, self.window or 0, self.num_heads, self.num_kv_heads, self.head_dim,
                                  softcap=self.softcap, slopes=slopes)
