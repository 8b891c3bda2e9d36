"""A Llama step made of yinqiwen/lmsf's own kernels in the reference's own order: the comparison arm of bench.py.

The reference's engine is Rust and cannot be built here; its CUDA kernels can (build_ref.py).  This file strings
them together the way the reference does and imports nothing of `lmsf_b200`:

    embedding lookup                                   core/src/model_executor/models/llama/llama.rs:409
    per layer (llama.rs:286-339):
      rms_norm (first layer) / fused_add_rms_norm      vllm/kernels/layernorm_kernels.cu
      merged q,k,v product (cuBLASLt in the reference: tops/csrc/tops/tensorrt_llm/common/cublasMMWrapper.cpp:122;
                            here torch.mm, the same library)
      rotary_embedding in place on q and k             vllm/kernels/pos_encoding_kernels.cu
      reshape_and_cache                                vllm/kernels/cache_kernels.cu
      prompt: float32 softmax(mask(q k^T / sqrt(hd))) v on materialised scores with repeated kv heads
              (core/src/model_executor/layers/attention.rs:107-155; library products + softmax)
      decode: paged_attention_v1 or _v2 by the reference's rule (attention.rs:255-257)
      output product, fused_add_rms_norm, merged gate/up product, vllm_silu_and_mul, down product
    fused_add_rms_norm with the final weight, the last position of each request, head product (llama.rs:461-471)
    greedy choice: argmax of the float32 log-softmax    core/src/model_executor/layers/sampler.rs:363-384, :915-922

Buffers are allocated once per batch shape (the reference draws them from arenas, llama.rs:415-418); there is no
CUDA graph, as in the reference.  Kernel launches go to the null stream like the reference's
(vllm/src/rms_norm.rs:68), which orders itself with torch's default stream.
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch

from . import ref_kernels as rk


class ReferenceLlama:
    def __init__(self, cfg: Dict, n_layers: int, num_blocks: int, block_size: int, device, seed: int = 0, std: float = 0.02):
        self.cfg, self.n_layers, self.bs, self.dev = cfg, n_layers, block_size, torch.device(device)
        self.H, self.I, self.V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
        self.nh, self.nkv, self.hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
        self.eps = float(cfg["rms_norm_eps"])
        self.scale = 1.0 / math.sqrt(self.hd)
        g = torch.Generator(device=self.dev).manual_seed(seed)
        dt = torch.bfloat16

        def w(*shape):
            return (torch.randn(*shape, device=self.dev, generator=g, dtype=torch.float32) * std).to(dt)

        self.embed = w(self.V, self.H)
        self.head = self.embed if cfg.get("tie_word_embeddings") else w(self.V, self.H)
        self.layers = []
        qkv_rows = (self.nh + 2 * self.nkv) * self.hd
        for _ in range(n_layers):
            self.layers.append(dict(n1=torch.ones(self.H, dtype=dt, device=self.dev), qkv=w(qkv_rows, self.H),
                                    o=w(self.H, self.nh * self.hd), n2=torch.ones(self.H, dtype=dt, device=self.dev),
                                    gate_up=w(2 * self.I, self.H), down=w(self.H, self.I)))
        self.norm = torch.ones(self.H, dtype=dt, device=self.dev)
        self.caches = []
        for _ in range(n_layers):
            kc, vc = rk.new_caches(num_blocks, self.nkv, self.hd, block_size, dt, self.dev)
            kc.normal_(0.0, 1.0)
            vc.normal_(0.0, 1.0)
            self.caches.append((kc, vc))
        # the reference's table: theta fixed at 10000 in its code (rotary_embedding.rs:104); config's theta here
        self.cos_sin = rk.cos_sin_cache(float(cfg.get("rope_theta", 10000.0)), self.hd, cfg["max_position_embeddings"], dt, self.dev)
        self._bufs: Dict[int, Dict[str, torch.Tensor]] = {}
        self.launches = 0

    def _buffers(self, n: int) -> Dict[str, torch.Tensor]:
        b = self._bufs.get(n)
        if b is None:
            dt, dev = torch.bfloat16, self.dev
            qkv_rows = (self.nh + 2 * self.nkv) * self.hd
            b = self._bufs[n] = dict(
                x=torch.empty(n, self.H, dtype=dt, device=dev), res=torch.empty(n, self.H, dtype=dt, device=dev),
                h=torch.empty(n, self.H, dtype=dt, device=dev), qkv=torch.empty(n, qkv_rows, dtype=dt, device=dev),
                attn=torch.empty(n, self.nh * self.hd, dtype=dt, device=dev), o=torch.empty(n, self.H, dtype=dt, device=dev),
                gu=torch.empty(n, 2 * self.I, dtype=dt, device=dev), m=torch.empty(n, self.I, dtype=dt, device=dev))
        return b

    def _layers(self, b, n, positions_i64, slots_i64, attend) -> None:
        """The blocks of llama.rs:286-339 on b['x'] (hidden states) and b['res'] (residual)."""
        q_w, kv_w = self.nh * self.hd, self.nkv * self.hd
        for i, L in enumerate(self.layers):
            if i == 0:
                rk.rms_norm(b["h"], b["x"], L["n1"], self.eps)
                b["res"].copy_(b["x"])
                h = b["h"]
            else:
                rk.fused_add_rms_norm(b["x"], b["res"], L["n1"], self.eps)
                h = b["x"]
            torch.mm(h, L["qkv"].t(), out=b["qkv"])
            q, k, v = b["qkv"][:, :q_w], b["qkv"][:, q_w:q_w + kv_w], b["qkv"][:, q_w + kv_w:]
            rk.rotary_embedding(positions_i64, q, k, self.cos_sin, self.hd, self.nh, self.nkv, True)
            kc, vc = self.caches[i]
            rk.reshape_and_cache(k, v, kc, vc, slots_i64, self.nkv, self.hd, self.bs)
            attend(i, q, k, v, b["attn"])
            torch.mm(b["attn"], L["o"].t(), out=b["o"])
            rk.fused_add_rms_norm(b["o"], b["res"], L["n2"], self.eps)
            torch.mm(b["o"], L["gate_up"].t(), out=b["gu"])
            rk.silu_and_mul(b["m"], b["gu"])
            torch.mm(b["m"], L["down"].t(), out=b["x"])
            self.launches += 10 + (1 if i == 0 else 0)

    def decode_step(self, token_ids, positions_i64, slots_i64, block_tables, context_lens, max_context_len) -> torch.Tensor:
        """One token per request; returns the chosen tokens [n] (int64, on the device)."""
        n = token_ids.numel()
        b = self._buffers(n)
        torch.index_select(self.embed, 0, token_ids, out=b["x"])

        def attend(i, q, k, v, out):
            kc, vc = self.caches[i]
            ws = b.get("ws")
            parts = -(-max_context_len // rk.PARTITION_SIZE)
            if ws is None or ws[0].shape[2] != parts:
                ws = b["ws"] = (torch.empty((n, self.nh, parts, self.hd), dtype=torch.bfloat16, device=self.dev),
                                torch.empty((n, self.nh, parts), dtype=torch.float32, device=self.dev),
                                torch.empty((n, self.nh, parts), dtype=torch.float32, device=self.dev))
            which = rk.paged_attention(out.view(n, self.nh, self.hd), q.view(n, self.nh, self.hd), kc, vc, block_tables,
                                       context_lens, max_context_len, self.scale, self.nkv, workspace=ws)
            self.launches += 1 if which == "v2" else 0

        self._layers(b, n, positions_i64, slots_i64, attend)
        rk.fused_add_rms_norm(b["x"], b["res"], self.norm, self.eps)
        logits = torch.mm(b["x"], self.head.t()).float()
        self.launches += 6
        return torch.argmax(torch.log_softmax(logits, dim=-1), dim=-1)

    def prefill(self, token_ids, positions_i64, slots_i64) -> torch.Tensor:
        """One whole prompt of T tokens (batch 1, no padding needed); returns the chosen token."""
        T = token_ids.numel()
        b = self._buffers(T)
        torch.index_select(self.embed, 0, token_ids, out=b["x"])
        rep = self.nh // self.nkv
        mask = torch.ones(T, T, dtype=torch.bool, device=self.dev).triu(1)

        def attend(i, q, k, v, out):
            qf = q.reshape(T, self.nh, self.hd).transpose(0, 1).float().contiguous()
            kf = k.reshape(T, self.nkv, self.hd).transpose(0, 1)
            vf = v.reshape(T, self.nkv, self.hd).transpose(0, 1)
            if rep > 1:
                kf = kf.unsqueeze(1).expand(self.nkv, rep, T, self.hd).reshape(self.nh, T, self.hd)
                vf = vf.unsqueeze(1).expand(self.nkv, rep, T, self.hd).reshape(self.nh, T, self.hd)
            kf, vf = kf.float().contiguous(), vf.float().contiguous()
            att = torch.bmm(qf, kf.transpose(1, 2)) / math.sqrt(self.hd)
            att = torch.softmax(att.masked_fill(mask, float("-inf")), dim=-1)
            out.view(T, self.nh, self.hd).copy_(torch.bmm(att, vf).transpose(0, 1))
            self.launches += 12

        self._layers(b, T, positions_i64, slots_i64, attend)
        rk.fused_add_rms_norm(b["x"], b["res"], self.norm, self.eps)
        logits = torch.mm(b["x"][T - 1:T], self.head.t()).float()
        return torch.argmax(torch.log_softmax(logits, dim=-1), dim=-1)


class DecodeBatch:
    """`batch` requests of `context` cached tokens each with pages of their own, and the per-step inputs the
    reference's worker prepares for decoding (core/src/worker/model_worker.rs:381-505): token ids, positions,
    slot mapping, block tables, context lengths, staged in pinned host memory and copied every step."""

    def __init__(self, model: ReferenceLlama, batch: int, context: int, first_page: int = 0, seed: int = 0):
        self.m, self.batch, self.context = model, batch, context
        bs = model.bs
        self.max_blocks = -(-(context + 600) // bs)
        g = torch.Generator().manual_seed(seed)
        pages = (torch.randperm(batch * self.max_blocks, generator=g) + first_page).view(batch, self.max_blocks)
        self.tables_host = pages.to(torch.int32).pin_memory()
        self.len = [context - 1] * batch               # cached tokens so far
        self.tok_host = torch.zeros(batch, dtype=torch.int64).pin_memory()
        self.pos_host = torch.zeros(batch, dtype=torch.int64).pin_memory()
        self.slot_host = torch.zeros(batch, dtype=torch.int64).pin_memory()
        self.ctx_host = torch.zeros(batch, dtype=torch.int32).pin_memory()
        dev = model.dev
        self.tok, self.pos, self.slot = (torch.zeros(batch, dtype=torch.int64, device=dev) for _ in range(3))
        self.ctx = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.tables = torch.zeros(batch, self.max_blocks, dtype=torch.int32, device=dev)
        self.out_host = torch.zeros(batch, dtype=torch.int64).pin_memory()
        self.h2d_bytes = sum(t.numel() * t.element_size() for t in (self.tok_host, self.pos_host, self.slot_host,
                                                                    self.ctx_host, self.tables_host))
        self.d2h_bytes = self.out_host.numel() * 8

    def pages_needed(self) -> int:
        return self.batch * self.max_blocks

    def step(self, tokens: List[int], copy: bool = True, read_back: bool = True):
        """One decode step from host token ids to host token ids."""
        bs = self.m.bs
        for j in range(self.batch):
            p = self.len[j]
            self.tok_host[j] = tokens[j]
            self.pos_host[j] = p
            self.slot_host[j] = int(self.tables_host[j, p // bs]) * bs + p % bs
            self.ctx_host[j] = p + 1
        if copy:
            self.tok.copy_(self.tok_host, non_blocking=True)
            self.pos.copy_(self.pos_host, non_blocking=True)
            self.slot.copy_(self.slot_host, non_blocking=True)
            self.ctx.copy_(self.ctx_host, non_blocking=True)
            self.tables.copy_(self.tables_host, non_blocking=True)
        out = self.m.decode_step(self.tok, self.pos, self.slot, self.tables, self.ctx, max(self.len) + 1)
        for j in range(self.batch):
            self.len[j] += 1
        if read_back:
            self.out_host.copy_(out, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            return self.out_host.tolist()
        return out

    def rewind(self, n: int) -> None:
        for j in range(self.batch):
            self.len[j] -= n
