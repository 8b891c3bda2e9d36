"""The step function: one batch of (request, its next tokens) through the model, from the cache.

The reference's Worker builds either a padded batch of whole prompts or a batch of single decode
tokens (core/src/worker/model_worker.rs:213-264, :266-353, :427-505) and samples inside the same
call.  Here a step takes any mix of prompt portions and decoded tokens as one flat batch, runs
only the tokens it is given and returns float32 logits at the wanted places; sampling is apart.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.block_allocator import OutOfPages
from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage, plan_groups, split_pages
from ..parts.base import Q_TILE, CacheGroupView, StepContext
from ..parts.decoder import DecoderModel


@dataclass
class StepEntry:
    """The next tokens of one request; `want`: places among them whose logits are asked for."""
    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)


class StepError(RuntimeError):
    pass


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


class ModelRunner:
    def __init__(self, model: DecoderModel, dtype: torch.dtype, device: torch.device, block_size: int,
                 num_blocks: Optional[List[int]] = None, max_num_seqs: int = 256,
                 gpu_memory_utilization: float = 0.9, max_model_len: Optional[int] = None,
                 activation_reserve_bytes: int = 0):
        if device.type != "cuda":
            raise StepError("lmsf_b200 runs on a CUDA device only; there is no CPU path")
        self.model, self.dtype, self.device, self.block_size = model, dtype, device, block_size
        self.max_model_len = max_model_len or model.spec.max_model_len
        self.max_num_seqs = max_num_seqs
        groups, _ = plan_groups(model)
        if num_blocks is None:
            # pages from what is free after the weights are on the device
            # (core/src/worker/model_worker.rs:146-153: total * utilization - used)
            free, total = torch.cuda.mem_get_info(device)
            budget = int(total * gpu_memory_utilization) - (total - free) - activation_reserve_bytes
            if budget <= 0:
                raise StepError("no memory is left for the cache; raise gpu_memory_utilization")
            num_blocks = split_pages(groups, block_size, dtype, budget, self.max_model_len)
        elif isinstance(num_blocks, int):
            num_blocks = [num_blocks] * len(groups)
        self.storage = CacheStorage(model, block_size, num_blocks, max_num_seqs, dtype, device)
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=device)
        self.vocab_size = model.spec.vocab_size
        self.h2d_bytes = 0          # bytes of step inputs copied from pinned host memory so far

    def make_cache_manager(self) -> CacheManager:
        return self.storage.make_manager()

    # ------------------------------------------------------------------ building a batch
    def build_context(self, entries: Sequence[StepEntry], mgr: CacheManager,
                      pad_blocks_to: Optional[int] = None) -> Tuple[StepContext, torch.Tensor]:
        """Reserves the pages the entries need (all or nothing) and lays the batch out on the device.
        Returns the context and the int32 rows of the step's tokens whose logits are wanted."""
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            if len(e.tokens) == 0:
                raise StepError(f"request {e.request_id!r} brings no tokens")
            for t in e.tokens:
                if not (0 <= int(t) < self.vocab_size):
                    raise StepError(f"request {e.request_id!r}: token id {t} is outside the vocabulary "
                                    f"(0..{self.vocab_size - 1})")
            for w in e.want:
                if not (0 <= int(w) < len(e.tokens)):
                    raise StepError(f"request {e.request_id!r}: wanted place {w} is outside its {len(e.tokens)} tokens")
            if mgr.num_tokens(e.request_id) + len(e.tokens) > self.max_model_len:
                raise StepError(f"request {e.request_id!r} would exceed max_model_len={self.max_model_len}")
        reserved = []
        try:
            for e in entries:
                lack = mgr.num_tokens(e.request_id) + len(e.tokens) - mgr.num_reserved(e.request_id)
                if lack > 0:
                    mgr.reserve(e.request_id, lack)
                    reserved.append(e.request_id)
        except OutOfPages:
            for rid in reserved:
                mgr.rollback(rid)
            raise

        S = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        starts = [mgr.num_tokens(e.request_id) for e in entries]
        ctx_lens = [s + n for s, n in zip(starts, q_lens)]
        N = sum(q_lens)
        rows: List[int] = []
        off = 0
        for e, n in zip(entries, q_lens):
            rows.extend(off + int(w) for w in e.want)
            off += n
        dec_ids = [i for i, n in enumerate(q_lens) if n == 1]
        tile_seq = [i for i, n in enumerate(q_lens) if n > 1 for _ in range(0, n, Q_TILE)]
        tile_q0 = [q0 for n in q_lens if n > 1 for q0 in range(0, n, Q_TILE)]
        n_groups = len(self.storage.groups)
        tables = [[mgr.block_table(e.request_id, g) for e in entries] for g in range(n_groups)]
        max_blocks = [max(pad_blocks_to or 1, max(len(t) for t in tables[g])) for g in range(n_groups)]

        # one int32 buffer, every segment 16-byte aligned
        seg = {}
        total = 0
        for name, length in [("token_ids", N), ("positions", N), ("token_seq", N), ("cu_q", S + 1), ("ctx_len", S),
                             ("state_slot", S), ("rows", len(rows)), ("dec_ids", len(dec_ids)),
                             ("tile_seq", len(tile_seq)), ("tile_q0", len(tile_q0))] + \
                            [(f"bt{g}", S * max_blocks[g]) for g in range(n_groups)]:
            seg[name] = (total, length)
            total += _align(max(length, 1))
        host = np.full(total, -1, dtype=np.int32)

        def put(name, values):
            o, n = seg[name]
            host[o:o + n] = values

        put("token_ids", np.fromiter((int(t) for e in entries for t in e.tokens), dtype=np.int32, count=N))
        put("positions", np.concatenate([np.arange(s, s + n, dtype=np.int32) for s, n in zip(starts, q_lens)]))
        put("token_seq", np.repeat(np.arange(S, dtype=np.int32), q_lens))
        put("cu_q", np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32))
        put("ctx_len", np.asarray(ctx_lens, dtype=np.int32))
        slots = [mgr.state_slot(e.request_id) for e in entries]
        put("state_slot", np.asarray(slots, dtype=np.int32))
        for name, values in (("rows", rows), ("dec_ids", dec_ids), ("tile_seq", tile_seq), ("tile_q0", tile_q0)):
            if values:
                put(name, np.asarray(values, dtype=np.int32))
        for g in range(n_groups):
            o, _ = seg[f"bt{g}"]
            bt = host[o:o + S * max_blocks[g]].reshape(S, max_blocks[g])
            for i, t in enumerate(tables[g]):
                bt[i, :len(t)] = t
        dev = torch.from_numpy(host).pin_memory().to(self.device, non_blocking=True)
        self.h2d_bytes += host.nbytes

        def view(name):
            o, n = seg[name]
            return dev[o:o + n]

        groups = [CacheGroupView(view(f"bt{g}").view(S, max_blocks[g]), self.block_size) for g in range(n_groups)]
        ctx = StepContext(n_tokens=N, n_seqs=S, dtype=self.dtype, device=self.device, token_ids=view("token_ids"),
                          positions=view("positions"), token_seq=view("token_seq"), cu_q=view("cu_q"),
                          ctx_len=view("ctx_len"), state_slot=view("state_slot"), groups=groups, q_lens=q_lens,
                          ctx_lens=ctx_lens, state_slots=slots, error_flag=self.error_flag,
                          decode_seq_ids=view("dec_ids"), n_decode_seqs=len(dec_ids), q_tile_seq=view("tile_seq"),
                          q_tile_q0=view("tile_q0"), n_q_tiles=len(tile_seq))
        return ctx, view("rows")

    # ------------------------------------------------------------------ the step
    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry], mgr: CacheManager, check: bool = True) -> torch.Tensor:
        """Runs the entries as one batch; returns float32 logits [wanted, vocab] on the device, in the order
        of the entries and of their `want`.  Afterwards the tokens count as cached (`mgr.commit`)."""
        ctx, rows = self.build_context(entries, mgr)
        self.storage.zero_state_slots(mgr.take_fresh_slots())
        logits = self.model.forward(ctx, self.storage.layer_caches, rows)
        for e in entries:
            mgr.commit(e.request_id, len(e.tokens))
        if check:
            self.check_device_errors()
        return logits

    def decode_step(self, entries: Sequence[StepEntry], mgr: CacheManager) -> torch.Tensor:
        """A step whose entries all bring one token; device errors are left for the caller to check."""
        return self.step(entries, mgr, check=False)

    def check_device_errors(self) -> None:
        code = int(self.error_flag.item())
        if code:
            self.error_flag.zero_()
            what = {1: "a token id outside the vocabulary reached the embedding",
                    2: "a token was to be cached at a position that has no page"}.get(code, f"code {code}")
            raise StepError(f"the device reported an error during the step: {what}")
