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

from ..cache.manager import OutOfPages
from ..cache import native
from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage, plan_groups, split_pages
from ..parts.base import Q_TILE, CacheGroupView, StepContext
from ..parts.decoder import DecoderModel
from .. import kernels


@dataclass
class StepEntry:
    """The next tokens of one request; `want`: places among them whose logits are asked for.
    `last_from`: when not None, the entry's LAST token is not known on the host yet: it is element `last_from`
    of the device tensor given to `step(..., pending_tokens=...)` (the value in `tokens` is a placeholder)."""
    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)
    last_from: Optional[int] = None


class StepError(RuntimeError):
    pass


@dataclass
class _HostBatch:
    pinned: torch.Tensor
    event: "torch.cuda.Event"
    total: int
    seg: dict
    N: int
    S: int
    q_lens: List[int]
    ctx_lens: List[int]
    slots: List[int]
    max_blocks: List[int]
    n_dec: int
    n_tiles: int
    n_tiles128: int = 0
    has_patches: bool = False


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


class ModelRunner:
    def __init__(self, model: DecoderModel, dtype: torch.dtype, device: torch.device, block_size: int,
                 num_blocks: Optional[List[int]] = None, max_num_seqs: int = 256,
                 gpu_memory_utilization: float = 0.9, max_model_len: Optional[int] = None,
                 activation_reserve_bytes: int = 0, enforce_eager: bool = False):
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
        self.error_flag = kernels.error_word(device)      # shared with the kernels that have no step context
        self.vocab_size = model.spec.vocab_size
        self.h2d_bytes = 0          # bytes of step inputs copied from pinned host memory so far
        self._ring = [(None, None)] * 4
        self._ring_pos = 0
        # CUDA graphs of decode steps
        self.enforce_eager = enforce_eager
        self.max_graph_batch = max_num_seqs
        self.graph_safe = all(getattr(part, "graph_safe", False) for part, _ in model.parts_with_specs())
        self._graphs = {}
        self._seen_sizes = set()
        self._graph_pool = None
        self._capture_stream = None

    def make_cache_manager(self) -> CacheManager:
        return self.storage.make_manager()

    # ------------------------------------------------------------------ building a batch
    def _prepare(self, entries: Sequence[StepEntry], mgr: CacheManager, static_blocks: Optional[int] = None,
                 pad_to: int = 0) -> "_HostBatch":
        """Checks the entries, reserves the pages they need (all or nothing) and lays the batch out in one
        int32 host buffer whose segments are 16-byte aligned."""
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            if len(e.tokens) == 0:
                raise StepError(f"request {e.request_id!r} brings no tokens")
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

        # the layout itself is made by the native runtime, straight into pinned memory
        S = len(entries)
        n_groups = len(self.storage.groups)
        q_lens = [len(e.tokens) for e in entries]
        tok = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        if tok.min() < 0 or tok.max() >= self.vocab_size:
            for rid in reserved:
                mgr.rollback(rid)
            for e in entries:
                bad = [int(t) for t in e.tokens if not (0 <= int(t) < self.vocab_size)]
                if bad:
                    raise StepError(f"request {e.request_id!r}: token id {bad[0]} is outside the vocabulary "
                                    f"(0..{self.vocab_size - 1})")
        tok = np.ascontiguousarray(tok, dtype=np.int32)
        rids = np.fromiter((mgr.native_id(e.request_id) for e in entries), dtype=np.int64, count=S)
        q_arr = np.asarray(q_lens, dtype=np.int32)
        want_counts = np.fromiter((len(e.want) for e in entries), dtype=np.int32, count=S)
        want_flat = np.fromiter((int(w) for e in entries for w in e.want), dtype=np.int32, count=int(want_counts.sum()))
        last_from = np.fromiter((-1 if e.last_from is None else int(e.last_from) for e in entries), dtype=np.int32, count=S)
        seg_arr = np.zeros(2 * (14 + max(n_groups, 1)), dtype=np.int32)
        info = np.zeros(7 + max(n_groups, 1), dtype=np.int32)
        S_pad = max(S, pad_to)
        ctx_arr = np.zeros(S_pad, dtype=np.int32)
        null_pages = np.asarray(self.storage.null_pages or [0], dtype=np.int32)
        ptr = lambda arr: arr.ctypes.data
        lib, h = native.lib(), mgr.handle()
        args = (h, S, ptr(rids), ptr(q_arr), ptr(tok), ptr(want_counts), ptr(want_flat), ptr(last_from),
                int(static_blocks or 0), Q_TILE, int(pad_to), ptr(null_pages))
        rc = lib.lmsf_cm_build_batch(*args, None, 0, ptr(seg_arr), ptr(info), ptr(ctx_arr))
        if rc != 0:
            raise StepError(f"the batch could not be laid out ({rc})")
        total = int(info[6])
        pinned, event = self._pinned_buffer(total)
        rc = lib.lmsf_cm_build_batch(*args, pinned.data_ptr(), pinned.numel(), ptr(seg_arr), ptr(info), ptr(ctx_arr))
        if rc != 0:
            raise StepError(f"the batch could not be laid out ({rc})")
        names = ["token_ids", "positions", "token_seq", "cu_q", "ctx_len", "state_slot", "patch_dst", "patch_src", "rows",
                 "dec_ids", "tile_seq", "tile_q0", "tile128_seq", "tile128_q0"] + [f"bt{g}" for g in range(n_groups)]
        seg = {name: (int(seg_arr[2 * i]), int(seg_arr[2 * i + 1])) for i, name in enumerate(names)}
        slots = pinned[seg["state_slot"][0]:seg["state_slot"][0] + S_pad].tolist()
        return _HostBatch(pinned, event, total, seg, int(info[0]), S_pad, q_lens + [1] * (S_pad - S), ctx_arr.tolist(), slots,
                          [int(info[7 + g]) for g in range(n_groups)], int(info[2]), int(info[3]), int(info[4]),
                          bool(info[5]))

    def _pinned_buffer(self, n_ints: int):
        """A pinned host buffer from a small ring; a buffer is used again only after the copy that last read it."""
        self._ring_pos = (self._ring_pos + 1) % len(self._ring)
        buf, event = self._ring[self._ring_pos]
        if event is not None:
            event.synchronize()
        if buf is None or buf.numel() < n_ints:
            buf = torch.empty(max(n_ints, 4096), dtype=torch.int32).pin_memory()
        event = torch.cuda.Event()
        self._ring[self._ring_pos] = (buf, event)
        return buf, event

    def _upload(self, hb: "_HostBatch", dev: Optional[torch.Tensor] = None) -> torch.Tensor:
        if dev is None:
            dev = torch.empty(hb.total, dtype=torch.int32, device=self.device)
        dev.copy_(hb.pinned[:hb.total], non_blocking=True)
        hb.event.record()
        self.h2d_bytes += hb.total * 4
        return dev

    def _context(self, hb: "_HostBatch", dev: torch.Tensor) -> Tuple[StepContext, torch.Tensor]:
        def view(name):
            o, n = hb.seg[name]
            return dev[o:o + n]

        groups = [CacheGroupView(view(f"bt{g}").view(hb.S, hb.max_blocks[g]), self.block_size)
                  for g in range(len(hb.max_blocks))]
        ctx = StepContext(n_tokens=hb.N, n_seqs=hb.S, dtype=self.dtype, device=self.device, token_ids=view("token_ids"),
                          positions=view("positions"), token_seq=view("token_seq"), cu_q=view("cu_q"),
                          ctx_len=view("ctx_len"), state_slot=view("state_slot"), groups=groups, q_lens=hb.q_lens,
                          ctx_lens=hb.ctx_lens, state_slots=hb.slots, error_flag=self.error_flag,
                          decode_seq_ids=view("dec_ids"), n_decode_seqs=hb.n_dec, q_tile_seq=view("tile_seq"),
                          q_tile_q0=view("tile_q0"), n_q_tiles=hb.n_tiles, q_tile128_seq=view("tile128_seq"),
                          q_tile128_q0=view("tile128_q0"), n_q_tiles128=hb.n_tiles128)
        return ctx, view("rows")

    def build_context(self, entries: Sequence[StepEntry], mgr: CacheManager) -> Tuple[StepContext, torch.Tensor]:
        """The context of a step and the rows of its tokens whose logits are wanted (pages are reserved)."""
        hb = self._prepare(entries, mgr)
        return self._context(hb, self._upload(hb))

    # ------------------------------------------------------------------ the step
    @staticmethod
    def graph_batch_size(n: int) -> int:
        """Decode batches are replayed from graphs of these sizes: 1, 2, 4, then multiples of 4 up to 32 (where the
        decode attention's plan changes within a few requests: 20 requests take 4.4 ms a step on their own graph and
        4.7 ms padded to 24), then multiples of 8."""
        if n <= 2:
            return n
        if n <= 32:
            return (n + 3) // 4 * 4
        return (n + 7) // 8 * 8

    def graph_context_bucket(self, max_ctx: int) -> int:
        """The launch geometry of a captured decode step (how the keys are split over blocks) is chosen for a
        context length; a graph serves all steps whose longest context lies in the same bucket: powers of two
        from 1,024 up to the longest context the model takes."""
        b = 1024
        while b < max_ctx and b < self.max_model_len:
            b *= 2
        return min(b, max(self.max_model_len, 1))

    @staticmethod
    def graph_skew_class(bucket: int, mean_ctx: float) -> int:
        """How far the mean context of a decode batch lies below its bucket: 0 when above half of it (all batches of
        equal contexts), else the number of halvings, up to 6 (a 64th and less).  A long request among short ones is
        split into more blocks than a batch of long requests would be; the class is part of a graph's key because
        the split is part of its geometry."""
        c = 0
        while c < 6 and mean_ctx * (2 << c) <= bucket:
            c += 1
        return c

    def _graph_eligible(self, entries: Sequence[StepEntry]) -> bool:
        return (not self.enforce_eager and self.graph_safe and len(entries) <= self.max_graph_batch
                and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries))

    def _patch(self, hb: "_HostBatch", dev: torch.Tensor, pending_tokens: Optional[torch.Tensor]) -> None:
        if not hb.has_patches:
            return
        if pending_tokens is None:
            raise StepError("an entry names a pending token but no pending_tokens tensor was given")
        seg = lambda name: dev[hb.seg[name][0]:hb.seg[name][0] + hb.seg[name][1]]
        kernels.patch_tokens(seg("token_ids"), seg("patch_dst"), seg("patch_src"), pending_tokens)

    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry], mgr: CacheManager, check: bool = True,
             pending_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Runs the entries as one batch; returns float32 logits [wanted, vocab] on the device, in the order
        of the entries and of their `want`.  Afterwards the tokens count as cached (`mgr.commit`).

        A batch in which every request brings one token and wants its logits is replayed from a CUDA graph
        (batch sizes are rounded up to 1, 2, a multiple of 4 up to 32 or a multiple of 8 with stand-in requests that touch only a
        spare page; there is a graph per batch size and bucket of context lengths, captured the second time
        the pair is seen); the returned tensor is then a view
        of the graph's own output buffer and holds its values until the next step of the same size."""
        graph_mode = self._graph_eligible(entries)
        bucket = skew = 0
        if graph_mode:
            lens = [mgr.num_tokens(e.request_id) + 1 for e in entries]
            bucket = self.graph_context_bucket(max(lens))
            skew = self.graph_skew_class(bucket, sum(lens) / len(lens))
        # a graph's block tables are as wide as its bucket of context lengths needs, not as the longest context allowed
        hb = self._prepare(entries, mgr, (bucket + self.block_size - 1) // self.block_size if graph_mode else None,
                           self.graph_batch_size(len(entries)) if graph_mode else 0)
        self.storage.zero_state_slots(mgr.take_fresh_slots())
        key = (hb.S, bucket, skew) if graph_mode else None
        if graph_mode and (key in self._graphs or key in self._seen_sizes):
            logits = self._replay(hb, key, pending_tokens)
        else:
            if graph_mode:
                self._seen_sizes.add(key)
            dev = self._upload(hb)
            self._patch(hb, dev, pending_tokens)
            ctx, rows = self._context(hb, dev)
            logits = self.model.forward(ctx, self.storage.layer_caches, rows)
        for e in entries:
            mgr.commit(e.request_id, len(e.tokens))
        if check:
            self.check_device_errors()
        return logits[:len(entries)] if graph_mode else logits

    def _replay(self, hb: "_HostBatch", key: Tuple[int, int, int], pending_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        g = self._graphs.get(key)
        if g is None:
            static_in = self._upload(hb)
            ctx, rows = self._context(hb, static_in)
            # launch geometry must not depend on the step, only on its bucket: the decode attention plans its splits
            # for the middle of the bucket's context lengths (the bucket below ends at half its top)
            ctx.extras["decode_max_ctx"] = key[1] - key[1] // 4 if key[1] > 1024 else key[1]
            # the middle of the graph's class of means: between bucket / (2 << c) and twice that (the last class: and
            # below); class 0 plans as if all contexts were as long as the longest
            ctx.extras["decode_mean_ctx"] = key[1] * 3 / (4 << key[2]) if key[2] else ctx.extras["decode_max_ctx"]
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
                self._capture_stream = torch.cuda.Stream(self.device)
            # Captured on a side stream with capture_begin / capture_end directly: the torch.cuda.graph context
            # would also empty the allocator's cache, which costs milliseconds for every batch size.
            graph = torch.cuda.CUDAGraph()
            before = kernels.launch_count()
            side = self._capture_stream
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                graph.capture_begin(pool=self._graph_pool)
                try:
                    static_out = self.model.forward(ctx, self.storage.layer_caches, rows)
                finally:
                    graph.capture_end()
            torch.cuda.current_stream(self.device).wait_stream(side)
            n_launches = kernels.launch_count() - before
            kernels.add_launches(-n_launches)                      # recorded, not run
            g = self._graphs[key] = (graph, static_in, static_out, n_launches, hb.total)
        graph, static_in, static_out, n_launches, total = g
        if total != hb.total:
            raise StepError("the layout of a replayed batch changed")
        self._upload(hb, static_in)
        self._patch(hb, static_in, pending_tokens)
        graph.replay()
        kernels.add_launches(n_launches)
        return static_out

    def decode_step(self, entries: Sequence[StepEntry], mgr: CacheManager) -> torch.Tensor:
        """A step whose entries all bring one token; device errors are left for the caller to check."""
        return self.step(entries, mgr, check=False)

    def check_device_errors(self) -> None:
        code = int(self.error_flag.item())
        if code:
            self.error_flag.zero_()
            what = {1: "a token id outside the vocabulary reached the embedding",
                    2: "a token was to be cached at a position that has no page",
                    3: "a tensor-core attention block gave up waiting for its own products",
                    4: "a block of the streaming matrix product gave up waiting for its own copies or products"}.get(code, f"code {code}")
            raise StepError(f"the device reported an error during the step: {what}")
