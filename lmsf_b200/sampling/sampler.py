"""Turns the logits of a step into one token per sampled request.

Order of the reference's Sampler::forward (core/src/model_executor/layers/sampler.rs:839-971): penalties,
temperature, top-k / top-p, min-p, then greedy (argmax) or random (exponential race) sampling.  Greedy and
plain temperature rows go through one kernel; rows with top-k / top-p / min-p through a second one that
finds the kept set by radix selection (six bits of an order-preserving key per pass) instead of sorting the
vocabulary (csrc/sampling.cu).
"""
from __future__ import annotations

import weakref
from typing import Dict, Sequence, Tuple

import numpy as np
import torch

from .. import kernels
from .params import SamplingParams


class _TokenHistory:
    """The distinct tokens of one request (prompt and output) with how often each occurs in the output, kept up
    to date by looking only at the output tokens that are new since the last step."""

    def __init__(self, prompt_token_ids: Sequence[int]):
        distinct = np.unique(np.asarray(prompt_token_ids, dtype=np.int32))
        self.n = int(distinct.shape[0])
        cap = max(64, 2 * self.n)
        self.tokens = np.zeros(cap, dtype=np.int32)
        self.counts = np.zeros(cap, dtype=np.int32)
        self.tokens[:self.n] = distinct
        self.where: Dict[int, int] = {int(t): i for i, t in enumerate(distinct.tolist())}
        self.seen_outputs = 0

    def update(self, output_token_ids: Sequence[int]) -> Tuple[np.ndarray, np.ndarray]:
        if len(output_token_ids) < self.seen_outputs:      # the output was cut back: count it again
            self.counts[:self.n] = 0
            self.seen_outputs = 0
        for t in output_token_ids[self.seen_outputs:]:
            i = self.where.get(t)
            if i is None:
                if self.n == self.tokens.shape[0]:
                    self.tokens = np.concatenate([self.tokens, np.zeros_like(self.tokens)])
                    self.counts = np.concatenate([self.counts, np.zeros_like(self.counts)])
                i = self.where[t] = self.n
                self.tokens[i] = t
                self.n += 1
            self.counts[i] += 1
        self.seen_outputs = len(output_token_ids)
        return self.tokens[:self.n], self.counts[:self.n]       # views: the caller copies them at once


class Sampler:
    def __init__(self, device: torch.device):
        self.device = device
        # token histories of the requests with penalties, by the identity of the request object; an entry goes
        # when its object does
        self._histories: Dict[int, Tuple["weakref.ref", _TokenHistory]] = {}

    def _history(self, seq) -> _TokenHistory:
        key = id(seq)
        entry = self._histories.get(key)
        if entry is not None and entry[0]() is seq:
            return entry[1]
        hist = _TokenHistory(seq.prompt_token_ids)
        try:
            ref = weakref.ref(seq, lambda _r, k=key, d=self._histories: d.pop(k, None))
        except TypeError:              # an object that cannot be referred to weakly: no memory between steps
            return hist
        self._histories[key] = (ref, hist)
        return hist

    def require_filters(self) -> None:
        """top_k, top_p, min_p and the penalties are built in; nothing to check."""

    def _dev(self, values, dtype) -> torch.Tensor:
        return torch.tensor(values, dtype=dtype).to(self.device, non_blocking=True)

    def _apply_penalties(self, logits: torch.Tensor, params: Sequence[SamplingParams], seqs) -> None:
        which, toks, counts = [], [], []
        for r, (p, seq) in enumerate(zip(params, seqs)):
            if not p.penalties_active:
                continue
            t, c = self._history(seq).update(seq.output_token_ids)
            which.append(r)
            toks.append(t)
            counts.append(c)
        if not which:
            return
        # one upload of integers [rows; tokens; counts] and one of the rows' three penalties
        lengths = [t.shape[0] for t in toks]
        n = sum(lengths)
        ints = np.empty((3, n), dtype=np.int32)
        ints[0] = np.repeat(np.asarray(which, dtype=np.int32), lengths)
        np.concatenate(toks, out=ints[1])
        np.concatenate(counts, out=ints[2])
        ints_dev = torch.from_numpy(ints).to(self.device, non_blocking=True)
        pen = self._dev([[p.presence_penalty for p in params], [p.frequency_penalty for p in params],
                         [p.repetition_penalty for p in params]], torch.float32)
        kernels.apply_penalties(logits, ints_dev[0], ints_dev[1], ints_dev[2], pen[0], pen[1], pen[2])

    @torch.inference_mode()
    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               steps: Sequence[int], seqs=None) -> torch.Tensor:
        """logits: float32 [rows, vocab] (changed in place when a row has penalties); row r is sampled with
        params[r]; `steps[r]` is the index of the output token being drawn, `seeds[r]` the request's seed,
        `seqs[r]` (needed for penalties) an object with prompt_token_ids and output_token_ids.
        Returns int32 [rows] on the device."""
        rows = logits.shape[0]
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        if rows == 0:
            return out
        if any(p.penalties_active for p in params):
            if seqs is None:
                raise ValueError("penalties need the token history of each row")
            self._apply_penalties(logits, params, seqs)
        if all(p.greedy for p in params):
            kernels.sample(out, logits)
            return out
        filtered = [r for r, p in enumerate(params) if p.filters_active]
        # one upload of the rows' floats and one of their integers
        if filtered:
            f = self._dev([[p.temperature for p in params], [p.top_p for p in params], [p.min_p for p in params]], torch.float32)
            i = self._dev([list(steps), [p.top_k for p in params]], torch.int32)
        else:
            f = self._dev([[p.temperature for p in params]], torch.float32)
            i = self._dev([list(steps)], torch.int32)
        temp, step = f[0], i[0]
        seed = torch.from_numpy(np.asarray([s & 0xFFFFFFFFFFFFFFFF for s in seeds], dtype=np.uint64).view(np.int64)
                                ).to(self.device, non_blocking=True)
        if len(filtered) < rows:
            kernels.sample(out, logits, temp, seed, step)
        if filtered:
            kernels.sample_filtered(out, logits, temp, seed, step, i[1], f[1], f[2],
                                    None if len(filtered) == rows else self._dev(filtered, torch.int32))
        return out
