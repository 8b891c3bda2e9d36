"""Turns the logits of a step into one token per sampled request.

Order of the reference's Sampler::forward (core/src/model_executor/layers/sampler.rs:839-971): penalties,
temperature, top-k / top-p, min-p, then greedy (argmax) or random (exponential race) sampling.  Greedy and
plain temperature rows go through one kernel; rows with top-k / top-p / min-p through a second one that
finds the kept set by bisection instead of sorting the vocabulary (csrc/sampling.cu).
"""
from __future__ import annotations

from collections import Counter
from typing import Sequence

import numpy as np
import torch

from .. import kernels
from .params import SamplingParams


class Sampler:
    def __init__(self, device: torch.device):
        self.device = device

    def require_filters(self) -> None:
        """top_k, top_p, min_p and the penalties are built in; nothing to check."""

    def _dev(self, values, dtype) -> torch.Tensor:
        return torch.tensor(values, dtype=dtype).to(self.device, non_blocking=True)

    def _apply_penalties(self, logits: torch.Tensor, params: Sequence[SamplingParams], seqs) -> None:
        rows, toks, counts = [], [], []
        for r, (p, seq) in enumerate(zip(params, seqs)):
            if not p.penalties_active:
                continue
            out_counts = Counter(seq.output_token_ids)
            seen = set(seq.prompt_token_ids) | set(out_counts)
            for t in seen:
                rows.append(r)
                toks.append(t)
                counts.append(out_counts.get(t, 0))
        if not rows:
            return
        n = len(params)
        kernels.apply_penalties(logits, self._dev(rows, torch.int32), self._dev(toks, torch.int32),
                                self._dev(counts, torch.int32),
                                self._dev([p.presence_penalty for p in params], torch.float32),
                                self._dev([p.frequency_penalty for p in params], torch.float32),
                                self._dev([p.repetition_penalty for p in params], torch.float32))

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
        temp = self._dev([p.temperature for p in params], torch.float32)
        seed = torch.from_numpy(np.asarray([s & 0xFFFFFFFFFFFFFFFF for s in seeds], dtype=np.uint64).view(np.int64)
                                ).to(self.device, non_blocking=True)
        step = self._dev(list(steps), torch.int32)
        kernels.sample(out, logits, temp, seed, step)
        filtered = [r for r, p in enumerate(params) if p.filters_active]
        if filtered:
            kernels.sample_filtered(out, logits, temp, seed, step, self._dev([p.top_k for p in params], torch.int32),
                                    self._dev([p.top_p for p in params], torch.float32),
                                    self._dev([p.min_p for p in params], torch.float32),
                                    None if len(filtered) == rows else self._dev(filtered, torch.int32))
        return out
