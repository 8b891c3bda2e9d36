"""Turns the logits of a step into one token per sampled request.

Greedy and temperature sampling run in one kernel (csrc/sampling.cu).  Reference:
Sampler::forward, core/src/model_executor/layers/sampler.rs:839-971.
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from .. import kernels
from .params import SamplingParams


class Sampler:
    def __init__(self, device: torch.device):
        self.device = device

    def require_filters(self) -> None:
        raise NotImplementedError("top_k, top_p, min_p and the penalties are not available in this build")

    @torch.inference_mode()
    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               steps: Sequence[int], seqs=None) -> torch.Tensor:
        """logits: float32 [rows, vocab]; row r is sampled with params[r]; `steps[r]` is the index of the
        output token being drawn, `seeds[r]` the request's seed.  Returns int32 [rows] on the device."""
        rows = logits.shape[0]
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        if rows == 0:
            return out
        if all(p.greedy for p in params):
            kernels.sample(out, logits)
            return out
        temp = torch.tensor([p.temperature for p in params], dtype=torch.float32).to(self.device, non_blocking=True)
        seed = torch.from_numpy(np.asarray([s & 0xFFFFFFFFFFFFFFFF for s in seeds], dtype=np.uint64).view(np.int64)
                                ).to(self.device, non_blocking=True)
        step = torch.tensor(list(steps), dtype=torch.int32).to(self.device, non_blocking=True)
        kernels.sample(out, logits, temp, seed, step)
        return out
