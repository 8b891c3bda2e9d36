"""The engine: requests in, tokens out, one `step` at a time.

Same verbs as the reference's LLMEngine (core/src/engine/llm_engine.rs:74-183, :536-582):
`add_request`, `abort_request`, `step`, `has_unfinished_requests`, `get_num_unfinished_requests`.
A step is schedule -> run the batch -> sample -> append, stop tests, free (llm_engine.rs:536-582,
:315-398); the stop tests are those of check_stop (llm_engine.rs:221-258) that work on token ids.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence as Seq

import torch

from ..config.engine_config import CacheConfig, EngineArgs, SchedulerConfig, resolve_max_model_len
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .factory import build_model
from .model_runner import ModelRunner, StepEntry
from .scheduler import Scheduler, SchedulerOutputs
from .sequence import RequestOutput, Sequence, SequenceStatus


@dataclass
class StepStats:
    """What one step did (printed as JSON by the command line)."""
    num_prefill_tokens: int = 0
    num_decode_tokens: int = 0
    num_running: int = 0
    num_waiting: int = 0
    num_preempted: int = 0
    free_pages: int = 0
    step_ms: float = 0.0


class LLMEngine:
    def __init__(self, args: EngineArgs, device: str = "cuda:0", load_format: str = "auto"):
        self.args = args
        self.device = torch.device(device)
        self.model, self.model_config, self.dtype = build_model(args.model, args.dtype, self.device, load_format,
                                                                args.seed)
        self.max_model_len = resolve_max_model_len(args.max_model_len, self.model.spec.max_model_len)
        self.cache_config = CacheConfig(args.block_size, args.gpu_memory_utilization, args.num_gpu_blocks)
        self.scheduler_config = SchedulerConfig.new(args.max_num_batched_tokens, args.max_num_seqs, self.max_model_len)
        act_bytes = self.scheduler_config.max_num_batched_tokens * self.model.spec.hidden_size * 64
        self.runner = ModelRunner(self.model, self.dtype, self.device, args.block_size,
                                  num_blocks=args.num_gpu_blocks, max_num_seqs=args.max_num_seqs,
                                  gpu_memory_utilization=args.gpu_memory_utilization,
                                  max_model_len=self.max_model_len, activation_reserve_bytes=act_bytes,
                                  enforce_eager=args.enforce_eager)
        self.cache = self.runner.make_cache_manager()
        if self.cache.groups and all(g.window is None for g in self.cache.groups) and \
                args.block_size * self.cache.num_total_pages(0) < self.max_model_len and args.num_gpu_blocks is None:
            # core/src/worker/model_worker.rs:115-118
            raise RuntimeError(f"the cache holds {args.block_size * self.cache.num_total_pages(0)} tokens, fewer "
                               f"than max_model_len={self.max_model_len}; raise gpu_memory_utilization or lower "
                               f"max_model_len")
        self.scheduler = Scheduler(self.scheduler_config, self.cache)
        self.sampler = Sampler(self.device)
        self.eos_token_ids = set(self.model.spec.eos_token_ids)
        self.tokenizer = self._load_tokenizer(args.model)
        self.seqs: Dict[Hashable, Sequence] = {}
        self.last_stats = StepStats()
        self._auto_id = 0

    @staticmethod
    def _load_tokenizer(model_dir: str):
        path = os.path.join(model_dir, "tokenizer.json")
        if not os.path.isfile(path):
            return None
        try:
            from tokenizers import Tokenizer   # the library the reference uses (llm_engine.rs:93-100)
        except ImportError:
            return None
        return Tokenizer.from_file(path)

    # ------------------------------------------------------------------ requests
    def add_request(self, request_id: Hashable, prompt: Optional[str], sampling_params: SamplingParams,
                    prompt_token_ids: Optional[Seq[int]] = None, arrival_time: Optional[float] = None) -> None:
        if request_id in self.seqs:
            raise KeyError(f"request {request_id!r} is already known")
        if prompt_token_ids is None:
            if self.tokenizer is None:
                raise ValueError("a text prompt needs tokenizer.json in the model folder; pass prompt_token_ids")
            prompt_token_ids = self.tokenizer.encode(prompt, add_special_tokens=True).ids
        ids = [int(t) for t in prompt_token_ids]
        if not ids:
            raise ValueError("a request needs at least one prompt token")
        vocab = self.model.spec.vocab_size
        bad = [t for t in ids if not (0 <= t < vocab)]
        if bad:
            raise ValueError(f"prompt token ids {bad[:5]} are outside the vocabulary (0..{vocab - 1})")
        if sampling_params.filters_active or sampling_params.penalties_active:
            self.sampler.require_filters()
        seed = sampling_params.seed if sampling_params.seed is not None else \
            (self.args.seed * 0x9E3779B97F4A7C15 + self._auto_id + 1) & 0xFFFFFFFFFFFFFFFF
        self._auto_id += 1
        seq = Sequence(request_id, ids, sampling_params, seed=seed)
        if arrival_time is not None:
            seq.arrival_time = arrival_time
        self.seqs[request_id] = seq
        self.scheduler.add_seq(seq)

    def abort_request(self, request_id: Hashable) -> None:
        self.scheduler.abort_seq(request_id)
        self.seqs.pop(request_id, None)

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_unfinished_seqs()

    def get_num_unfinished_requests(self) -> int:
        return self.scheduler.get_num_unfinished_seqs()

    # ------------------------------------------------------------------ the step
    def _check_stop(self, seq: Sequence) -> None:
        """core/src/engine/llm_engine.rs:221-258 without the string tests."""
        sp = seq.sampling_params
        last = seq.output_token_ids[-1]
        if last in sp.stop_token_ids:
            seq.status = SequenceStatus.FINISHED_STOPPED
        elif len(seq) >= self.max_model_len:
            seq.status = SequenceStatus.FINISHED_LENGTH
        elif len(seq.output_token_ids) >= sp.max_tokens:
            seq.status = SequenceStatus.FINISHED_LENGTH
        elif not sp.ignore_eos and last in self.eos_token_ids:
            seq.status = SequenceStatus.FINISHED_STOPPED

    def step(self) -> List[RequestOutput]:
        t0 = time.perf_counter()
        sched: SchedulerOutputs = self.scheduler.schedule()
        outputs: List[RequestOutput] = []
        for seq in sched.ignored:
            seq.finish_time = time.monotonic()
            outputs.append(self._output(seq))
            self.seqs.pop(seq.request_id, None)
        stats = StepStats(num_preempted=len(sched.preempted))
        if not sched.is_empty:
            entries, sampled = [], []
            for e in sched.entries:
                entries.append(StepEntry(e.seq.request_id, e.seq.next_tokens(e.num_tokens),
                                         [e.num_tokens - 1] if e.wants_logits else []))
                if e.wants_logits:
                    sampled.append(e.seq)
                if e.num_tokens == 1 and e.start >= len(e.seq.prompt_token_ids):
                    stats.num_decode_tokens += 1
                else:
                    stats.num_prefill_tokens += e.num_tokens
            logits = self.runner.step(entries, self.cache, check=False)
            tokens: List[int] = []
            if sampled:
                tok = self.sampler.sample(logits, [s.sampling_params for s in sampled], [s.seed for s in sampled],
                                          [len(s.output_token_ids) for s in sampled], sampled)
                tokens = tok.tolist()                 # the step's one device-to-host read
            self.runner.check_device_errors()
            for e in sched.entries:
                e.seq.num_computed += e.num_tokens
            now = time.monotonic()
            for seq, t in zip(sampled, tokens):
                seq.output_token_ids.append(int(t))
                if seq.first_token_time is None:
                    seq.first_token_time = now
                self._check_stop(seq)
                if seq.status.finished:
                    seq.finish_time = now
                    self.scheduler.free_seq(seq)
                    self.seqs.pop(seq.request_id, None)
                outputs.append(self._output(seq))
        stats.num_running = len(self.scheduler.running)
        stats.num_waiting = len(self.scheduler.waiting)
        stats.free_pages = self.cache.num_free_pages(0) if self.cache.groups else 0
        stats.step_ms = (time.perf_counter() - t0) * 1e3
        self.last_stats = stats
        return outputs

    def _output(self, seq: Sequence) -> RequestOutput:
        text = None
        if self.tokenizer is not None:
            text = self.tokenizer.decode(seq.output_token_ids, skip_special_tokens=True)
        return RequestOutput.from_sequence(seq, text)
