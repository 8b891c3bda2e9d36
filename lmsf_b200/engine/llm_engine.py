"""The engine: requests in, tokens out, one `step` at a time.

Same verbs as the reference's LLMEngine (core/src/engine/llm_engine.rs:74-183, :536-582):
`add_request`, `abort_request`, `step`, `has_unfinished_requests`, `get_num_unfinished_requests`.
A step is schedule -> run the batch -> sample -> append, stop tests, free (llm_engine.rs:536-582,
:315-398); the stop tests are those of check_stop (llm_engine.rs:221-258) that work on token ids.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence as Seq

import torch

from ..config.engine_config import CacheConfig, EngineArgs, SchedulerConfig, resolve_max_model_len
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from ..utils.tracing import span
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


@dataclass
class _InFlight:
    """A batch that has been launched and whose sampled tokens have not been read."""
    sampled: List[Sequence]
    row_of: Dict[Hashable, int]
    tokens_dev: Optional[torch.Tensor] = None
    host: Optional[torch.Tensor] = None
    event: Optional["torch.cuda.Event"] = None


class LLMEngine:
    def __init__(self, args: EngineArgs, device: str = "cuda:0", load_format: str = "auto"):
        self.args = args
        self.device = torch.device(device)
        self.model, self.model_config, self.dtype = build_model(args.model, args.dtype, self.device, load_format,
                                                                args.seed)
        self.max_model_len = resolve_max_model_len(args.max_model_len, self.model.spec.max_model_len)
        self.cache_config = CacheConfig(args.block_size, args.gpu_memory_utilization, args.num_gpu_blocks)
        self.scheduler_config = SchedulerConfig.new(args.max_num_batched_tokens, args.max_num_seqs, self.max_model_len)
        # what a step of the largest allowed batch keeps alive beside the cache: per token the widest part's
        # intermediates and a few rows of the model's width (hidden state, branch output, float32 residual),
        # and the float32 logits of every request; half as much again for the allocator's slack
        esize = torch.empty(0, dtype=self.dtype).element_size()
        widest = max([part.activation_width() for part, _ in self.model.parts_with_specs()] + [0])
        per_token = (widest + 4 * self.model.spec.hidden_size) * esize + 8 * self.model.spec.hidden_size
        act_bytes = int(1.5 * (self.scheduler_config.max_num_batched_tokens * per_token
                               + 2 * args.max_num_seqs * self.model.spec.vocab_size * 4))
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
        self.vocab_size = self.model.spec.vocab_size
        self.tokenizer = self._load_tokenizer(args.model)
        self.seqs: Dict[Hashable, Sequence] = {}
        self.last_stats = StepStats()
        self._auto_id = 0
        self.async_scheduling = not args.no_async_scheduling
        self._inflight: Optional[_InFlight] = None
        self._result_ring = [None] * 4
        self._result_pos = 0

    @classmethod
    def from_parts(cls, runner, cache, scheduler_config: SchedulerConfig, sampler, vocab_size: int,
                   eos_token_ids: Seq[int], max_model_len: int, async_scheduling: bool = True, seed: int = 0) -> "LLMEngine":
        """An engine around a runner, a cache manager and a sampler that already exist (no model is loaded): the
        host-side tests drive the scheduling, the overlapped steps and the stop rules this way with a stand-in
        runner.  `runner` needs `step(entries, cache, check=, pending_tokens=)`, `error_flag` and
        `check_device_errors()`; `sampler` needs `sample(...)` and `require_filters()`."""
        eng = cls.__new__(cls)
        eng.args = EngineArgs(model="", seed=seed)
        eng.device = torch.device("cpu")
        eng.model = eng.model_config = eng.dtype = None
        eng.vocab_size = int(vocab_size)
        eng.max_model_len = int(max_model_len)
        eng.scheduler_config = scheduler_config
        eng.runner, eng.cache, eng.sampler = runner, cache, sampler
        eng.scheduler = Scheduler(scheduler_config, cache)
        eng.eos_token_ids = set(eos_token_ids)
        eng.tokenizer = None
        eng.seqs = {}
        eng.last_stats = StepStats()
        eng._auto_id = 0
        eng.async_scheduling = bool(async_scheduling)
        eng._inflight = None
        eng._result_ring = [None] * 4
        eng._result_pos = 0
        return eng

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
        vocab = self.vocab_size
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
        seq = self.scheduler.abort_seq(request_id)
        if seq is None and request_id in self.seqs:      # e.g. held out of both queues
            self.seqs[request_id].status = SequenceStatus.FINISHED_ABORTED
        self.seqs.pop(request_id, None)

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_unfinished_seqs() or self._inflight is not None

    def get_num_unfinished_requests(self) -> int:
        return self.scheduler.get_num_unfinished_seqs()

    # ------------------------------------------------------------------ the step
    def _check_stop(self, seq: Sequence) -> None:
        """core/src/engine/llm_engine.rs:221-258 without the string tests."""
        sp = seq.sampling_params
        last = seq.output_token_ids[-1]
        if last in sp.stop_token_ids:
            seq.status = SequenceStatus.FINISHED_STOPPED
        elif len(seq.prompt_token_ids) + len(seq.output_token_ids) >= self.max_model_len:
            seq.status = SequenceStatus.FINISHED_LENGTH
        elif len(seq.output_token_ids) >= sp.max_tokens:
            seq.status = SequenceStatus.FINISHED_LENGTH
        elif not sp.ignore_eos and last in self.eos_token_ids:
            seq.status = SequenceStatus.FINISHED_STOPPED

    # A step has two halves.  `_launch` schedules, runs the batch and samples on the device; `_retire` reads the
    # sampled tokens, appends them, tests the stop conditions and frees what finished.  With
    # `async_scheduling` (the default) a step launches batch k + 1 BEFORE it retires batch k: the host's work
    # for the next batch overlaps the device's work on this one, and a request's newest token goes from the
    # sampler to the next batch's input on the device (`StepEntry.last_from`).  A request that turns out to
    # have stopped at batch k has then already been run once more; that result is dropped at the next retire.
    # Requests with penalties need their token history on the host when they are sampled: a batch that holds one
    # launches its model step first, then retires the batch before it, then samples.

    def _will_finish_by_length(self, seq: Sequence) -> bool:
        n_out = len(seq.output_token_ids) + seq.num_pending
        return n_out >= seq.sampling_params.max_tokens or len(seq) >= self.max_model_len

    def _launch(self, outputs: List[RequestOutput]) -> Optional["_InFlight"]:
        t0 = time.perf_counter()
        for seq in self.scheduler.running:
            seq.hold = seq.num_pending > 0 and self._will_finish_by_length(seq)
        with span("schedule"):
            sched: SchedulerOutputs = self.scheduler.schedule()
        for seq in sched.ignored:
            seq.finish_time = time.monotonic()
            outputs.append(self._output(seq))
            self.seqs.pop(seq.request_id, None)
        stats = StepStats(num_preempted=len(sched.preempted))
        flight = None
        if not sched.is_empty:
            entries, sampled = [], []
            prev = self._inflight
            for e in sched.entries:
                last_from = None
                if e.seq.covers_pending(e.num_tokens):
                    last_from = prev.row_of[e.seq.request_id]
                entries.append(StepEntry(e.seq.request_id, e.seq.next_tokens(e.num_tokens),
                                         [e.num_tokens - 1] if e.wants_logits else [], last_from))
                if e.wants_logits:
                    sampled.append(e.seq)
                if e.num_tokens == 1 and e.start >= len(e.seq.prompt_token_ids):
                    stats.num_decode_tokens += 1
                else:
                    stats.num_prefill_tokens += e.num_tokens
            with span(f"model step ({stats.num_prefill_tokens} prompt + {stats.num_decode_tokens} decoded tokens)"):
                logits = self.runner.step(entries, self.cache, check=False,
                                          pending_tokens=prev.tokens_dev if prev is not None else None)
            flight = _InFlight(sampled=sampled, row_of={s.request_id: i for i, s in enumerate(sampled)})
            if prev is not None and any(s.sampling_params.penalties_active for s in sampled):
                # penalties count the tokens so far: the batch before is retired (its tokens read) between this
                # batch's model step, which is already running, and its sampling, which is launched behind it
                self._retire(prev, outputs)
                self._inflight = None
            if sampled:
                with span("sample"):
                    flight.tokens_dev = self.sampler.sample(
                        logits, [s.sampling_params for s in sampled], [s.seed for s in sampled],
                        [len(s.output_token_ids) + s.num_pending for s in sampled], sampled)
            # tokens and the device's error word travel to pinned memory behind the step
            n = len(sampled)
            flight.host = self._result_buffer(n + 1)
            if n:
                flight.host[:n].copy_(flight.tokens_dev, non_blocking=True)
            flight.host[n:n + 1].copy_(self.runner.error_flag, non_blocking=True)
            flight.event = torch.cuda.Event()
            flight.event.record()
            for e in sched.entries:
                e.seq.num_computed += e.num_tokens
            for s in sampled:
                s.num_pending += 1
        stats.num_running = len(self.scheduler.running)
        stats.num_waiting = len(self.scheduler.waiting)
        stats.free_pages = self.cache.num_free_pages(0) if self.cache.groups else 0
        stats.step_ms = (time.perf_counter() - t0) * 1e3
        self.last_stats = stats
        return flight

    def _result_buffer(self, n: int) -> torch.Tensor:
        self._result_pos = (self._result_pos + 1) % len(self._result_ring)
        buf = self._result_ring[self._result_pos]
        if buf is None or buf.numel() < n:
            buf = self._result_ring[self._result_pos] = torch.empty(max(n, 512), dtype=torch.int32)
            if self.device.type == "cuda":
                buf = self._result_ring[self._result_pos] = buf.pin_memory()
        return buf

    def _retire(self, flight: Optional["_InFlight"], outputs: List[RequestOutput]) -> None:
        if flight is None:
            return
        flight.event.synchronize()
        n = len(flight.sampled)
        values = flight.host[:n + 1].tolist()
        if values[n]:
            self.runner.check_device_errors()
        now = time.monotonic()
        for seq, t in zip(flight.sampled, values[:n]):
            seq.num_pending -= 1
            if seq.status.finished:          # stopped at an earlier token (or aborted): this one is dropped
                continue
            seq.output_token_ids.append(int(t))
            if seq.first_token_time is None:
                seq.first_token_time = now
            self._check_stop(seq)
            if seq.status.finished:
                seq.finish_time = now
                self.scheduler.free_seq(seq)
                self.seqs.pop(seq.request_id, None)
            outputs.append(self._output(seq))

    def step(self) -> List[RequestOutput]:
        """Runs one batch.  Returns an output for every request that received a token (with async scheduling:
        the tokens of the batch launched by the PREVIOUS call; keep calling while has_unfinished_requests())."""
        outputs: List[RequestOutput] = []
        overlap = self.async_scheduling
        if not overlap and self._inflight is not None:
            self._retire(self._inflight, outputs)
            self._inflight = None
        flight = self._launch(outputs)
        if overlap:
            self._retire(self._inflight, outputs)
            self._inflight = flight
        else:
            self._retire(flight, outputs)
        return outputs

    def _output(self, seq: Sequence) -> RequestOutput:
        text = None
        if self.tokenizer is not None:
            text = self.tokenizer.decode(seq.output_token_ids, skip_special_tokens=True)
        return RequestOutput.from_sequence(seq, text)
