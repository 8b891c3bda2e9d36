"""The Python entry point: `LLM(...).generate(prompt_token_ids, SamplingParams(...))`.

The reference is driven from Rust (example/examples/llm_engine_example.rs:65-151: add requests,
loop `step` while `has_unfinished_requests`); this class is that loop with the engine's options as
keywords named like the reference's flags (core/src/common/config.rs:11-87).
"""
from __future__ import annotations

from typing import Hashable, List, Optional, Sequence, Tuple, Union

from ..config.engine_config import EngineArgs
from ..sampling.params import SamplingParams
from .llm_engine import LLMEngine
from .sequence import RequestOutput


class LLM:
    def __init__(self, model: str, dtype: Optional[str] = None, block_size: int = 16,
                 gpu_memory_utilization: float = 0.9, max_model_len: Optional[int] = None,
                 max_num_batched_tokens: Optional[int] = None, max_num_seqs: int = 256, seed: int = 0,
                 num_gpu_blocks: Optional[int] = None, enforce_eager: bool = False, load_format: str = "auto",
                 async_scheduling: bool = True,
                 device: str = "cuda:0"):
        self.engine = LLMEngine(EngineArgs(model=model, max_num_batched_tokens=max_num_batched_tokens,
                                           max_num_seqs=max_num_seqs, max_model_len=max_model_len,
                                           block_size=block_size, seed=seed,
                                           gpu_memory_utilization=gpu_memory_utilization, dtype=dtype,
                                           num_gpu_blocks=num_gpu_blocks, enforce_eager=enforce_eager,
                                           no_async_scheduling=not async_scheduling),
                                device=device, load_format=load_format)
        self._next_id = 0

    def generate(self, prompts: Optional[Union[str, Sequence[str]]] = None,
                 sampling_params: Optional[Union[SamplingParams, Sequence[SamplingParams]]] = None,
                 prompt_token_ids: Optional[Sequence[Sequence[int]]] = None) -> List[RequestOutput]:
        """Runs all prompts to their end; outputs come back in the order of the prompts."""
        if prompt_token_ids is None:
            if prompts is None:
                raise ValueError("give prompts or prompt_token_ids")
            prompts = [prompts] if isinstance(prompts, str) else list(prompts)
            n = len(prompts)
        else:
            n = len(prompt_token_ids)
            prompts = [None] * n
        if sampling_params is None:
            sampling_params = SamplingParams()
        params = [sampling_params] * n if isinstance(sampling_params, SamplingParams) else list(sampling_params)
        if len(params) != n:
            raise ValueError("one SamplingParams for all prompts, or one per prompt")
        ids = []
        for i in range(n):
            rid = self._next_id
            self._next_id += 1
            ids.append(rid)
            self.engine.add_request(rid, prompts[i], params[i],
                                    prompt_token_ids[i] if prompt_token_ids is not None else None)
        done = {}
        while self.engine.has_unfinished_requests():
            for out in self.engine.step():
                if out.finished:
                    done[out.request_id] = out
        return [done[r] for r in ids]

    def step_logits(self, entries: Sequence[Tuple[Hashable, Sequence[int], Sequence[int]]],
                    end: Sequence[Hashable] = ()) -> "torch.Tensor":
        """One call of the step function, as `bin/trace_run` makes it, for tests and for looking at a model: each
        entry is (request id, its next tokens, the places among them whose logits are wanted); all entries run as
        one batch from the cache that earlier calls left.  Returns float32 logits [wanted, vocab] on the host, in the
        order of the entries and of their wanted places.  Requests named in `end` give back what they hold after the
        step.  Nothing is sampled.  The requests live in the engine's own cache manager under ids of their own
        (("step_logits", id)), so the pages they hold until they are ended are not available to generate()."""
        from .model_runner import StepEntry
        mgr = self.engine.cache
        batch = []
        for rid, tokens, want in entries:
            key = ("step_logits", rid)
            if not mgr.has(key):
                mgr.add(key)
            batch.append(StepEntry(key, list(tokens), list(want)))
        logits = self.engine.runner.step(batch, mgr) if batch else None
        out = logits.to("cpu", copy=True) if logits is not None else None
        for rid in end:
            if mgr.has(("step_logits", rid)):
                mgr.free(("step_logits", rid))
        return out
