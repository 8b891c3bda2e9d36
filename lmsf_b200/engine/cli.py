"""Command line in the manner of the reference's example/examples/llm_engine_example.rs: engine flags
with the reference's names (core/src/common/config.rs:11-87), a few prompts, `step` until done,
tokens and elapsed time printed."""
from __future__ import annotations

import argparse
import json
import sys
import time
from dataclasses import asdict

from ..config.engine_config import EngineArgs
from ..sampling.params import SamplingParams


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="llm_engine_example", description=__doc__)
    EngineArgs.add_cli_args(ap)
    ap.add_argument("--prompt", action="append", default=[], help="a text prompt (needs tokenizer.json); repeatable")
    ap.add_argument("--prompt-ids", action="append", default=[],
                    help="a prompt as comma-separated token ids; repeatable")
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--top-k", type=int, default=-1)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--min-p", type=float, default=0.0)
    ap.add_argument("--presence-penalty", type=float, default=0.0)
    ap.add_argument("--frequency-penalty", type=float, default=0.0)
    ap.add_argument("--repetition-penalty", type=float, default=1.0)
    ap.add_argument("--max-tokens", type=int, default=128)
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--load-format", default="auto", choices=["auto", "dummy"],
                    help="dummy: random weights made on the device from config.json alone")
    ap.add_argument("--step-stats", action="store_true", help="print one JSON line of counters per step")
    ns = ap.parse_args(argv)

    from .llm_engine import LLMEngine
    engine = LLMEngine(EngineArgs.from_cli_args(ns), load_format=ns.load_format)
    sp = SamplingParams(temperature=ns.temperature, top_k=ns.top_k, top_p=ns.top_p, min_p=ns.min_p,
                        presence_penalty=ns.presence_penalty, frequency_penalty=ns.frequency_penalty,
                        repetition_penalty=ns.repetition_penalty, max_tokens=ns.max_tokens, ignore_eos=ns.ignore_eos)
    rid = 0
    for text in ns.prompt:
        engine.add_request(rid, text, sp)
        rid += 1
    for ids in ns.prompt_ids:
        engine.add_request(rid, None, sp, prompt_token_ids=[int(t) for t in ids.split(",") if t.strip()])
        rid += 1
    if rid == 0:
        if engine.tokenizer is not None:
            engine.add_request(0, "To be or not to be, ", sp)     # the reference's own prompt
        else:
            engine.add_request(0, None, sp, prompt_token_ids=[1])
    from ..utils.tracing import profiler_start, profiler_stop
    profiler_start()                # with LMSF_NVTX=1: the generation is the profiler's region of interest
    start = time.perf_counter()
    steps = generated = 0
    while engine.has_unfinished_requests():
        for out in engine.step():
            generated += 1
            if out.finished:
                c = out.outputs[0]
                print(json.dumps({"request_id": out.request_id, "finish_reason": c.finish_reason,
                                  "token_ids": c.token_ids, "text": c.text,
                                  "metrics": out.metrics.summary(len(c.token_ids))}))
        steps += 1
        if ns.step_stats:
            print(json.dumps(asdict(engine.last_stats)), file=sys.stderr)
    dt = time.perf_counter() - start
    profiler_stop()
    print(f"End cost {dt:.3f}s to gen {generated} tokens in {steps} steps ({generated / max(dt, 1e-9):.1f} tok/s)",
          file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
