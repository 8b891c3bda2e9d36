"""Named ranges for profilers, off unless LMSF_NVTX=1 is in the environment.

The reference wraps its layers in tracing spans (core/src/model_executor/models/llama/llama.rs:33, :157-158, :257,
:350) and brackets a run with cuProfilerStart / cuProfilerStop (core/src/engine/llm_engine.rs:761-768).  Here the
same places (an engine step, scheduling, the model's step, each layer call, sampling) become NVTX ranges that a
timeline shows; with the flag off `span` costs one test of a module constant.
"""
from __future__ import annotations

import contextlib
import os

ENABLED = os.environ.get("LMSF_NVTX", "0") not in ("", "0")


@contextlib.contextmanager
def _range(name: str):
    import torch
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


_NULL = contextlib.nullcontext()


def span(name: str):
    """A context manager: an NVTX range called `name` when tracing is on, nothing otherwise."""
    return _range(name) if ENABLED else _NULL


def profiler_start() -> None:
    """cudaProfilerStart when tracing is on (a capture limited to a region of interest)."""
    if ENABLED:
        import torch
        torch.cuda.profiler.start()


def profiler_stop() -> None:
    if ENABLED:
        import torch
        torch.cuda.profiler.stop()
