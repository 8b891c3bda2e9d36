"""lmsf_b200: a small, whole inference engine for Llama-architecture models on one NVIDIA B200.

    from lmsf_b200 import LLM, SamplingParams
    outs = LLM(model_dir).generate(prompt_token_ids=[[1, 2, 3]], sampling_params=SamplingParams(temperature=0))
"""
from .config.engine_config import EngineArgs
from .sampling.params import SamplingParams


def __getattr__(name):   # the engine pulls in torch and CUDA; load it when asked for
    if name in ("LLM",):
        from .engine.llm import LLM
        return LLM
    if name in ("LLMEngine",):
        from .engine.llm_engine import LLMEngine
        return LLMEngine
    if name in ("RequestOutput", "CompletionOutput", "RequestMetrics"):
        from .engine import sequence
        return getattr(sequence, name)
    raise AttributeError(name)
