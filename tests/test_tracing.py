"""The tracing switch: off by default and free of any CUDA call; on, it opens and closes ranges."""
import importlib


def test_span_is_a_no_op_unless_switched_on(monkeypatch):
    from lmsf_b200.utils import tracing
    monkeypatch.delenv("LMSF_NVTX", raising=False)
    importlib.reload(tracing)
    assert tracing.ENABLED is False
    with tracing.span("x"):
        pass                                   # touches neither torch nor CUDA
    tracing.profiler_start()
    tracing.profiler_stop()
    monkeypatch.setenv("LMSF_NVTX", "1")
    importlib.reload(tracing)
    assert tracing.ENABLED is True
    monkeypatch.delenv("LMSF_NVTX")
    importlib.reload(tracing)
