"""Replay on the GPU against the plain implementation: the same requests whole, with the last 32 tokens
one by one, in portions of changing size, and mixed with other requests so that pages are used again; in
float32 and bfloat16, on tiny configurations that differ in every size."""
import numpy as np
import pytest

import plain_llama as P
import traces
import util

pytestmark = pytest.mark.gpu

# max |difference| allowed, as a fraction of the largest reference logit
REL = {"float32": 1e-5, "bfloat16": 5e-2}
LENGTHS = {"A": [5, 17, 33, 70], "B": [1, 9, 40, 64, 130], "W": [3, 50, 90, 41], "C": [2, 60, 140, 300]}


def requests_for(name, seed=0):
    cfg = util.CONFIGS[name]
    return {f"r{i}": util.random_ids(n, cfg["vocab_size"], seed * 100 + i) for i, n in enumerate(LENGTHS[name])}


_ref_cache = {}


def reference(name, dtype, std, reqs):
    key = (name, dtype, std, tuple(sorted((k, tuple(v)) for k, v in reqs.items())))
    if key not in _ref_cache:
        cfg, w = P.load_model(util.model_folder(name, dtype, std))
        _ref_cache[key] = {rid: P.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    return _ref_cache[key]


def check(rows, ref, dtype, reqs):
    assert len(rows) == sum(len(t) for t in reqs.values())
    scale = max(1.0, max(float(np.abs(r).max()) for r in ref.values()))
    worst = max(float(np.abs(row - ref[rid][pos]).max()) for (rid, pos), row in rows.items())
    assert worst <= REL[dtype] * scale, f"max |diff| {worst:.3e} at logit scale {scale:.3f}"
    return worst


@pytest.mark.parametrize("std", [0.02, 0.15])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "W", "C"])
def test_every_way_of_cutting_agrees_with_the_plain_implementation(name, dtype, std):
    reqs = requests_for(name)
    ref = reference(name, dtype, std, reqs)
    folder = util.model_folder(name, dtype, std)
    bs = util.BLOCK_SIZE[name]
    results = {}
    plans = {"whole": traces.whole(reqs), "tail32": traces.whole(reqs, tail=32),
             "portions": traces.portions(reqs, [7, 2, 13, 2, 31, 3]), "mixed": traces.mixed(reqs, seed=1)}
    for mode, steps in plans.items():
        need = traces.max_live_tokens(steps, round_to=bs)      # as few pages as the trace can run with
        out = traces.run_inprocess(folder, dtype, steps, bs, need)
        results[mode] = traces.collect(steps, out)
        check(results[mode], ref, dtype, reqs)
    if dtype == "float32":
        # the float32 kernels fix the order of every sum: the cut must not change a single bit
        for mode in ("tail32", "portions", "mixed"):
            for key, row in results["whole"].items():
                assert np.array_equal(row, results[mode][key]), (mode, key)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_program_itself(dtype):
    """bin/trace_run as a process: protocol, files, pages used again (five requests through room for three)."""
    name = "B"
    reqs = requests_for(name, seed=3)
    steps = traces.mixed(reqs, seed=5, max_live=3)
    folder = util.model_folder(name, dtype, 0.15)
    out = traces.run_program(folder, dtype, steps, traces.max_live_tokens(steps))
    check(traces.collect(steps, out), reference(name, dtype, 0.15, reqs), dtype, reqs)


def test_steps_without_wanted_logits_and_requests_that_sit_out():
    name, dtype = "A", "float32"
    cfg = util.CONFIGS[name]
    a, b = util.random_ids(40, cfg["vocab_size"], 7), util.random_ids(23, cfg["vocab_size"], 8)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:20], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": b[:21], "want": [20]}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[21:23], "want": [0, 1]}, {"id": "a", "tokens": a[20:38], "want": [17]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": a[38:], "want": [1, 0]}], "end": ["a"]},
    ]
    folder = util.model_folder(name, dtype, 0.15)
    out = traces.run_inprocess(folder, dtype, steps, util.BLOCK_SIZE[name], traces.max_live_tokens(steps, 8))
    assert 0 not in out and out[2].shape[0] == 3
    c, w = P.load_model(folder)
    ra, rb = P.forward(c, w, a).numpy(), P.forward(c, w, b).numpy()
    tol = 1e-5 * max(1.0, np.abs(ra).max())
    assert np.abs(out[1][0] - rb[20]).max() < tol
    assert np.abs(out[2] - np.stack([rb[21], rb[22], ra[37]])).max() < tol
    assert np.abs(out[3] - np.stack([ra[39], ra[38]])).max() < tol          # the order of `want` is kept
