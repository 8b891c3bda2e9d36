"""Replay on the GPU against the plain implementation: the same requests whole, with the last 32 tokens
one by one, in portions of changing size, and mixed with other requests so that pages are used again; in
float32 and bfloat16, on tiny configurations that differ in every size."""
import numpy as np
import pytest

import plain_llama as P
import traces
import util

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 17, 33, 70], "B": [1, 9, 40, 64, 130], "W": [3, 50, 90, 41], "C": [2, 60, 140, 300]}


def requests_for(name, seed=0):
    cfg = util.CONFIGS[name]
    return {f"r{i}": util.random_ids(n, cfg["vocab_size"], seed * 100 + i) for i, n in enumerate(LENGTHS[name])}


_ref_cache = {}


def reference(name, dtype, std, reqs):
    key = (name, dtype, std, tuple(sorted((k, tuple(v)) for k, v in reqs.items())))
    if key not in _ref_cache:
        cfg, w = P.load_model(util.model_folder(name, dtype, std))
        _ref_cache[key] = util.oracle_logits(cfg, w, reqs, dtype)
    return _ref_cache[key]


def check(rows, ref, dtype, reqs, std, what=""):
    assert len(rows) == sum(len(t) for t in reqs.values())
    bound, scale = util.logits_bound(dtype, std, ref)
    worst = util.worst_difference(rows, ref)
    util.note_worst(f"replay {what} {dtype} std {std}", worst, bound)
    assert worst <= bound, f"{what}: max |diff| {worst:.3e} against a bound of {bound:.3e} at logit scale {scale:.3f}"
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
        check(results[mode], ref, dtype, reqs, std, f"{name} {mode}")
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
    check(traces.collect(steps, out), reference(name, dtype, 0.15, reqs), dtype, reqs, 0.15, "program")


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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_live", [21, 40])
def test_many_live_requests_decoding_together(n_live, dtype):
    """21 and 40 requests decode at once (decode batches above 16 rows: the graph sizes 24 and 40, one padded with
    stand-in requests, the products of more than 16 rows with the rotation and the cache write as kernels of
    their own, one key split per request), each compared with the plain implementation."""
    name, std = "C", 0.15
    cfg = util.CONFIGS[name]
    rng_lengths = [12 + (37 * i) % 90 for i in range(n_live)]
    reqs = {f"m{i}": util.random_ids(n, cfg["vocab_size"], 500 + i) for i, n in enumerate(rng_lengths)}
    ref = reference(name, dtype, std, reqs)
    steps = traces.many_live(reqs, tail=10, per_step=8)
    bs = util.BLOCK_SIZE[name]
    out = traces.run_inprocess(util.model_folder(name, dtype, std), dtype, steps, bs,
                               traces.max_live_tokens(steps, round_to=bs), max_live=n_live)
    rows = traces.collect(steps, out)
    full = [s for s in steps if len(s["entries"]) == n_live and all(len(e["tokens"]) == 1 for e in s["entries"])]
    assert len(full) >= 4                          # steps in which every request brings one token
    bound, scale = util.logits_bound(dtype, std, ref)
    worst = util.worst_difference(rows, ref)
    util.note_worst(f"many live {n_live} {dtype}", worst, bound)
    assert worst <= bound, (worst, bound, scale)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_long_request_decoding_among_short_ones(dtype):
    """A request of 480 tokens decodes beside eleven of 12 to 30: the decode graph of such a batch splits every
    request's keys as the long one needs it, so most blocks of the short ones find no keys."""
    name, std = "C", 0.15
    cfg = util.CONFIGS[name]
    lengths = [480] + [12 + (7 * i) % 19 for i in range(11)]
    reqs = {f"k{i}": util.random_ids(n, cfg["vocab_size"], 700 + i) for i, n in enumerate(lengths)}
    ref = reference(name, dtype, std, reqs)
    steps = traces.many_live(reqs, tail=10, per_step=12)
    bs = util.BLOCK_SIZE[name]
    out = traces.run_inprocess(util.model_folder(name, dtype, std), dtype, steps, bs,
                               traces.max_live_tokens(steps, round_to=bs), max_live=len(lengths))
    rows = traces.collect(steps, out)
    bound, scale = util.logits_bound(dtype, std, ref)
    worst = util.worst_difference(rows, ref)
    util.note_worst(f"one long among short {dtype}", worst, bound)
    assert worst <= bound, (worst, bound, scale)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_request_dropped_in_the_middle_of_its_prompt_and_replayed(dtype):
    """What preemption by recompute does, at the level of the step function: a live request gives back what it
    holds after 45 of its 130 tokens, its pages go to the others, and it runs again from its first token."""
    name, std = "B", 0.15
    reqs = requests_for(name, seed=4)
    ref = reference(name, dtype, std, reqs)
    steps = traces.dropped_and_replayed(reqs, "r4", 45)
    assert sum(1 for s in steps if "r4" in s["end"]) == 2
    bs = util.BLOCK_SIZE[name]
    out = traces.run_inprocess(util.model_folder(name, dtype, std), dtype, steps, bs, traces.max_live_tokens(steps, round_to=bs))
    check(traces.collect(steps, out), ref, dtype, reqs, std, "dropped and replayed")
