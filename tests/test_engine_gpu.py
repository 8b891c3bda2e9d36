"""The engine end to end on the GPU: generation through the Python entry point against the plain
implementation, sampling, preemption, long decoding."""
import pytest
import torch

import plain_llama as P
import util

pytestmark = pytest.mark.gpu


def _llm(name, dtype, std=0.15, **kw):
    from lmsf_b200 import LLM
    return LLM(util.model_folder(name, dtype, std), dtype=dtype, block_size=util.BLOCK_SIZE[name], **kw)


@pytest.mark.parametrize("name,lengths,steps", [("A", [5, 17, 33], 8), ("B", [1, 9, 40, 64, 130], 12)])
def test_greedy_generation_matches_the_plain_implementation(name, lengths, steps):
    from lmsf_b200 import SamplingParams
    cfg, w = P.load_model(util.model_folder(name, "float32", 0.15))
    prompts = [util.random_ids(n, cfg["vocab_size"], i) for i, n in enumerate(lengths)]
    llm = _llm(name, "float32", num_gpu_blocks=64, max_num_batched_tokens=48, max_num_seqs=4)
    outs = llm.generate(prompt_token_ids=prompts,
                        sampling_params=SamplingParams(temperature=0.0, max_tokens=steps, ignore_eos=True))
    for p, o in zip(prompts, outs):
        ref, _ = P.generate(cfg, w, p, steps)
        assert o.outputs[0].token_ids == ref and o.outputs[0].finish_reason == "length" and o.finished
        assert o.prompt_token_ids == p


def test_step_logits_through_the_entry_point():
    """`LLM.step_logits`: the step function behind the public class, two requests in portions and single tokens,
    against the plain implementation; the pages it held are free again when its requests are ended, and
    generation goes on as before."""
    from lmsf_b200 import SamplingParams
    name = "A"
    cfg, w = P.load_model(util.model_folder(name, "float32", 0.15))
    a, b = util.random_ids(23, cfg["vocab_size"], 41), util.random_ids(9, cfg["vocab_size"], 42)
    ref_a = P.forward(cfg, w, torch.tensor(a), torch.float32)
    ref_b = P.forward(cfg, w, torch.tensor(b), torch.float32)
    llm = _llm(name, "float32", num_gpu_blocks=32, max_num_seqs=4)
    free0 = llm.engine.cache.num_free_pages(0)
    got = llm.step_logits([("a", a[:15], [0, 14]), ("b", b[:7], [6])])
    assert got.shape == (3, cfg["vocab_size"]) and got.dtype == torch.float32 and not got.is_cuda
    want = torch.stack([ref_a[0], ref_a[14], ref_b[6]])
    scale = want.abs().max().item()
    assert (got - want).abs().max().item() <= util.F32_REL * scale
    got = llm.step_logits([("a", a[15:22], []), ("b", b[7:8], [0])])
    assert (got - ref_b[7:8]).abs().max().item() <= util.F32_REL * scale
    got = llm.step_logits([("a", a[22:], [0]), ("b", b[8:], [0])], end=["a", "b"])
    assert (got - torch.stack([ref_a[22], ref_b[8]])).abs().max().item() <= util.F32_REL * scale
    assert llm.engine.cache.num_free_pages(0) == free0
    out = llm.generate(prompt_token_ids=[a], sampling_params=SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    assert out[0].outputs[0].token_ids == P.generate(cfg, w, a, 4)[0]


def test_temperature_sampling_is_reproducible_and_independent_of_the_batch():
    from lmsf_b200 import SamplingParams
    name = "B"
    cfg, w = P.load_model(util.model_folder(name, "float32", 0.15))
    prompts = [util.random_ids(n, cfg["vocab_size"], 10 + i) for i, n in enumerate([1, 9, 40, 64, 130])]
    sp = [SamplingParams(temperature=0.8, seed=1 + i, max_tokens=12, ignore_eos=True) for i in range(5)]
    llm = _llm(name, "float32", num_gpu_blocks=64, max_num_batched_tokens=48, max_num_seqs=4)
    together = [o.outputs[0].token_ids for o in llm.generate(prompt_token_ids=prompts, sampling_params=sp)]
    alone = [llm.generate(prompt_token_ids=[p], sampling_params=s)[0].outputs[0].token_ids for p, s in zip(prompts, sp)]
    assert together == alone
    for p, s, got in zip(prompts, sp, together):
        ref, _ = P.generate(cfg, w, p, 12, temperature=0.8, seed=s.seed)
        assert got == ref


def test_preemption_by_recompute_gives_the_same_tokens():
    from lmsf_b200 import SamplingParams
    name = "A"
    cfg = util.CONFIGS[name]
    prompts = [util.random_ids(n, cfg["vocab_size"], 20 + i) for i, n in enumerate([30, 25, 28, 20])]
    sp = [SamplingParams(temperature=0.7 if i % 2 else 0.0, seed=5 + i, max_tokens=40, ignore_eos=True) for i in range(4)]
    roomy = _llm(name, "float32", num_gpu_blocks=128, max_num_seqs=4)
    want = [o.outputs[0].token_ids for o in roomy.generate(prompt_token_ids=prompts, sampling_params=sp)]
    assert roomy.engine.scheduler.num_preemptions == 0
    tight = _llm(name, "float32", num_gpu_blocks=22, max_num_seqs=4)       # 176 slots for up to 4 * 70 tokens
    got = [o.outputs[0].token_ids for o in tight.generate(prompt_token_ids=prompts, sampling_params=sp)]
    assert tight.engine.scheduler.num_preemptions > 0
    assert got == want
    tight.engine.cache.check_invariants()
    assert tight.engine.cache.num_free_pages() == 22


def test_stop_conditions_and_rejection():
    from lmsf_b200 import SamplingParams
    name = "A"
    cfg, w = P.load_model(util.model_folder(name, "float32", 0.15))
    p = util.random_ids(12, cfg["vocab_size"], 31)
    ref, _ = P.generate(cfg, w, p, 10)
    llm = _llm(name, "float32", num_gpu_blocks=32, max_model_len=64)
    o = llm.generate(prompt_token_ids=[p], sampling_params=SamplingParams(temperature=0, max_tokens=10,
                                                                           stop_token_ids=[ref[4]]))[0]
    k = ref.index(ref[4])
    assert o.outputs[0].token_ids == ref[:k + 1] and o.outputs[0].finish_reason == "stop"
    # a prompt beyond max_model_len never runs; one that reaches it stops with "length"
    outs = llm.generate(prompt_token_ids=[list(range(1, 70)), util.random_ids(60, 256, 1)],
                        sampling_params=SamplingParams(temperature=0, max_tokens=50, ignore_eos=True))
    assert outs[0].outputs[0].finish_reason == "ignored" and outs[0].outputs[0].token_ids == []
    assert outs[1].outputs[0].finish_reason == "length" and len(outs[1].outputs[0].token_ids) == 4
    with pytest.raises(ValueError):
        llm.generate(prompt_token_ids=[[999]])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_stays_on_the_reference(dtype):
    """300 decoded tokens fed back one by one (teacher-forced with the plain implementation's tokens)."""
    import traces
    name = "B"
    cfg, w = P.load_model(util.model_folder(name, dtype, 0.15))
    ids = util.random_ids(250, cfg["vocab_size"], 77)
    ref = util.oracle_logits(cfg, w, {"x": ids}, dtype)
    steps = traces.whole({"x": ids}, tail=240)
    out = traces.collect(steps, traces.run_inprocess(util.model_folder(name, dtype, 0.15), dtype, steps, 16, 256))
    bound, _ = util.logits_bound(dtype, 0.15, ref)
    worst = util.worst_difference(out, ref)
    util.note_worst(f"long decoding {dtype}", worst, bound)
    assert len(out) == 250 and worst <= bound, (worst, bound)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_across_a_bucket_of_context_lengths(dtype):
    """Decode steps are replayed from a graph per batch size and bucket of context lengths (1,024, 2,048, ...):
    a request that grows from 1,016 to 1,040 tokens runs eagerly, from the first bucket's graph, eagerly again and
    from the second bucket's graph, and stays on the plain implementation throughout."""
    import tempfile
    import traces
    from lmsf_b200.weights import write_random_model
    cfg_d = dict(util.TINY_C, max_position_embeddings=4096)
    with tempfile.TemporaryDirectory(prefix="lmsf_bucket_") as folder:
        write_random_model(folder, cfg_d, seed=5, dtype=dtype, std=0.05)
        cfg, w = P.load_model(folder)
        ids = util.random_ids(1040, cfg["vocab_size"], 78)
        ref = util.oracle_logits(cfg, w, {"x": ids}, dtype)
        steps = traces.whole({"x": ids}, tail=24)
        out = traces.collect(steps, traces.run_inprocess(folder, dtype, steps, 16, 1040 + 16))
    bound, _ = util.logits_bound(dtype, 0.05, ref)
    worst = util.worst_difference(out, ref)
    util.note_worst(f"bucket of context lengths {dtype}", worst, bound)
    assert len(out) == 1040 and worst <= bound, (worst, bound)


def test_bfloat16_generation_through_the_entry_point():
    """Greedy and seeded generation in bfloat16: every token is the plain implementation's choice or within
    rounding of it, given the tokens before it (util.assert_tokens_within_rounding)."""
    from lmsf_b200 import SamplingParams
    for name, lengths in (("A", [5, 17, 33]), ("C", [2, 60, 140])):
        cfg, w = P.load_model(util.model_folder(name, "bfloat16", 0.15))
        prompts = [util.random_ids(n, cfg["vocab_size"], 41 + i) for i, n in enumerate(lengths)]
        sps = [SamplingParams(temperature=0.0 if i != 1 else 0.8, seed=7, max_tokens=12, ignore_eos=True) for i in range(3)]
        llm = _llm(name, "bfloat16", num_gpu_blocks=64, max_num_batched_tokens=48, max_num_seqs=4)
        outs = llm.generate(prompt_token_ids=prompts, sampling_params=sps)
        for p, sp, o in zip(prompts, sps, outs):
            assert len(o.outputs[0].token_ids) == 12
            util.assert_tokens_within_rounding(cfg, w, p, o.outputs[0].token_ids, "bfloat16", 0.15, sp.temperature, 7)


def test_preemption_by_recompute_in_bfloat16():
    """With few pages the youngest request is dropped and recomputed from its prompt and its tokens so far.  The
    recomputation runs those tokens as a prompt portion, not one by one, so in bfloat16 it may round differently;
    every token must still be within rounding of the best, and every page must come back."""
    from lmsf_b200 import SamplingParams
    name = "A"
    cfg, w = P.load_model(util.model_folder(name, "bfloat16", 0.15))
    prompts = [util.random_ids(n, cfg["vocab_size"], 20 + i) for i, n in enumerate([30, 25, 28, 20])]
    sp = [SamplingParams(temperature=0.7 if i % 2 else 0.0, seed=5 + i, max_tokens=40, ignore_eos=True) for i in range(4)]
    tight = _llm(name, "bfloat16", num_gpu_blocks=22, max_num_seqs=4)
    outs = tight.generate(prompt_token_ids=prompts, sampling_params=sp)
    assert tight.engine.scheduler.num_preemptions > 0
    for p, s, o in zip(prompts, sp, outs):
        assert len(o.outputs[0].token_ids) == 40
        util.assert_tokens_within_rounding(cfg, w, p, o.outputs[0].token_ids, "bfloat16", 0.15, s.temperature, s.seed)
    tight.engine.cache.check_invariants()
    assert tight.engine.cache.num_free_pages() == 22


def test_async_scheduling_in_bfloat16():
    from lmsf_b200 import SamplingParams
    name = "C"
    cfg, w = P.load_model(util.model_folder(name, "bfloat16", 0.15))
    prompts = [util.random_ids(n, cfg["vocab_size"], 60 + i) for i, n in enumerate([9, 30, 4, 150])]
    sps = [SamplingParams(temperature=0, max_tokens=14, ignore_eos=True), SamplingParams(temperature=0, max_tokens=3, ignore_eos=True),
           SamplingParams(temperature=0.9, seed=3, max_tokens=9, ignore_eos=True), SamplingParams(temperature=0, max_tokens=20, ignore_eos=True)]
    for mode in (True, False):
        llm = _llm(name, "bfloat16", num_gpu_blocks=40, max_num_batched_tokens=64, max_num_seqs=4, async_scheduling=mode)
        outs = llm.generate(prompt_token_ids=prompts, sampling_params=sps)
        for p, s, o in zip(prompts, sps, outs):
            assert len(o.outputs[0].token_ids) == s.max_tokens and o.outputs[0].finish_reason == "length"
            util.assert_tokens_within_rounding(cfg, w, p, o.outputs[0].token_ids, "bfloat16", 0.15, s.temperature, s.seed or 0)
        llm.engine.cache.check_invariants()
        assert llm.engine.cache.num_free_pages() == 40 and not llm.engine.has_unfinished_requests()


def test_the_example_program_from_a_model_folder_to_tokens():
    """bin/llm_engine_example as a process, with the reference's flag names: a model folder and prompts in,
    one JSON line per request out; the tokens are the plain implementation's."""
    import json
    import os
    import subprocess
    import sys
    name = "B"
    folder = util.model_folder(name, "float32", 0.15)
    cfg, w = P.load_model(folder)
    prompts = [util.random_ids(n, cfg["vocab_size"], 90 + i) for i, n in enumerate([7, 33])]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, os.path.join(root, "bin", "llm_engine_example"), "--model", folder, "--dtype", "float32",
           "--block-size", "16", "--num-gpu-blocks", "32", "--max-num-seqs", "4", "--max-num-batched-tokens", "24",
           "--temperature", "0", "--max-tokens", "8", "--ignore-eos"]
    for p in prompts:
        cmd += ["--prompt-ids", ",".join(str(t) for t in p)]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [json.loads(ln) for ln in proc.stdout.splitlines() if ln.startswith("{")]
    by_id = {d["request_id"]: d for d in lines}
    assert sorted(by_id) == [0, 1]
    for i, p in enumerate(prompts):
        assert by_id[i]["token_ids"] == P.generate(cfg, w, p, 8)[0] and by_id[i]["finish_reason"] == "length"
        m = by_id[i]["metrics"]                     # time to the first token and per later token, in seconds
        assert m["ttft_s"] > 0 and m["tpot_s"] > 0 and m["finished_s"] >= m["ttft_s"]
    assert "End cost" in proc.stderr


def test_top_k_top_p_and_penalties_through_the_entry_point():
    """The reference example's own options (temperature 0.8, top-k 5, presence penalty 0.2) and the others."""
    from lmsf_b200 import SamplingParams
    name = "A"
    cfg, w = P.load_model(util.model_folder(name, "float32", 0.15))
    prompt = util.random_ids(14, cfg["vocab_size"], 51)
    sp = SamplingParams(temperature=0.8, top_k=5, top_p=0.9, min_p=0.02, presence_penalty=0.2, frequency_penalty=0.1,
                        repetition_penalty=1.3, seed=9, max_tokens=10, ignore_eos=True)
    llm = _llm(name, "float32", num_gpu_blocks=32)
    got = llm.generate(prompt_token_ids=[prompt], sampling_params=sp)[0].outputs[0].token_ids
    ids, out = list(prompt), []
    for step in range(10):
        row = P.forward(cfg, w, ids)[-1]
        row = P.apply_penalties(row, prompt, out, 0.2, 0.1, 1.3)
        tok = P.sample_filtered(row, 0.8, 9, step, 5, 0.9, 0.02)
        out.append(tok)
        ids.append(tok)
    assert got == out
    # a greedy request beside it is not disturbed
    both = llm.generate(prompt_token_ids=[prompt, prompt],
                        sampling_params=[sp, SamplingParams(temperature=0, max_tokens=5, ignore_eos=True)])
    assert both[0].outputs[0].token_ids == out and both[1].outputs[0].token_ids == P.generate(cfg, w, prompt, 5)[0]


def test_async_scheduling_gives_the_same_tokens_and_drops_what_ran_past_a_stop():
    """With async scheduling the next batch is launched before the last one's tokens are read; a request that
    stopped has then been run once more and that result must vanish."""
    from lmsf_b200 import SamplingParams
    name = "A"
    cfg, w = P.load_model(util.model_folder(name, "float32", 0.15))
    prompts = [util.random_ids(n, cfg["vocab_size"], 60 + i) for i, n in enumerate([9, 30, 4, 21])]
    refs = [P.generate(cfg, w, p, 14)[0] for p in prompts]
    # request 0 stops on its 5th token, request 2 on its 1st; the others run to max_tokens
    sps = [SamplingParams(temperature=0, max_tokens=14, stop_token_ids=[refs[0][4]]),
           SamplingParams(temperature=0, max_tokens=14, ignore_eos=True),
           SamplingParams(temperature=0, max_tokens=14, stop_token_ids=[refs[2][0]]),
           SamplingParams(temperature=0.9, seed=3, max_tokens=9, ignore_eos=True)]
    results = {}
    for mode in (True, False):
        llm = _llm(name, "float32", num_gpu_blocks=40, max_num_batched_tokens=16, max_num_seqs=4, async_scheduling=mode)
        outs = llm.generate(prompt_token_ids=prompts, sampling_params=sps)
        results[mode] = [(o.outputs[0].token_ids, o.outputs[0].finish_reason) for o in outs]
        llm.engine.cache.check_invariants()
        assert llm.engine.cache.num_free_pages() == 40 and not llm.engine.has_unfinished_requests()
    assert results[True] == results[False]
    got = results[True]
    assert got[0] == (refs[0][:refs[0].index(refs[0][4]) + 1], "stop")
    assert got[1] == (refs[1], "length")
    assert got[2] == (refs[2][:1], "stop")
    assert got[3][0] == P.generate(cfg, w, prompts[3], 9, temperature=0.9, seed=3)[0]


def test_engine_step_api_and_abort():
    from lmsf_b200 import EngineArgs, LLMEngine, SamplingParams
    name = "A"
    engine = LLMEngine(EngineArgs(model=util.model_folder(name, "float32", 0.15), dtype="float32", block_size=8,
                                  num_gpu_blocks=32, max_num_seqs=4))
    sp = SamplingParams(temperature=0, max_tokens=30, ignore_eos=True)
    engine.add_request("a", None, sp, prompt_token_ids=[5, 6, 7])
    engine.add_request("b", None, sp, prompt_token_ids=[8, 9])
    with pytest.raises(KeyError):
        engine.add_request("a", None, sp, prompt_token_ids=[1])
    assert engine.get_num_unfinished_requests() == 2
    seen = {"a": 0, "b": 0}
    for _ in range(6):
        for out in engine.step():
            seen[out.request_id] = len(out.outputs[0].token_ids)
    assert seen["a"] >= 4 and seen["b"] >= 4
    engine.abort_request("a")
    while engine.has_unfinished_requests():
        for out in engine.step():
            assert out.request_id == "b"
            seen["b"] = len(out.outputs[0].token_ids)
    assert seen["b"] == 30
    engine.cache.check_invariants()
    assert engine.cache.num_free_pages() == 32


@pytest.mark.parametrize("seed,dtype", [(3, "float32"), (5, "float32"), (6, "float32"), (9, "float32"), (10, "float32"),
                                        (11, "float32"), (6, "bfloat16"), (10, "bfloat16")])
def test_random_workloads_through_the_engine(seed, dtype):
    """Requests that arrive over time, random prompt and output lengths, greedy or seeded sampling, a random token
    budget, few pages (seeds 6, 9, 10 and 11 preempt) and synchronous or asynchronous scheduling: every request
    gets the plain implementation's tokens (in bfloat16: tokens within rounding of the best) and every page comes
    back."""
    import random
    from lmsf_b200 import EngineArgs, LLMEngine, SamplingParams
    rng = random.Random(seed)
    name = rng.choice(["A", "B", "W", "C"])
    cfgd, bs = util.CONFIGS[name], util.BLOCK_SIZE[name]
    folder = util.model_folder(name, dtype, 0.15)
    cfg, w = P.load_model(folder)
    n_req = rng.randint(3, 9)
    max_len = min(cfgd["max_position_embeddings"], 120)
    prompts = [util.random_ids(rng.randint(1, 60), cfgd["vocab_size"], seed * 50 + i) for i in range(n_req)]
    gens = [rng.randint(1, 30) for _ in range(n_req)]
    pages = max(-(-max(len(p) + g for p, g in zip(prompts, gens)) // bs) + 2, rng.randint(6, 40))
    budget, max_seqs, async_s = rng.choice([8, 16, 33, 64, 256]), rng.choice([2, 3, 4, 8]), rng.random() < 0.5
    eng = LLMEngine(EngineArgs(model=folder, dtype=dtype, block_size=bs, num_gpu_blocks=pages,
                               max_num_batched_tokens=budget, max_num_seqs=max_seqs, max_model_len=max_len,
                               no_async_scheduling=not async_s))
    sps = [SamplingParams(temperature=0.0 if rng.random() < 0.6 else 0.8, seed=seed * 7 + i, max_tokens=g, ignore_eos=True)
           for i, g in enumerate(gens)]
    arrivals = sorted((rng.randint(0, 12), i) for i in range(n_req))
    results, step, ai = {}, 0, 0
    while ai < len(arrivals) or eng.has_unfinished_requests():
        while ai < len(arrivals) and arrivals[ai][0] <= step:
            i = arrivals[ai][1]
            eng.add_request(i, None, sps[i], prompt_token_ids=prompts[i])
            ai += 1
        for o in eng.step():
            if o.finished:
                results[o.request_id] = o.outputs[0].token_ids
        step += 1
        assert step < 5000
    if seed in (6, 9, 10, 11):
        assert eng.scheduler.num_preemptions > 0
    for i in range(n_req):
        if dtype == "float32":
            ref, _ = P.generate(cfg, w, prompts[i], gens[i], temperature=sps[i].temperature, seed=sps[i].seed)
            assert results[i] == ref, (i, len(prompts[i]), gens[i], sps[i].temperature)
        else:
            assert len(results[i]) == gens[i]
            util.assert_tokens_within_rounding(cfg, w, prompts[i], results[i], dtype, 0.15, sps[i].temperature, sps[i].seed)
    eng.cache.check_invariants()
    assert eng.cache.num_free_pages() == pages


def test_penalties_give_the_same_tokens_with_and_without_overlap():
    """A batch with penalties retires the batch before it between its model step and its sampling; the tokens must be
    those of steps that run strictly in order, also when requests stop early, arrive late and pages are scarce."""
    from lmsf_b200 import EngineArgs, LLMEngine, SamplingParams
    name = "A"
    cfgd, bs = util.CONFIGS[name], util.BLOCK_SIZE[name]
    folder = util.model_folder(name, "float32", 0.15)
    prompts = [util.random_ids(n, cfgd["vocab_size"], 300 + i) for i, n in enumerate([12, 40, 7, 33, 21, 5])]
    sps = [SamplingParams(temperature=0.9 if i % 3 else 0.0, seed=40 + i, max_tokens=10 + 4 * i, top_k=20 if i % 2 else -1,
                          presence_penalty=0.3 if i != 2 else 0.0, frequency_penalty=0.2, repetition_penalty=1.2,
                          stop_token_ids=[3, 17, 41, 77, 100, 150]) for i in range(len(prompts))]
    got = {}
    for no_async in (True, False):
        eng = LLMEngine(EngineArgs(model=folder, dtype="float32", block_size=bs, num_gpu_blocks=14, max_num_batched_tokens=32,
                                   max_num_seqs=4, max_model_len=120, no_async_scheduling=no_async))
        res, step, nxt = {}, 0, 0
        while nxt < len(prompts) or eng.has_unfinished_requests():
            if nxt < len(prompts) and step % 3 == 0:
                eng.add_request(nxt, None, sps[nxt], prompt_token_ids=prompts[nxt])
                nxt += 1
            for o in eng.step():
                if o.finished:
                    res[o.request_id] = (o.outputs[0].token_ids, o.outputs[0].finish_reason)
            step += 1
            assert step < 2000
        eng.cache.check_invariants()
        assert eng.cache.num_free_pages() == 14
        got[no_async] = res
    assert got[True] == got[False]


def test_a_windowed_prompt_longer_than_the_cache_runs_in_portions():
    """Sliding window of 24 keys, 4 pages of 16 tokens: a 90-token prompt cannot hold its pages all at once, so the
    scheduler cuts it to what the pages hold and the window gives pages back between the portions."""
    from lmsf_b200 import SamplingParams
    name = "W"
    cfg, w = P.load_model(util.model_folder(name, "float32", 0.15))
    prompts = [util.random_ids(90, cfg["vocab_size"], 61), util.random_ids(50, cfg["vocab_size"], 62)]
    llm = _llm(name, "float32", num_gpu_blocks=4, max_num_batched_tokens=256, max_num_seqs=2, max_model_len=120)
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    for p, o in zip(prompts, outs):
        ref, _ = P.generate(cfg, w, p, 8)
        assert o.outputs[0].token_ids == ref
    llm.engine.cache.check_invariants()
    assert llm.engine.cache.num_free_pages() == 4
