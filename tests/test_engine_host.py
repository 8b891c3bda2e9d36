"""The engine's host side without a GPU: scheduling, overlapped steps (a batch is launched before the one before it
is read), stop rules, aborts and preemptions, driven through `LLMEngine.from_parts` with a stand-in runner whose next
token is a hash of everything before it.  Whatever the scheduling does, a request must get exactly the sequence that
such a model produces, and every page must come back."""
import random

import pytest
import torch

from lmsf_b200.cache.manager import CacheManager, GroupSpec
from lmsf_b200.config.engine_config import SchedulerConfig
from lmsf_b200.engine import llm_engine as engine_module
from lmsf_b200.engine.llm_engine import LLMEngine
from lmsf_b200.sampling.params import SamplingParams

VOCAB = 97
EOS = 2


def next_token(history):
    h = len(history) * 1000003
    for i, t in enumerate(history):
        h = (h * 31 + (i + 1) * (t + 7)) % 2147483647
    return h % VOCAB


class StandInRunner:
    """Keeps each request's tokens by position, as the cache would, and answers with the hash of the history."""

    def __init__(self, max_model_len):
        self.hist, self.max_model_len = {}, max_model_len
        self.error_flag = torch.zeros(1, dtype=torch.int32)

    def check_device_errors(self):
        pass

    def step(self, entries, mgr, check=True, pending_tokens=None):
        rows = []
        for e in entries:
            toks = list(e.tokens)
            if e.last_from is not None:                  # the newest token is still "on the device"
                toks[-1] = int(pending_tokens[e.last_from])
            pos = mgr.num_tokens(e.request_id)
            assert pos + len(toks) <= self.max_model_len
            lack = pos + len(toks) - mgr.num_reserved(e.request_id)
            if lack > 0:
                mgr.reserve(e.request_id, lack)
            h = self.hist.setdefault(e.request_id, [])
            del h[pos:]                                  # a recomputation starts again at 0
            h.extend(toks)
            rows += [next_token(h[:pos + w + 1]) for w in e.want]
            mgr.commit(e.request_id, len(toks))
        return torch.tensor(rows, dtype=torch.int32).view(-1, 1)


class StandInSampler:
    def require_filters(self):
        pass

    def sample(self, logits, params, seeds, steps, seqs=None):
        return logits.view(-1).clone()


class NoEvent:
    def record(self):
        pass

    def synchronize(self):
        pass


def make_engine(pages, bs, budget, max_seqs, max_len, window, overlap):
    cache = CacheManager([GroupSpec(window)], [pages], bs, max_seqs)
    return LLMEngine.from_parts(StandInRunner(max_len), cache, SchedulerConfig.new(budget, max_seqs, max_len), StandInSampler(),
                                VOCAB, [EOS], max_len, async_scheduling=overlap)


def expected(prompt, sp, max_len):
    out = []
    while True:
        t = next_token(prompt + out)
        out.append(t)
        if t in sp.stop_token_ids:
            return out, "stop"
        if len(prompt) + len(out) >= max_len or len(out) >= sp.max_tokens:
            return out, "length"
        if not sp.ignore_eos and t == EOS:
            return out, "stop"


@pytest.fixture(autouse=True)
def no_cuda_events(monkeypatch):
    monkeypatch.setattr(engine_module.torch.cuda, "Event", NoEvent)


def run_workload(seed):
    rng = random.Random(seed)
    kw = dict(pages=rng.randint(3, 30), bs=rng.choice([1, 2, 4, 8, 16]), budget=rng.choice([1, 2, 8, 16, 48, 200]),
              max_seqs=rng.randint(1, 8), max_len=rng.choice([16, 48, 128]), window=rng.choice([None, None, None, 4, 12]),
              overlap=rng.random() < 0.7)
    eng = make_engine(**kw)
    reqs = []
    for _ in range(rng.randint(1, 14)):
        sp = SamplingParams(temperature=0.0, max_tokens=rng.randint(1, 25), ignore_eos=rng.random() < 0.5,
                            stop_token_ids=[rng.randrange(VOCAB) for _ in range(rng.choice([0, 0, 3, 10]))],
                            presence_penalty=0.3 if rng.random() < 0.3 else 0.0)
        reqs.append(([rng.randrange(VOCAB) for _ in range(rng.randint(1, 40))], sp))
    pending, results, aborted, steps = list(range(len(reqs))), {}, set(), 0
    while pending or eng.has_unfinished_requests():
        for _ in range(rng.randint(0, 3)):
            if pending:
                i = pending.pop(0)
                eng.add_request(i, None, reqs[i][1], prompt_token_ids=reqs[i][0])
        if rng.random() < 0.02 and eng.seqs:
            victim = rng.choice(list(eng.seqs))
            eng.abort_request(victim)
            aborted.add(victim)
        for o in eng.step():
            if o.finished:
                results[o.request_id] = (list(o.outputs[0].token_ids), o.outputs[0].finish_reason)
        eng.cache.check_invariants()
        steps += 1
        assert steps < 4000, f"seed {seed}: no end"
    assert eng.cache.num_free_pages() == kw["pages"], f"seed {seed}: pages lost"
    for i, (prompt, sp) in enumerate(reqs):
        if i in aborted:
            continue
        want, got = expected(prompt, sp, kw["max_len"]), results.get(i)
        if got == (want[0], want[1]):
            continue
        # a request that the cache cannot hold alone is ignored, or ends early with "length": a prefix of the sequence
        total = len(prompt) + len(want[0])
        need = total if kw["window"] is None else min(total, kw["window"] + 2 * kw["bs"])
        too_large = len(prompt) > kw["max_len"] or need > kw["pages"] * kw["bs"] - kw["bs"]
        assert too_large and got is not None and got[1] in ("length", "ignored") and got[0] == want[0][:len(got[0])], \
            f"seed {seed} {kw}: request {i} (prompt of {len(prompt)}) got {got}, the model gives {want}"


def test_random_workloads_get_the_models_sequence():
    for seed in range(600):
        run_workload(seed)


def test_a_request_that_ends_while_preempted_does_not_come_back():
    """Overlapped steps: a request is preempted while its newest token is still on its way from the device, and that
    token is a stop token.  It must end there (it used to stay in the waiting queue and generate on)."""
    # 9 pages of 8 tokens, three long prompts: the third is preempted right after its first token was sampled
    run_workload(337)
    run_workload(264)
    run_workload(391)


def test_several_cache_groups_with_and_without_windows():
    """Layers with different needs have page pools of their own: a request runs only when every group has its pages."""
    for seed in range(200):
        rng = random.Random(10_000 + seed)
        bs = rng.choice([1, 2, 4, 8, 16])
        windows = [rng.choice([None, 4, 12, 40]) for _ in range(rng.randint(2, 3))]
        pages = [rng.randint(3, 40) for _ in windows]
        max_len, max_seqs = rng.choice([16, 48, 128]), rng.randint(1, 8)
        cache = CacheManager([GroupSpec(w) for w in windows], pages, bs, max_seqs)
        eng = LLMEngine.from_parts(StandInRunner(max_len), cache, SchedulerConfig.new(rng.choice([1, 2, 8, 16, 48, 200]), max_seqs, max_len),
                                   StandInSampler(), VOCAB, [EOS], max_len, async_scheduling=rng.random() < 0.7)
        reqs = [([rng.randrange(VOCAB) for _ in range(rng.randint(1, 40))],
                 SamplingParams(temperature=0.0, max_tokens=rng.randint(1, 25), ignore_eos=rng.random() < 0.5,
                                stop_token_ids=[rng.randrange(VOCAB) for _ in range(rng.choice([0, 0, 3, 10]))]))
                for _ in range(rng.randint(1, 14))]
        pending, results, steps = list(range(len(reqs))), {}, 0
        while pending or eng.has_unfinished_requests():
            for _ in range(rng.randint(0, 3)):
                if pending:
                    i = pending.pop(0)
                    eng.add_request(i, None, reqs[i][1], prompt_token_ids=reqs[i][0])
            for o in eng.step():
                if o.finished:
                    assert o.request_id not in results
                    results[o.request_id] = (list(o.outputs[0].token_ids), o.outputs[0].finish_reason)
            cache.check_invariants()
            steps += 1
            assert steps < 6000, f"seed {seed}: no end"
        assert all(cache.num_free_pages(g) == pages[g] for g in range(len(pages))), f"seed {seed}: pages lost"
        for i, (prompt, sp) in enumerate(reqs):
            want, got = expected(prompt, sp, max_len), results.get(i)
            if got == (want[0], want[1]):
                continue
            total = len(prompt) + len(want[0])
            too_large = len(prompt) > max_len or any((total if w is None else min(total, w + 2 * bs)) > pages[g] * bs - bs
                                                     for g, w in enumerate(windows))
            assert too_large and got is not None and got[1] in ("length", "ignored") and got[0] == want[0][:len(got[0])], \
                f"seed {seed}: request {i} (prompt of {len(prompt)}) got {got}, the model gives {want}"
