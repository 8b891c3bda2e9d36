"""The scheduler's decisions, on a fake step (no GPU)."""
import random

from lmsf_b200.cache import CacheManager, GroupSpec
from lmsf_b200.config import SchedulerConfig
from lmsf_b200.engine.scheduler import Scheduler
from lmsf_b200.engine.sequence import Sequence, SequenceStatus
from lmsf_b200.sampling.params import SamplingParams


def make(pages=64, bs=4, budget=16, max_seqs=8, max_len=256, window=None):
    cache = CacheManager([GroupSpec(window)], [pages], bs, max_seqs)
    return Scheduler(SchedulerConfig.new(budget, max_seqs, max_len), cache), cache


def seq(rid, n_prompt, t=None, max_tokens=4):
    s = Sequence(rid, list(range(1, n_prompt + 1)), SamplingParams(temperature=0, max_tokens=max_tokens))
    if t is not None:
        s.arrival_time = t
    return s


def run_step(sched, cache, out, token=7):
    """What the engine does after a step: commit, count, append a token where logits were wanted."""
    finished = []
    for e in out.entries:
        cache.commit(e.seq.request_id, e.num_tokens)
        e.seq.num_computed += e.num_tokens
    for e in out.entries:
        if e.wants_logits:
            e.seq.output_token_ids.append(token)
            if len(e.seq.output_token_ids) >= e.seq.sampling_params.max_tokens:
                e.seq.status = SequenceStatus.FINISHED_LENGTH
                sched.free_seq(e.seq)
                finished.append(e.seq)
    cache.check_invariants()
    return finished


def test_prompt_is_cut_under_the_budget_and_only_its_end_wants_logits():
    sched, cache = make(budget=16)
    s = seq("a", 40, 0.0)
    sched.add_seq(s)
    seen = []
    for _ in range(3):
        out = sched.schedule()
        assert [e.seq.request_id for e in out.entries] == ["a"]
        seen.append((out.entries[0].start, out.entries[0].num_tokens, out.entries[0].wants_logits))
        run_step(sched, cache, out)
    assert seen == [(0, 16, False), (16, 16, False), (32, 8, True)]
    out = sched.schedule()
    assert (out.entries[0].start, out.entries[0].num_tokens, out.entries[0].wants_logits) == (40, 1, True)


def test_decodes_first_then_portions_then_admissions_fcfs():
    sched, cache = make(budget=16)
    a, b, c = seq("a", 3, 0.0, max_tokens=50), seq("b", 30, 1.0), seq("c", 5, 2.0)
    for s in (a, b, c):
        sched.add_seq(s)
    out = sched.schedule()
    assert [(e.seq.request_id, e.num_tokens, e.wants_logits) for e in out.entries] == [("a", 3, True), ("b", 13, False)]
    run_step(sched, cache, out)
    out = sched.schedule()          # a decodes (1), b goes on (15 left of budget), c waits: no budget left
    assert [(e.seq.request_id, e.start, e.num_tokens) for e in out.entries] == [("a", 3, 1), ("b", 13, 15)]
    run_step(sched, cache, out)
    out = sched.schedule()
    assert [(e.seq.request_id, e.num_tokens, e.wants_logits) for e in out.entries] == \
        [("a", 1, True), ("b", 2, True), ("c", 5, True)]
    assert out.num_batched_tokens == 8


def test_max_num_seqs_and_state_slots_bound_admission():
    sched, cache = make(max_seqs=2, budget=64)
    for i in range(4):
        sched.add_seq(seq(i, 4, float(i)))
    out = sched.schedule()
    assert [e.seq.request_id for e in out.entries] == [0, 1] and len(sched.waiting) == 2


def test_too_long_prompts_are_ignored_not_run():
    sched, cache = make(pages=4, bs=4, max_len=64, budget=64)
    sched.add_seq(seq("long", 65, 0.0))          # beyond max_model_len
    sched.add_seq(seq("fat", 20, 1.0))           # 5 pages needed, 4 exist
    sched.add_seq(seq("ok", 6, 2.0))
    out = sched.schedule()
    assert [s.request_id for s in out.ignored] == ["long", "fat"]
    assert all(s.status == SequenceStatus.FINISHED_IGNORED for s in out.ignored)
    assert [e.seq.request_id for e in out.entries] == ["ok"]


def test_out_of_pages_preempts_the_youngest_and_recomputes_it():
    sched, cache = make(pages=6, bs=4, budget=64)
    a, b = seq("a", 8, 0.0, max_tokens=20), seq("b", 8, 1.0, max_tokens=20)
    sched.add_seq(a)
    sched.add_seq(b)
    run_step(sched, cache, sched.schedule())       # both prompts: 2 + 2 pages, 2 free
    steps = 0
    while True:
        out = sched.schedule()
        if out.preempted:
            break
        run_step(sched, cache, out)
        steps += 1
        assert steps < 20
    # a (older) keeps running, b (youngest) went back to the FRONT of the waiting queue with its tokens
    assert [s.request_id for s in out.preempted] == ["b"] and sched.waiting[0] is b
    assert b.num_computed == 0 and len(b.output_token_ids) > 0 and b.num_preemptions == 1
    assert not cache.has("b") and [e.seq.request_id for e in out.entries] == ["a"]
    got_before = len(b.output_token_ids)
    run_step(sched, cache, out)
    # nothing is admitted in the step that preempted; later b returns as one portion of prompt + generated
    for _ in range(40):
        out = sched.schedule()
        eb = [e for e in out.entries if e.seq is b]
        if eb:
            assert eb[0].start == 0 and eb[0].num_tokens == 8 + got_before and eb[0].wants_logits
            break
        run_step(sched, cache, out)
    else:
        raise AssertionError("b never came back")


def test_request_that_outgrows_the_cache_alone_ends_with_length():
    sched, cache = make(pages=3, bs=4, budget=64, max_len=256)
    a = seq("a", 10, 0.0, max_tokens=100)
    sched.add_seq(a)
    for _ in range(10):
        out = sched.schedule()
        if out.ignored:
            break
        run_step(sched, cache, out)
    assert out.ignored == [a] and a.status == SequenceStatus.FINISHED_LENGTH
    # 12 positions fit; the 13th token was sampled but can never be cached
    assert len(a) == 13 and a.num_computed == 12 and not sched.has_unfinished_seqs() and cache.num_free_pages() == 3


def test_abort_frees_pages_from_either_queue():
    sched, cache = make(pages=8, bs=4, budget=8)
    a, b = seq("a", 6, 0.0), seq("b", 6, 1.0)
    sched.add_seq(a)
    sched.add_seq(b)
    run_step(sched, cache, sched.schedule())
    assert sched.abort_seq("a").status == SequenceStatus.FINISHED_ABORTED
    assert sched.abort_seq("b") is b and sched.abort_seq("zzz") is None
    assert cache.num_free_pages() == 8 and not sched.has_unfinished_seqs()


def test_random_workloads_finish_and_lose_no_page():
    for seed in range(6):
        rng = random.Random(seed)
        sched, cache = make(pages=rng.randint(8, 24), bs=4, budget=rng.choice([8, 16, 48]), max_seqs=4,
                            window=rng.choice([None, 12]))
        seqs = [seq(i, rng.randint(1, 30), float(i), max_tokens=rng.randint(1, 12)) for i in range(12)]
        for s in seqs:
            sched.add_seq(s)
        done, steps = [], 0
        while sched.has_unfinished_seqs():
            out = sched.schedule()
            assert out.num_batched_tokens <= sched.config.max_num_batched_tokens
            assert out.entries or out.ignored or out.preempted
            done += out.ignored + run_step(sched, cache, out)
            steps += 1
            assert steps < 2000
        assert len(done) == 12 and all(p.num_free == p.num_blocks for p in cache.pools)


def test_a_windowed_prompt_longer_than_the_cache_is_cut_to_what_the_pages_hold():
    """6 pages of 4 tokens and a window of 4: a 30-token prompt never holds more than a few pages once it runs, but a
    portion's pages are all held until its step is over.  The portion is cut to what fits (it used to wait for ever),
    and the rest follows as the window gives pages back."""
    sched, cache = make(pages=6, bs=4, budget=200, max_seqs=3, max_len=64, window=4)
    a = seq(0, 30, 0.0, max_tokens=5)
    sched.add_seq(a)
    done, steps, portions = [], 0, []
    while sched.has_unfinished_seqs():
        out = sched.schedule()
        assert out.entries, "the request must make progress in every step"
        portions.append(out.entries[0].num_tokens)
        done += run_step(sched, cache, out)
        cache.check_invariants()
        steps += 1
        assert steps < 100
    assert portions[0] < 30 and sum(portions[:portions.index(1)]) == 30     # the prompt in several portions, then single tokens
    assert done == [a] and len(a.output_token_ids) == 5
    assert all(p.num_free == p.num_blocks for p in cache.pools)


def test_many_random_workloads_with_windows_aborts_and_late_arrivals():
    for seed in range(300):
        rng = random.Random(seed)
        sched, cache = make(pages=rng.randint(4, 40), bs=rng.choice([1, 2, 4, 8, 16]), budget=rng.choice([1, 2, 8, 16, 48, 200]),
                            max_seqs=rng.randint(1, 9), max_len=rng.choice([16, 64, 256]), window=rng.choice([None, None, 4, 12, 40]))
        pending = [seq(i, rng.randint(1, 60), float(i), max_tokens=rng.randint(1, 30)) for i in range(rng.randint(1, 20))]
        steps = 0
        while pending or sched.has_unfinished_seqs():
            for _ in range(rng.randint(0, 3)):
                if pending:
                    sched.add_seq(pending.pop(0))
            if rng.random() < 0.03 and sched.running:
                sched.abort_seq(rng.choice(sched.running).request_id)
            if not sched.has_unfinished_seqs():
                continue
            out = sched.schedule()
            assert out.num_batched_tokens <= sched.config.max_num_batched_tokens
            assert out.entries or out.ignored or out.preempted, f"seed {seed}: a step in which nothing happens"
            run_step(sched, cache, out)
            cache.check_invariants()
            steps += 1
            assert steps < 5000, f"seed {seed}: no end"
        assert all(p.num_free == p.num_blocks for p in cache.pools), f"seed {seed}: pages lost"
