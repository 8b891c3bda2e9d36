"""Host-side rules that need no GPU: the choice of key splits for the decode attention, the buckets of context
lengths of the decode graphs, and the sampler's token histories."""
import random
from collections import Counter

import numpy as np

from lmsf_b200 import kernels
from lmsf_b200.sampling.sampler import _TokenHistory

# clusters of 1..8 decode blocks that a B200 holds at a time (head size 128: two blocks per SM, 148 SMs)
B200_CLUSTERS = (296, 148, 93, 71, 56, 45, 37, 33)


def test_key_splits_fill_one_wave_when_they_can():
    pick = lambda n, ctx: kernels.decode_num_splits(n, 8, 4, ctx, B200_CLUSTERS)
    assert pick(8, 2048) == 4                 # 64 clusters of 4: 71 fit
    assert pick(5, 2048) == 6                 # 40 clusters: 45 of 6 fit, only 37 of 7
    assert pick(12, 2048) == 2                # 96 clusters: 93 of 3 would need a second wave
    assert pick(32, 2048) == 1 and pick(64, 2048) == 1
    assert pick(1, 2048) == 8                 # the cluster's shared memory beats global memory for short contexts
    assert pick(1, 32768) > 8                 # a long context wants every slot busy
    for n in (1, 2, 3, 7, 8, 20, 64, 200):
        for ctx in (1, 64, 100, 128, 129, 500, 2048, 100000):
            s = pick(n, ctx)
            assert 1 <= s <= 64
            assert s == 1 or ctx / s >= 64    # a split keeps at least 128 keys (rounded to tiles of 64)


def test_split_choice_does_not_depend_on_what_it_should_not():
    # more query heads per kv head up to 16 share a block: same answer
    assert kernels.decode_num_splits(8, 8, 1, 2048, B200_CLUSTERS) == kernels.decode_num_splits(8, 8, 16, 2048, B200_CLUSTERS)
    # 17 to 32 heads per kv head need two blocks per kv head: as if there were twice the kv heads
    assert kernels.decode_num_splits(8, 8, 32, 2048, B200_CLUSTERS) == kernels.decode_num_splits(8, 16, 4, 2048, B200_CLUSTERS)


def test_buckets_of_context_lengths():
    from lmsf_b200.engine.model_runner import ModelRunner
    class R:                                  # the rule needs only max_model_len
        max_model_len = 10000
    b = lambda n: ModelRunner.graph_context_bucket(R, n)
    assert [b(n) for n in (1, 1024, 1025, 2048, 2049, 8192, 8193, 10000)] == [1024, 1024, 2048, 2048, 4096, 8192, 10000, 10000]
    R.max_model_len = 300
    assert b(1) == 300 and b(300) == 300


def test_token_history_counts_like_a_recount():
    rng = random.Random(0)
    for _ in range(20):
        prompt = [rng.randrange(50) for _ in range(rng.randint(0, 40))]
        h = _TokenHistory(prompt)
        out = []
        for _ in range(rng.randint(1, 120)):
            out.extend(rng.randrange(60) for _ in range(rng.randint(0, 3)))
            t, c = h.update(out)
            counts = Counter(out)
            want = {tok: counts.get(tok, 0) for tok in set(prompt) | set(out)}
            assert dict(zip(t.tolist(), c.tolist())) == want and len(t) == len(want)
        t, c = h.update(out[:3])              # the output was cut back (never happens in the engine): counted again
        assert dict(zip(t.tolist(), c.tolist())) == {tok: Counter(out[:3]).get(tok, 0) for tok in set(prompt) | set(out)}
        assert t.dtype == np.int32 and c.dtype == np.int32


def test_histories_go_with_their_requests():
    import gc
    import torch
    from lmsf_b200.engine.sequence import Sequence
    from lmsf_b200.sampling.params import SamplingParams
    from lmsf_b200.sampling.sampler import Sampler
    sampler = Sampler(torch.device("cpu"))
    a = Sequence("a", [3, 4, 4], SamplingParams(presence_penalty=0.5))
    b = Sequence("b", [9], SamplingParams(presence_penalty=0.5))
    ha = sampler._history(a)
    assert sampler._history(a) is ha and sampler._history(b) is not ha and len(sampler._histories) == 2
    del a, ha
    gc.collect()
    assert len(sampler._histories) == 1       # the entry went with the request object
    class Plain:                              # an object without weak references: served, but nothing is kept
        __slots__ = ("prompt_token_ids", "output_token_ids")
    p = Plain()
    p.prompt_token_ids, p.output_token_ids = [1, 2], [2]
    t, c = sampler._history(p).update(p.output_token_ids)
    assert dict(zip(t.tolist(), c.tolist())) == {1: 0, 2: 1} and len(sampler._histories) == 1
