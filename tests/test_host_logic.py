"""Host-side rules that need no GPU: the choice of key splits for the decode attention, the buckets of context
lengths of the decode graphs, and the sampler's token histories."""
import random
from collections import Counter

import numpy as np

from lmsf_b200 import kernels
from lmsf_b200.sampling.sampler import _TokenHistory

# The widths of a decode block on a B200 at head size 128 (148 SMs): wide blocks of four warps with 68 KB in flight,
# two per SM, and narrow ones of two warps with 34 KB, four per SM; for each the clusters of 1..8 blocks that fit.
B200_WIDE = (4, 2 * 2 * 64 * 272 / 65536.0, (296, 148, 93, 71, 56, 45, 37, 33))
B200_NARROW = (2, 2 * 2 * 32 * 272 / 65536.0, (592, 296, 187, 142, 112, 93, 78, 71))
B200_WIDTHS = (B200_WIDE, B200_NARROW)


def test_key_splits_fill_one_wave_when_they_can():
    pick = lambda n, ctx, kv=8, group=4: kernels.decode_plan(n, kv, group, ctx, 128, B200_WIDTHS)
    assert pick(8, 2048) == (4, 4)            # 64 clusters of 4: 71 fit
    assert pick(5, 2048) in ((5, 4), (6, 4))  # 40 clusters: 45 of 6 fit, only 37 of 7 (5 and 6 splits are a near tie)
    assert pick(12, 2048) == (2, 4)           # 96 clusters: 93 of 3 would need a second wave
    assert pick(32, 2048) == (1, 4)           # 256 wide blocks fit at once
    assert pick(48, 2048) == (1, 2) and pick(64, 2048) == (1, 2)   # 384 and 512 do not; narrow ones do
    assert pick(8, 4000, 40, 1) == (3, 2)     # 320 pairs of a model without grouping: 187 narrow clusters of 3 fit
    assert pick(20, 2048) == (3, 2)           # 160 pairs: 187 narrow clusters of 3 fit, wide ones need two waves or no split
    assert pick(48, 8000) == (2, 4)           # narrow blocks in 4 splits are 4 % better by the model: not enough to leave the wide ones
    assert pick(1, 2048) == (8, 4)            # the cluster's shared memory beats global memory for short contexts
    assert pick(1, 32768)[0] > 8              # a long context wants every slot busy
    for n in (1, 2, 3, 7, 8, 20, 64, 200):
        for ctx in (1, 64, 100, 128, 129, 500, 2048, 100000):
            s, w = pick(n, ctx)
            assert 1 <= s <= 64 and w in (2, 4)
            assert s == 1 or ctx / s >= 64    # a split keeps at least 128 keys (rounded to tiles of 64)
    # one width only (head sizes up to 64): the same rule among its split counts
    assert kernels.decode_plan(64, 8, 4, 2048, 64, (B200_NARROW[:1] + (0.5,) + B200_NARROW[2:],))[0] == 1


def test_one_long_request_among_short_ones_is_split_as_if_nearly_alone():
    plan = lambda n, ctx, mean=None: kernels.decode_plan(n, 8, 4, ctx, 128, B200_WIDTHS, mean_ctx=mean)
    alone = plan(1, 30000)
    assert alone[0] >= 16
    assert plan(64, 30000)[0] == 1                        # 64 long requests fill the device without a split
    s, w = plan(64, 30000, mean=960)                      # one of them long: its keys are split
    assert s >= 6
    from lmsf_b200.engine.model_runner import ModelRunner
    c = ModelRunner.graph_skew_class
    assert [c(4096, m) for m in (4096, 2049, 2048, 1024, 600, 512, 100, 64, 1)] == [0, 0, 1, 2, 2, 3, 5, 6, 6]


def test_split_choice_does_not_depend_on_what_it_should_not():
    plan = lambda n, kv, group: kernels.decode_plan(n, kv, group, 2048, 128, B200_WIDTHS)
    # more query heads per kv head up to 16 share a block: same answer
    assert plan(8, 8, 1) == plan(8, 8, 16)
    # 17 to 32 heads per kv head need two blocks per kv head: as if there were twice the kv heads
    assert plan(8, 8, 32) == plan(8, 16, 4)


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


def test_a_norm_is_split_between_products_only_when_everybody_can():
    """The offer a block makes to the part before a norm (parts/block.py: norm_after): the producer says fuses_norm,
    the reader of the norm says takes_prenormed, the norm says splittable, the step is bfloat16 and has at most 16
    tokens, and there is a residual stream already."""
    import types

    import torch

    from lmsf_b200.parts import block as block_mod
    from lmsf_b200.parts.base import FeedForward, Mixer, Norm, NormAfter

    class Able(Mixer):
        fuses_norm = True
        takes_prenormed = True

    class Plain(FeedForward):
        pass

    class Split(Norm):
        splittable = True

    res = torch.zeros(2, 4)
    step = lambda n, dt=torch.bfloat16: types.SimpleNamespace(dtype=dt, n_tokens=n)
    offer = block_mod.norm_after(step(16), Able(), Split(), Able(), res)
    assert isinstance(offer, NormAfter) and offer.res is res
    assert block_mod.norm_after(step(17), Able(), Split(), Able(), res) is None              # the library's products
    assert block_mod.norm_after(step(8, torch.float32), Able(), Split(), Able(), res) is None
    assert block_mod.norm_after(step(8), Able(), Split(), Able(), None) is None               # the first norm of a step
    assert block_mod.norm_after(step(8), Plain(), Split(), Able(), res) is None
    assert block_mod.norm_after(step(8), Able(), Split(), Plain(), res) is None
    assert block_mod.norm_after(step(8), Able(), Norm(), Able(), res) is None
    assert block_mod.norm_after(None, Plain(), Norm(), Plain(), res) is None                   # parts are asked first
    old = block_mod.FUSE_NORMS
    try:
        block_mod.FUSE_NORMS = False
        assert block_mod.norm_after(step(8), Able(), Split(), Able(), res) is None
    finally:
        block_mod.FUSE_NORMS = old
