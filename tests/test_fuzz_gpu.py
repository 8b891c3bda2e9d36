"""Random tiny configurations through the replay harness: head sizes in steps of 16 up to 256, any number of heads
and groups, widths, feed-forward sizes and vocabularies that are no power of two, windows, frequency scaling, tied
heads and page sizes, each replayed three ways in float32 and bfloat16 against the plain implementation."""
import random
import tempfile

import numpy as np
import pytest

import plain_llama as P
import traces
import util

pytestmark = pytest.mark.gpu



def random_config(seed):
    rng = random.Random(seed)
    nkv = rng.choice([1, 2, 3, 4])
    nh = nkv * rng.choice([1, 1, 2, 3, 4, 5, 8])
    cfg = dict(architectures=["LlamaForCausalLM"], model_type="llama",
               hidden_size=rng.choice([24, 40, 56, 72, 88, 104, 120, 136, 200]), num_hidden_layers=rng.choice([1, 2, 3]),
               num_attention_heads=nh, num_key_value_heads=nkv,
               head_dim=rng.choice([16, 32, 48, 64, 64, 80, 96, 112, 128, 128, 144, 192, 256]),
               intermediate_size=rng.choice([40, 72, 100, 172, 250, 328]), vocab_size=rng.choice([97, 211, 256, 391, 1001, 2049]),
               rope_theta=rng.choice([10000.0, 500000.0]), rms_norm_eps=rng.choice([1e-5, 1e-6]),
               tie_word_embeddings=rng.random() < 0.5, max_position_embeddings=1024, hidden_act="silu",
               bos_token_id=1, eos_token_id=2)
    if rng.random() < 0.3:
        cfg["sliding_window"] = rng.choice([8, 24, 40, 100])
    if rng.random() < 0.3:
        cfg["rope_scaling"] = dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                   original_max_position_embeddings=64)
    block_size = rng.choice([8, 16, 32])
    # drawn last so that the sizes of a seed stay what they were: biases and the other gate activation
    extra = random.Random(seed + 1000)
    cfg["attention_bias"], cfg["mlp_bias"] = extra.random() < 0.4, extra.random() < 0.4
    if extra.random() < 0.3:
        cfg["hidden_act"] = "gelu_pytorch_tanh"
    lengths = [rng.choice([1, 2, 3, 9, 17, 40, 64, 65, 127, 128, 129, 200, 300]) for _ in range(4)]
    return cfg, block_size, lengths, rng.choice([0.02, 0.15])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(10))
def test_random_configurations(seed, dtype):
    from lmsf_b200 import models  # noqa: F401
    from lmsf_b200.weights import write_random_model
    cfg, bs, lengths, std = random_config(seed)
    with tempfile.TemporaryDirectory(prefix="lmsf_fuzz_") as folder:
        write_random_model(folder, dict(cfg), seed=seed, dtype=dtype, std=std)
        reqs = {f"r{i}": util.random_ids(n, cfg["vocab_size"], seed * 100 + i) for i, n in enumerate(lengths)}
        c, w = P.load_model(folder)
        ref = util.oracle_logits(c, w, reqs, dtype)
        # the random shapes reach kernels and paths that the four tiny configurations do not: 0.026 of the logit
        # scale was the worst seen at a standard deviation of 0.15, 0.0051 at 0.02
        bound, scale = util.logits_bound(dtype, std, ref, bf16_rel=1.4 * util.BF16_REL[std])
        plans = {"tail32": traces.whole(reqs, tail=32), "mixed": traces.mixed(reqs, seed=seed),
                 "portions": traces.portions(reqs, [7, 2, 13, 2, 31, 3])}
        for mode, steps in plans.items():
            out = traces.run_inprocess(folder, dtype, steps, bs, traces.max_live_tokens(steps, round_to=bs))
            rows = traces.collect(steps, out)
            assert len(rows) == sum(len(t) for t in reqs.values())
            worst = util.worst_difference(rows, ref)
            util.note_worst(f"fuzz {seed} {mode} {dtype} std {std} hd {cfg['head_dim']} width {cfg['hidden_size']}", worst, bound)
            assert worst <= bound, (f"{mode}: max |diff| {worst:.3e} against {bound:.3e} at logit scale {scale:.3f}; "
                                    f"{cfg}, pages of {bs}, prompts of {lengths}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,inter,vocab,hd", [(33, 21, 55, 16), (7, 5, 11, 16), (50, 99, 211, 32)])
def test_odd_widths(hidden, inter, vocab, hd, dtype):
    """Widths, feed-forward sizes and vocabularies that are odd or no multiple of 8: the vectorised kernels and the
    weight-streaming products must step aside for their plain forms, never give a wrong result."""
    from lmsf_b200 import models  # noqa: F401
    from lmsf_b200.weights import write_random_model
    cfg = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=hidden, num_hidden_layers=2,
               num_attention_heads=3, num_key_value_heads=1, head_dim=hd, intermediate_size=inter, vocab_size=vocab,
               rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=hidden % 2 == 0, max_position_embeddings=256,
               hidden_act="silu", bos_token_id=1, eos_token_id=2)
    with tempfile.TemporaryDirectory(prefix="lmsf_fuzz_") as folder:
        write_random_model(folder, dict(cfg), seed=1, dtype=dtype, std=0.05)
        reqs = {f"r{i}": util.random_ids(n, vocab, i) for i, n in enumerate([3, 40, 129, 17])}
        c, w = P.load_model(folder)
        ref = util.oracle_logits(c, w, reqs, dtype)
        bound, scale = util.logits_bound(dtype, 0.05, ref)
        for steps in (traces.whole(reqs, tail=32), traces.mixed(reqs, seed=3)):
            out = traces.run_inprocess(folder, dtype, steps, 16, traces.max_live_tokens(steps, round_to=16))
            rows = traces.collect(steps, out)
            worst = util.worst_difference(rows, ref)
            util.note_worst(f"odd widths {hidden} {dtype}", worst, bound)
            assert worst <= bound, f"max |diff| {worst:.3e} against {bound:.3e} at logit scale {scale:.3f}"
