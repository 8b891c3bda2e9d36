"""Llama-3-8B's layer sizes (hidden 4096, 32 query / 8 kv heads of 128, intermediate 14336) with two layers and a
small vocabulary: the kernels at the sizes that serving uses (tcgen05 prefill attention, split-key decode, the
weight-streaming products, CUDA graphs), against the plain implementation, in float32 and in bfloat16."""
import numpy as np
import pytest

import plain_llama as P
import traces
import util

pytestmark = pytest.mark.gpu

REAL = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=4096, num_hidden_layers=2,
            num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=4099,
            rope_theta=500000.0,
            rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                              original_max_position_embeddings=8192),
            rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=8192, hidden_act="silu",
            bos_token_id=1, eos_token_id=2)
util.CONFIGS["REAL"] = REAL


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_layer_sizes(dtype):
    folder = util.model_folder("REAL", dtype, 0.02)
    cfg, w = P.load_model(folder)
    reqs = {"a": util.random_ids(300, cfg["vocab_size"], 1), "b": util.random_ids(70, cfg["vocab_size"], 2)}
    ref = util.oracle_logits(cfg, w, reqs, dtype)
    # sums over 4,096 and 14,336 terms round more than the tiny models' do: 0.0103 of the logit scale was seen
    bound, scale = util.logits_bound(dtype, 0.02, ref, bf16_rel=2.0e-2)
    if dtype == "float32":
        bound *= 2.0                         # sums over 4,096 and 14,336 terms
    # whole; a long portion then single tokens (the decode path and its CUDA graph); mixed portions
    plans = {"whole": traces.whole(reqs), "tail": traces.whole(reqs, tail=20), "mixed": traces.mixed(reqs, seed=3, tail=10)}
    for mode, steps in plans.items():
        out = traces.collect(steps, traces.run_inprocess(folder, dtype, steps, 16, traces.max_live_tokens(steps, 16)))
        worst = util.worst_difference(out, ref)
        util.note_worst(f"real sizes {mode} {dtype}", worst, bound)
        assert len(out) == 370 and worst <= bound, (mode, worst, bound, scale)
