"""Tiny configurations, model folders and trace helpers shared by the tests."""
import random
import tempfile

# Two tiny Llama configurations that differ in every size and option.
TINY_A = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=64, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, intermediate_size=172, vocab_size=256,
              rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=128,
              hidden_act="silu", bos_token_id=1, eos_token_id=2)
TINY_B = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=96, num_hidden_layers=3,
              num_attention_heads=3, num_key_value_heads=1, head_dim=32, intermediate_size=256, vocab_size=320,
              rope_theta=500000.0,
              rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                original_max_position_embeddings=64),
              rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=256, hidden_act="silu",
              bos_token_id=1, eos_token_id=[2, 3])
# a third one with a sliding window and a head size that is no power of two
TINY_W = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=80, num_hidden_layers=2,
              num_attention_heads=5, num_key_value_heads=5, head_dim=48, intermediate_size=100, vocab_size=211,
              rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=512,
              sliding_window=24, hidden_act="silu", bos_token_id=1, eos_token_id=2)

# a fourth one with the head size of the tcgen05 attention kernel, an odd group of query heads (a pair and a single
# head per block) and prompts that span several 128-token query tiles
TINY_C = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=80, num_hidden_layers=2,
              num_attention_heads=6, num_key_value_heads=2, head_dim=64, intermediate_size=112, vocab_size=391,
              rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=512,
              hidden_act="silu", bos_token_id=1, eos_token_id=2)

BLOCK_SIZE = {"A": 8, "B": 16, "W": 16, "C": 16}
CONFIGS = {"A": TINY_A, "B": TINY_B, "W": TINY_W, "C": TINY_C}

_folders = {}


def model_folder(name, dtype="float32", std=0.02, seed=0):
    """A temporary model folder for a tiny configuration (made once per process)."""
    from lmsf_b200 import models  # noqa: F401
    from lmsf_b200.weights import write_random_model
    key = (name, dtype, std, seed)
    if key not in _folders:
        d = tempfile.mkdtemp(prefix=f"lmsf_tiny_{name}_")
        write_random_model(d, dict(CONFIGS[name]), seed=seed, dtype=dtype, std=std)
        _folders[key] = d
    return _folders[key]


def random_ids(n, vocab, seed):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


def cut(tokens, sizes):
    """Cuts a token list into portions of the given sizes (cycled), the last one shortened."""
    out, i, k = [], 0, 0
    while i < len(tokens):
        n = sizes[k % len(sizes)]
        out.append(tokens[i:i + n])
        i += n
        k += 1
    return out


# ----------------------------------------------------------------------------- bounds of the model-level comparisons

# bfloat16 runs are compared with the plain implementation evaluated with the same stored roundings
# (plain_llama.forward(stored=torch.bfloat16)); the bound is a fraction of the largest logit, about twice the worst
# difference seen per standard deviation of the weights (0.0046 at 0.02, 0.017 at 0.15 on the tiny configurations):
# a page of 16 keys read twice in place of its neighbour moves the logits by 0.2 to 1.2 of their scale, one wrong
# key by about a sixteenth of that.
BF16_REL = {0.02: 1.0e-2, 0.05: 2.0e-2, 0.15: 3.5e-2}
F32_REL = 1e-5


def oracle_logits(cfg, weights, reqs, dtype):
    """{request: logits [T, vocab]} of the plain implementation; for bfloat16 with the engine's stored roundings."""
    import plain_llama as P
    import torch
    stored = torch.bfloat16 if dtype == "bfloat16" else None
    return {rid: P.forward(cfg, weights, toks, stored=stored).numpy() for rid, toks in reqs.items()}


def logits_bound(dtype, std, ref, bf16_rel=None):
    """The largest |difference| a run in `dtype` may show against `ref` (a dict of logit arrays); bf16_rel replaces
    the table's fraction where a test has measured its own."""
    import numpy as np
    scale = max(float(np.abs(r).max()) for r in ref.values())
    if dtype == "float32":
        return F32_REL * max(1.0, scale), scale
    return (bf16_rel or BF16_REL[std]) * scale, scale


def worst_difference(rows, ref):
    import numpy as np
    return max(float(np.abs(row - ref[rid][pos]).max()) for (rid, pos), row in rows.items())


def note_worst(what, worst, bound):
    """Appends the worst difference of a comparison to the file $LMSF_TEST_WORST names (to set bounds by)."""
    import os
    path = os.environ.get("LMSF_TEST_WORST")
    if path:
        with open(path, "a") as f:
            f.write(f"{what}\t{worst:.3e}\t{bound:.3e}\t{worst / bound:.3f}\n")


def assert_tokens_within_rounding(cfg, weights, prompt, got, dtype, std, temperature=0.0, seed=0):
    """Every generated token must be the best choice, or within rounding of it, given the tokens generated before
    it: the plain implementation is run once over prompt + got and the row that predicts got[i] is looked at.
    float32 runs must pick the best exactly; bfloat16 runs may pick another token whose (noised) score lies within
    twice the logit bound of the best."""
    import numpy as np
    import plain_llama as P
    import torch
    stored = torch.bfloat16 if dtype == "bfloat16" else None
    rows = P.forward(cfg, weights, list(prompt) + list(got), stored=stored)[len(prompt) - 1:len(prompt) - 1 + len(got)]
    bound, _ = logits_bound(dtype, std, {"x": rows.numpy()})
    for i, tok in enumerate(got):
        z = rows[i].double().numpy()
        if temperature >= 1e-5:
            z = z / temperature - np.log(P.exponential_noise(seed, i, len(z)))
            tol = 2.0 * bound / temperature
        else:
            tol = 2.0 * bound
        best = int(np.argmax(z))
        if dtype == "float32":
            assert tok == best, (i, tok, best)
        else:
            assert z[best] - z[tok] <= tol, (i, tok, best, float(z[best] - z[tok]), tol)
