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
