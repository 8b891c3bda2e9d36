"""Configuration and registry (no GPU)."""
import json

import pytest

import util
from lmsf_b200 import models  # noqa: F401
from lmsf_b200.config import (CacheConfig, ConfigError, EngineArgs, LlamaConfig, SchedulerConfig, canonical_dtype,
                              load_model_config, registered_architectures, resolve_architecture,
                              resolve_max_model_len)


def test_defaults_and_derived_sizes():
    c = LlamaConfig.from_dict(dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4))
    assert c.num_key_value_heads == 4 and c.head_dim == 16
    assert c.rope_theta == 10000.0 and c.rope_scaling.rope_type == "default"
    assert c.rms_norm_eps == 1e-5 and not c.tie_word_embeddings and c.sliding_window is None
    assert c.max_model_len == 4096 and c.vocab_size == 32000 and c.intermediate_size == 11008


def test_every_key_is_read():
    c = LlamaConfig.from_dict(util.TINY_B)
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads) == (96, 3, 3, 1)
    assert c.head_dim == 32 and c.intermediate_size == 256 and c.vocab_size == 320
    assert c.rope_theta == 500000.0 and c.rms_norm_eps == 1e-5 and c.tie_word_embeddings
    rs = c.rope_scaling
    assert (rs.rope_type, rs.factor, rs.low_freq_factor, rs.high_freq_factor,
            rs.original_max_position_embeddings) == ("llama3", 8.0, 1.0, 4.0, 64)
    assert c.eos_token_ids == [2, 3] and c.max_position_embeddings == 256
    # round trip through to_dict
    assert LlamaConfig.from_dict(c.to_dict()) == c


def test_rope_parameters_spelling():
    d = dict(hidden_size=64, num_hidden_layers=1, num_attention_heads=4,
             rope_parameters=dict(rope_type="linear", rope_theta=123.0, factor=2.0))
    c = LlamaConfig.from_dict(d)
    assert c.rope_theta == 123.0 and c.rope_scaling.rope_type == "linear" and c.rope_scaling.factor == 2.0


@pytest.mark.parametrize("patch,needle", [
    (dict(num_attention_heads=5), "not a multiple"),
    (dict(num_key_value_heads=3), "num_key_value_heads"),
    (dict(rope_scaling=dict(rope_type="yarn", factor=2.0)), "yarn"),
    (dict(rope_scaling=dict(rope_type="llama3", factor=2.0)), "lacks"),
    (dict(hidden_act="relu"), "hidden_act"),
    (dict(rms_norm_eps=0.0), "rms_norm_eps"),
    (dict(head_dim=15), "head_dim"),
    (dict(torch_dtype="int8"), "torch_dtype"),
    (dict(sliding_window=0), "sliding_window"),
])
def test_bad_values_are_refused(patch, needle):
    d = dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4)
    d.update(patch)
    with pytest.raises(ConfigError) as e:
        LlamaConfig.from_dict(d)
    assert needle in str(e.value)


def test_missing_mandatory_key():
    with pytest.raises(ConfigError) as e:
        LlamaConfig.from_dict(dict(hidden_size=64, num_attention_heads=4))
    assert "num_hidden_layers" in str(e.value)


def test_registry_lookup_and_miss(tmp_path):
    assert "LlamaForCausalLM" in registered_architectures()
    assert resolve_architecture({"architectures": ["llamaforcausallm"]}).name == "LlamaForCausalLM"
    assert resolve_architecture({"model_type": "LLAMA"}).name == "LlamaForCausalLM"
    with pytest.raises(ConfigError) as e:
        resolve_architecture({"architectures": ["GemmaForCausalLM"], "model_type": "gemma"})
    assert "LlamaForCausalLM" in str(e.value) and "Gemma" in str(e.value)
    with pytest.raises(ConfigError):
        resolve_architecture({})
    (tmp_path / "config.json").write_text(json.dumps(util.TINY_A))
    arch, cfg = load_model_config(str(tmp_path))
    assert arch.name == "LlamaForCausalLM" and cfg.intermediate_size == 172
    with pytest.raises(ConfigError):
        load_model_config(str(tmp_path / "nothing"))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_model_config(str(tmp_path))


def test_spec_carries_every_constant():
    from lmsf_b200.models.llama import llama_spec
    spec = llama_spec(LlamaConfig.from_dict(util.TINY_B))
    assert len(spec.layers) == 3 and [c.layer for c in spec.order] == [0, 1, 2]
    mixer = spec.layers[1].parts["mixer"]
    assert mixer.params["num_heads"] == 3 and mixer.params["num_kv_heads"] == 1 and mixer.params["head_dim"] == 32
    rope = mixer.params["position_encoding"]
    assert rope.params["theta"] == 500000.0 and rope.params["scaling_type"] == "llama3" and rope.params["factor"] == 8.0
    assert spec.layers[0].parts["mixer_norm"].params["eps"] == 1e-5
    assert spec.lm_head.weights["weight"] == "model.embed_tokens.weight"      # tied
    assert llama_spec(LlamaConfig.from_dict(util.TINY_A)).lm_head.weights["weight"] == "lm_head.weight"
    assert llama_spec(LlamaConfig.from_dict(util.TINY_W)).layers[0].parts["mixer"].params["window"] == 24


def test_engine_options():
    assert canonical_dtype("bf16") == "bfloat16" and canonical_dtype("float") == "float32"
    with pytest.raises(ConfigError):
        canonical_dtype("float16")
    assert SchedulerConfig.new(None, 256, 128).max_num_batched_tokens == 2048
    assert SchedulerConfig.new(None, 256, 8192).max_num_batched_tokens == 8192
    assert SchedulerConfig.new(None, 256, 131072).max_num_batched_tokens == 8192      # prompts are cut into portions
    assert SchedulerConfig.new(48, 4, 128).max_num_batched_tokens == 48
    with pytest.raises(ConfigError):
        CacheConfig(block_size=12)
    with pytest.raises(ConfigError):
        CacheConfig(gpu_memory_utilization=1.5)
    assert resolve_max_model_len(None, 128) == 128 and resolve_max_model_len(64, 128) == 64
    with pytest.raises(ConfigError):
        resolve_max_model_len(256, 128)
    import argparse
    ns = EngineArgs.add_cli_args(argparse.ArgumentParser()).parse_args(
        ["--model", "m", "--block-size", "8", "--max-num-batched-tokens", "48", "--gpu-memory-utilization", "0.5",
         "--max-model-len", "100", "--max-num-seqs", "4", "--seed", "7", "--dtype", "float32"])
    a = EngineArgs.from_cli_args(ns)
    assert (a.model, a.block_size, a.max_num_batched_tokens, a.gpu_memory_utilization, a.max_model_len,
            a.max_num_seqs, a.seed, a.dtype) == ("m", 8, 48, 0.5, 100, 4, 7, "float32")
