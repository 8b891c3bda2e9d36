"""Llama: the description of the decoder as data, and its registry entry.

Structure and tensor names follow core/src/model_executor/models/llama/llama.rs:387-536
(embedding :485, layers :496-505, final norm :494-495, lm_head :487-492) and the weight names that
the linear loaders ask for (core/src/model_executor/layers/linear.rs:573-623, :364-400).
Unlike the reference, `rope_theta`, `rope_scaling`, `head_dim` and `tie_word_embeddings` are
honoured and every constant below comes from config.json.
"""
from __future__ import annotations

from ..config.model_config import LlamaConfig
from ..config.registry import register_architecture
from ..parts.base import LayerCall, LayerSpec, ModelSpec, PartSpec


def llama_spec(cfg: LlamaConfig) -> ModelSpec:
    rs = cfg.rope_scaling
    rope = PartSpec("rotary", dict(rot_dim=cfg.head_dim, theta=cfg.rope_theta, is_neox=True,
                                   scaling_type=rs.rope_type, factor=rs.factor, low_freq_factor=rs.low_freq_factor,
                                   high_freq_factor=rs.high_freq_factor,
                                   original_max_position_embeddings=rs.original_max_position_embeddings))
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        attn_w = {"qkv": [p + "self_attn.q_proj.weight", p + "self_attn.k_proj.weight", p + "self_attn.v_proj.weight"],
                  "o": p + "self_attn.o_proj.weight"}
        if cfg.attention_bias:
            attn_w.update(qkv_bias=[p + "self_attn.q_proj.bias", p + "self_attn.k_proj.bias", p + "self_attn.v_proj.bias"],
                          o_bias=p + "self_attn.o_proj.bias")
        mlp_w = {"gate_up": [p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight"], "down": p + "mlp.down_proj.weight"}
        if cfg.mlp_bias:
            mlp_w.update(gate_up_bias=[p + "mlp.gate_proj.bias", p + "mlp.up_proj.bias"], down_bias=p + "mlp.down_proj.bias")
        layers.append(LayerSpec("pre_norm", {
            "mixer_norm": PartSpec("rmsnorm", dict(hidden_size=cfg.hidden_size, eps=cfg.rms_norm_eps),
                                   {"weight": p + "input_layernorm.weight"}),
            "mixer": PartSpec("paged_attention",
                              dict(hidden_size=cfg.hidden_size, num_heads=cfg.num_attention_heads,
                                   num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
                                   position_encoding=rope, window=cfg.sliding_window, bias=cfg.attention_bias),
                              attn_w),
            "ffn_norm": PartSpec("rmsnorm", dict(hidden_size=cfg.hidden_size, eps=cfg.rms_norm_eps),
                                 {"weight": p + "post_attention_layernorm.weight"}),
            "feed_forward": PartSpec("gated_mlp",
                                     dict(hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
                                          activation=cfg.hidden_act, bias=cfg.mlp_bias),
                                     mlp_w),
        }))
    head_name = "model.embed_tokens.weight" if cfg.tie_word_embeddings else "lm_head.weight"
    ignored = [r".*\.rotary_emb\.inv_freq$"]
    if cfg.tie_word_embeddings:
        ignored.append(r"^lm_head\.weight$")
    return ModelSpec(
        hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size, max_model_len=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size),
                           {"weight": "model.embed_tokens.weight"}),
        layers=layers,
        order=[LayerCall(i) for i in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", dict(hidden_size=cfg.hidden_size, eps=cfg.rms_norm_eps),
                            {"weight": "model.norm.weight"}),
        lm_head=PartSpec("dense", dict(in_features=cfg.hidden_size, out_features=cfg.vocab_size, out_dtype="float32"),
                         {"weight": head_name}),
        eos_token_ids=list(cfg.eos_token_ids),
        ignored_weights=ignored,
    )


register_architecture("LlamaForCausalLM", LlamaConfig.from_dict, llama_spec, aliases=("llama",))
