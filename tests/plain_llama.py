"""Plain, slow implementation of the Llama decoder used as the oracle of the tests.

It is written from the formulas of yinqiwen/lmsf's sources (each function cites file:line).  The reference's
model code is Rust on top of a CUDA-only tensor library and can neither be imported nor compiled on a CPU box,
so there is no golden output of its whole model.  Its CUDA kernels, however, compile unmodified, and
tests/golden/reference_kernels_f32.npz holds what they returned on a B200 (made by
tests/golden/make_reference_kernel_goldens.py): tests/test_golden_reference_kernels.py pins `rms_norm` (with and
without the residual sum), `rotary_neox`, the gated SiLU of `silu_gated_mlp` and `causal_attention` to those
outputs.  What the reference has no code for (rope_theta from config.json, llama3 frequency scaling, tied head,
the keying of the sampler's noise) rests on the formulas alone.

Whole sequences, no cache, one function per part, all arithmetic in one float type
(float32 by default, float64 to bound rounding).  Nothing here imports the product
package: the safetensors reader, the rotary frequencies and the sampler noise are
restated independently.
"""
import json
import math
import struct

import numpy as np
import torch

_ST_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
              "I32": torch.int32, "I64": torch.int64, "F64": torch.float64}


def read_safetensors(path):
    """8-byte little-endian header length, JSON header, raw little-endian data.
    Layout as mmapped by the reference (core/src/model_executor/models/model_factory.rs:133-139)."""
    with open(path, "rb") as f:
        blob = f.read()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n].decode("utf-8"))
    data = memoryview(blob)[8 + n:]
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        b, e = meta["data_offsets"]
        dt = _ST_DTYPES[meta["dtype"]]
        t = torch.frombuffer(bytearray(data[b:e]), dtype=dt) if e > b else torch.empty(0, dtype=dt)
        out[name] = t.reshape(meta["shape"]).clone()
    return out


def load_model(folder):
    with open(f"{folder}/config.json") as f:
        cfg = json.load(f)
    return cfg, read_safetensors(f"{folder}/model.safetensors")


# ----------------------------------------------------------------------------- parts

def head_dim_of(cfg):
    """hd = hidden / heads (core/src/common/config.rs:193-195); an explicit head_dim key wins."""
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


def rope_inv_freq(cfg):
    """inv_freq_i = theta^(-2i/hd) (vllm/src/pos_encoding.rs:8-16).  The reference ignores
    rope_theta and has no scaling (core/src/model_executor/models/llama/llama.rs:207-215);
    here theta comes from config.json and the llama3 rule rescales by wavelength."""
    hd = head_dim_of(cfg)
    theta = float(cfg.get("rope_theta", 10000.0))
    inv = [theta ** (-(2.0 * i) / hd) for i in range(hd // 2)]
    sc = cfg.get("rope_scaling")
    if sc:
        kind = sc.get("rope_type", sc.get("type", "default"))
        if kind == "llama3":
            factor, low, high = float(sc["factor"]), float(sc["low_freq_factor"]), float(sc["high_freq_factor"])
            old = float(sc["original_max_position_embeddings"])
            res = []
            for f in inv:
                wavelen = 2.0 * math.pi / f
                if wavelen < old / high:
                    res.append(f)
                elif wavelen > old / low:
                    res.append(f / factor)
                else:
                    s = (old / wavelen - low) / (high - low)
                    res.append((1.0 - s) * f / factor + s * f)
            inv = res
        elif kind == "linear":
            inv = [f / float(sc["factor"]) for f in inv]
        elif kind != "default":
            raise ValueError(kind)
    return torch.tensor(inv, dtype=torch.float64)


def embedding(table, ids):
    """x[t] = E[id_t] (core/src/model_executor/layers/vocab_parallel_embedding.rs:28-37)."""
    return table[ids]


def rms_norm(x, w, eps):
    """x * rsqrt(mean(x^2) + eps) * w (vllm/kernels/layernorm_kernels.cu:13-37)."""
    var = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * w


def rotary_neox(v, positions, inv_freq):
    """NeoX pairs (i, i + hd/2): x' = x cos - y sin, y' = y cos + x sin
    (vllm/kernels/pos_encoding_kernels.cu:12-41).  v: [T, heads, hd].
    Angles are formed as float32(position) * float32(inv_freq) like the reference's table
    (vllm/src/pos_encoding.rs:24-31) unless v is float64."""
    adt = torch.float64 if v.dtype == torch.float64 else torch.float32
    ang = positions.to(adt)[:, None] * inv_freq.to(adt)[None, :]
    cos, sin = ang.cos().to(v.dtype)[:, None, :], ang.sin().to(v.dtype)[:, None, :]
    half = v.shape[-1] // 2
    x, y = v[..., :half], v[..., half:]
    return torch.cat([x * cos - y * sin, y * cos + x * sin], dim=-1)


def causal_attention(q, k, v, scale, window=None):
    """softmax(mask(q k^T * scale)) v, kv head g serves query heads g*r .. g*r+r-1
    (core/src/model_executor/layers/attention.rs:91-155).  q: [T, nh, hd]; k, v: [T, nkv, hd].
    window w keeps keys j with i - w < j <= i."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    r = nh // nkv
    out = torch.empty_like(q)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    dead = j > i
    if window:
        dead = dead | (j <= i - window)
    for h in range(nh):
        g = h // r
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        s = s.masked_fill(dead, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, g, :]
    return out


def silu_gated_mlp(h, w_gate, w_up, w_down):
    """(silu(h Wg^T) * (h Wu^T)) Wd^T (core/src/model_executor/models/llama/llama.rs:235-250,
    vllm/kernels/activation_kernels.cu:26-41)."""
    g = h @ w_gate.T
    u = h @ w_up.T
    return ((g / (1.0 + torch.exp(-g))) * u) @ w_down.T


def gate_activation(g, name):
    """silu: x / (1 + e^-x) (vllm/kernels/activation_kernels.cu:26-29); gelu_pytorch_tanh: the tanh form
    0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) (activation_kernels.cu:44-51, gelu_new / gelu_fast family)."""
    if name in ("silu", "swish"):
        return g / (1.0 + torch.exp(-g))
    if name in ("gelu_tanh", "gelu_pytorch_tanh"):
        return 0.5 * g * (1.0 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g * g * g)))
    raise ValueError(name)


def linear(x, w, name):
    """x W^T + b; the bias is there only when config.json asks for it (core/src/model_executor/layers/linear.rs:95-104)."""
    y = x @ w[name + ".weight"].T
    b = w.get(name + ".bias")
    return y if b is None else y + b


def _identity(x):
    return x


def attention_block(cfg, w, prefix, h, positions, inv_freq, r=_identity):
    """q,k,v projections, rotary on q and k, causal attention, output projection
    (core/src/model_executor/models/llama/llama.rs:95-135).  r rounds what the engine stores (see forward)."""
    nh, hd = cfg["num_attention_heads"], head_dim_of(cfg)
    nkv = cfg.get("num_key_value_heads") or nh
    T = h.shape[0]
    q = r(linear(h, w, prefix + "q_proj")).reshape(T, nh, hd)
    k = r(linear(h, w, prefix + "k_proj")).reshape(T, nkv, hd)
    v = r(linear(h, w, prefix + "v_proj")).reshape(T, nkv, hd)
    q = r(rotary_neox(q, positions, inv_freq))
    k = r(rotary_neox(k, positions, inv_freq))
    o = r(causal_attention(q, k, v, 1.0 / math.sqrt(hd), cfg.get("sliding_window")))
    return r(linear(o.reshape(T, nh * hd), w, prefix + "o_proj"))


def forward(cfg, weights, token_ids, dtype=torch.float32, stored=None):
    """Logits [T, vocab] of one whole sequence (core/src/model_executor/models/llama/llama.rs:397-476;
    the residual adds that the reference folds into the next norm are written out).

    `stored` (e.g. torch.bfloat16) rounds every tensor that a bfloat16 engine writes to memory to that type and
    back: the outputs of norms, projections, the rotation, the attention and the gated product.  The sums inside
    a product or a softmax and the residual stream stay in `dtype`.  It states what a bfloat16 run may differ by
    from exact arithmetic, so that a comparison with it can be held to a tighter bound than one with the exact
    result; the formulas are the same."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    r = _identity if stored is None else (lambda x: x.to(stored).to(dtype))
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    positions = torch.arange(len(ids))
    inv_freq = rope_inv_freq(cfg)
    eps = float(cfg.get("rms_norm_eps", 1e-5))
    x = embedding(w["model.embed_tokens.weight"], ids)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        h = r(rms_norm(x, w[p + "input_layernorm.weight"], eps))
        x = x + attention_block(cfg, w, p + "self_attn.", h, positions, inv_freq, r)
        h = r(rms_norm(x, w[p + "post_attention_layernorm.weight"], eps))
        act = cfg.get("hidden_act", "silu")
        if stored is None and act == "silu" and not cfg.get("mlp_bias"):
            x = x + silu_gated_mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                                   w[p + "mlp.down_proj.weight"])
        else:
            g, u = r(linear(h, w, p + "mlp.gate_proj")), r(linear(h, w, p + "mlp.up_proj"))
            x = x + r(linear(r(gate_activation(g, act) * u), w, p + "mlp.down_proj"))
    x = r(rms_norm(x, w["model.norm.weight"], eps))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return x @ head.T


# ----------------------------------------------------------------------------- sampling

def greedy(logits_row):
    """argmax, lowest index wins ties (core/src/model_executor/layers/sampler.rs:363-384)."""
    return int(torch.argmax(logits_row.double()).item())


_PHILOX_M0, _PHILOX_M1 = 0xD2511F53, 0xCD9E8D57
_PHILOX_W0, _PHILOX_W1 = 0x9E3779B9, 0xBB67AE85


def philox4x32(counter, key):
    """Philox-4x32-10 (Salmon et al. 2011) on numpy uint64 lanes; counter: 4 arrays, key: 2 ints."""
    c = [np.asarray(x, dtype=np.uint64) for x in counter]
    k0, k1 = np.uint64(key[0]), np.uint64(key[1])
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = np.uint64(_PHILOX_M0) * c[0]
        p1 = np.uint64(_PHILOX_M1) * c[2]
        hi0, lo0 = p0 >> np.uint64(32), p0 & mask
        hi1, lo1 = p1 >> np.uint64(32), p1 & mask
        c = [(hi1 ^ c[1] ^ k0) & mask, lo1, (hi0 ^ c[3] ^ k1) & mask, lo0]
        k0 = (k0 + np.uint64(_PHILOX_W0)) & mask
        k1 = (k1 + np.uint64(_PHILOX_W1)) & mask
    return c


def exponential_noise(seed, step, vocab):
    """q_v ~ Exp(1) for every vocabulary id: u from the first Philox word of counter
    (v, step, 0, 0) under key (seed lo, seed hi); q = -log(u), u in (0, 1]."""
    v = np.arange(vocab, dtype=np.uint64)
    z = np.zeros(vocab, dtype=np.uint64)
    r = philox4x32([v, z + np.uint64(step), z, z], (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))
    u = (r[0].astype(np.float64) + 1.0) * (1.0 / 4294967296.0)
    return -np.log(u)


def sample_temperature(logits_row, temperature, seed, step):
    """argmax(softmax(logits / T) / q), q ~ Exp(1)
    (core/src/model_executor/layers/sampler.rs:326-361, :887-888)."""
    z = logits_row.double().numpy() / temperature
    score = z - np.log(exponential_noise(seed, step, len(z)))
    return int(np.argmax(score))


def generate(cfg, weights, prompt, n_tokens, temperature=0.0, seed=0, dtype=torch.float32):
    """Recompute the whole sequence for every new token."""
    ids = list(prompt)
    out, rows = [], []
    for step in range(n_tokens):
        logits = forward(cfg, weights, ids, dtype)[-1]
        rows.append(logits)
        tok = greedy(logits) if temperature < 1e-5 else sample_temperature(logits.float(), temperature, seed, step)
        out.append(tok)
        ids.append(tok)
    return out, torch.stack(rows)


def apply_penalties(logits_row, prompt, output, presence, frequency, repetition):
    """core/src/model_executor/layers/sampler.rs:48-137: repetition on tokens of prompt or output
    (x > 0 ? x / r : x * r), then x -= frequency * count(output), then x -= presence * [count(output) > 0]."""
    x = logits_row.clone().double()
    seen = set(prompt) | set(output)
    for t in seen:
        x[t] = x[t] / repetition if x[t] > 0 else x[t] * repetition
    for t in set(output):
        c = output.count(t)
        x[t] -= frequency * c
        x[t] -= presence
    return x.float()


def filter_logits(z, top_k=-1, top_p=1.0, min_p=0.0):
    """z = logits / T.  top-k then top-p on the ascending sort (core/src/model_executor/layers/sampler.rs:139-210):
    values below the k-th largest go to -inf; of the rest the ascending prefix whose cumulative probability is
    <= 1 - p goes to -inf, the largest always stays.  min-p (sampler.rs:305-312): probability < min_p * largest."""
    z = z.clone().double()
    V = len(z)
    srt, idx = torch.sort(z)
    if 0 < top_k < V:
        kth = srt[V - top_k]
        srt = srt.masked_fill(srt < kth, float("-inf"))
    if top_p < 1.0:
        probs = torch.softmax(srt, dim=-1)
        cum = torch.cumsum(probs, dim=-1)
        mask = cum <= 1.0 - top_p
        mask[-1] = False
        srt = srt.masked_fill(mask, float("-inf"))
    out = torch.empty_like(z)
    out[idx] = srt
    if min_p > 0.0:
        probs = torch.softmax(out, dim=-1)
        out = out.masked_fill(probs < min_p * probs.max(), float("-inf"))
    return out


def sample_filtered(logits_row, temperature, seed, step, top_k=-1, top_p=1.0, min_p=0.0):
    z = filter_logits(logits_row.double() / temperature, top_k, top_p, min_p).numpy()
    score = z - np.log(exponential_noise(seed, step, len(z)))
    return int(np.argmax(score))
