"""The plain implementation against itself: properties that any correct Llama decoder has (no GPU)."""
import math

import numpy as np
import torch

import plain_llama as P
import util


def _load(name, std=0.15):
    return P.load_model(util.model_folder(name, "float32", std))


def test_float32_agrees_with_float64():
    for name in "ABW":
        cfg, w = _load(name)
        ids = util.random_ids(40, cfg["vocab_size"], 1)
        a, b = P.forward(cfg, w, ids), P.forward(cfg, w, ids, torch.float64)
        assert (a.double() - b).abs().max() < 2e-5 * max(1.0, b.abs().max())


def test_causality_prefix_logits_do_not_change():
    cfg, w = _load("A")
    ids = util.random_ids(30, cfg["vocab_size"], 2)
    full = P.forward(cfg, w, ids, torch.float64)
    part = P.forward(cfg, w, ids[:11], torch.float64)
    assert torch.allclose(full[:11], part, atol=1e-10)


def test_window_forgets_far_keys():
    cfg, w = _load("W")
    ids = util.random_ids(60, cfg["vocab_size"], 3)
    a = P.forward(cfg, w, ids, torch.float64)
    ids2 = list(ids)
    ids2[0] = (ids2[0] + 1) % cfg["vocab_size"]     # position 0 can reach position p only through layers * (window-1)
    b = P.forward(cfg, w, ids2, torch.float64)
    reach = cfg["num_hidden_layers"] * (cfg["sliding_window"] - 1)
    assert torch.allclose(a[reach + 1:], b[reach + 1:], atol=1e-10) and not torch.allclose(a[:reach], b[:reach], atol=1e-6)


def test_llama3_frequencies():
    cfg = dict(util.TINY_B)
    inv = P.rope_inv_freq(cfg)
    base = torch.tensor([500000.0 ** (-(2.0 * i) / 32) for i in range(16)], dtype=torch.float64)
    wl = 2 * math.pi / base
    assert torch.allclose(inv[wl < 64 / 4], base[wl < 64 / 4])
    assert torch.allclose(inv[wl > 64 / 1], base[wl > 64 / 1] / 8.0)
    mid = (wl >= 16) & (wl <= 64)
    assert mid.any() and torch.all(inv[mid] <= base[mid]) and torch.all(inv[mid] >= base[mid] / 8.0)


def test_rotary_is_a_rotation_and_relative():
    cfg = dict(util.TINY_A)
    inv = P.rope_inv_freq(cfg)
    q = torch.randn(5, 4, 16, dtype=torch.float64)
    k = torch.randn(5, 4, 16, dtype=torch.float64)
    pos = torch.tensor([0, 1, 7, 40, 100])
    rq, rk = P.rotary_neox(q, pos, inv), P.rotary_neox(k, pos, inv)
    assert torch.allclose(rq.norm(dim=-1), q.norm(dim=-1))
    assert torch.allclose(rq[0], q[0])
    rq2, rk2 = P.rotary_neox(q, pos + 13, inv), P.rotary_neox(k, pos + 13, inv)
    assert torch.allclose((rq * rk).sum(-1), (rq2 * rk2).sum(-1), atol=1e-9)


def test_gqa_equals_repeated_kv_heads():
    T, nh, nkv, hd = 9, 6, 2, 8
    q, k, v = torch.randn(T, nh, hd), torch.randn(T, nkv, hd), torch.randn(T, nkv, hd)
    a = P.causal_attention(q, k, v, 0.3)
    b = P.causal_attention(q, k.repeat_interleave(3, dim=1), v.repeat_interleave(3, dim=1), 0.3)
    assert torch.allclose(a, b, atol=1e-6)
    # first token attends to itself only
    assert torch.allclose(a[0], v.repeat_interleave(3, dim=1)[0], atol=1e-6)


def test_rms_norm_and_mlp_formulas():
    x = torch.randn(3, 10, dtype=torch.float64)
    w = torch.randn(10, dtype=torch.float64)
    y = P.rms_norm(x, w, 1e-6)
    assert torch.allclose(y, x / torch.sqrt((x ** 2).mean(-1, keepdim=True) + 1e-6) * w)
    h = torch.randn(4, 6, dtype=torch.float64)
    g, u, d = torch.randn(5, 6, dtype=torch.float64), torch.randn(5, 6, dtype=torch.float64), torch.randn(6, 5, dtype=torch.float64)
    ref = (torch.nn.functional.silu(h @ g.T) * (h @ u.T)) @ d.T
    assert torch.allclose(P.silu_gated_mlp(h, g, u, d), ref)


def test_tied_head_and_generation():
    cfg, w = _load("B")
    assert "lm_head.weight" not in w
    toks, rows = P.generate(cfg, w, [5, 6, 7], 4)
    assert len(toks) == 4 and rows.shape == (4, cfg["vocab_size"])
    assert toks[0] == int(P.forward(cfg, w, [5, 6, 7])[-1].argmax())
    t1, _ = P.generate(cfg, w, [5, 6, 7], 5, temperature=0.8, seed=1)
    t2, _ = P.generate(cfg, w, [5, 6, 7], 5, temperature=0.8, seed=1)
    t3, _ = P.generate(cfg, w, [5, 6, 7], 5, temperature=0.8, seed=2)
    assert t1 == t2 and t1 != t3


def test_philox_known_answer_and_noise_is_exponential():
    # Random123 known-answer vectors for philox4x32-10
    r = P.philox4x32([np.array([0]), np.array([0]), np.array([0]), np.array([0])], (0, 0))
    assert [int(x[0]) for x in r] == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    f = 0xFFFFFFFF
    r = P.philox4x32([np.array([f]), np.array([f]), np.array([f]), np.array([f])], (f, f))
    assert [int(x[0]) for x in r] == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    q = P.exponential_noise(seed=3, step=0, vocab=200000)
    assert abs(q.mean() - 1.0) < 0.01 and abs(q.var() - 1.0) < 0.03 and q.min() >= 0
    # sampling frequencies follow softmax(logits / T)
    logits = torch.tensor([0.0, 1.0, 2.0, -1.0])
    counts = np.zeros(4)
    for step in range(4000):
        counts[P.sample_temperature(logits, 0.7, seed=11, step=step)] += 1
    p = torch.softmax(logits / 0.7, -1).numpy()
    assert np.abs(counts / 4000 - p).max() < 0.03
