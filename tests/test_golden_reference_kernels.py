"""The plain implementation against outputs of yinqiwen/lmsf's own CUDA kernels.

tests/golden/reference_kernels_f32.npz holds what the reference's kernels (compiled unmodified for sm_100a, run
once on a B200 by tests/golden/make_reference_kernel_goldens.py) returned in float32 for the inputs of
tests/golden/golden_inputs.py.  These tests need no GPU: they rebuild the inputs and check that the functions of
tests/plain_llama.py give the same numbers, so RMSNorm with and without the residual sum, the NeoX rotation, the
gated SiLU and the attention of a query over its keys are pinned by the reference's output and not only by a
reading of its formulas.  (The reference was built with --use_fast_math and its softmax adds 1e-6 to the sum.)
"""
import math
import os
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import plain_llama  # noqa: E402
from golden_inputs import CASES, values  # noqa: E402

GOLDEN = os.path.join(HERE, "golden", "reference_kernels_f32.npz")
pytestmark = pytest.mark.skipif(not os.path.isfile(GOLDEN), reason="the golden file has not been made yet")


@pytest.fixture(scope="module")
def gold():
    return {k: torch.from_numpy(v) for k, v in np.load(GOLDEN).items()}


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a))


def close(a, b, tol):
    err = float((a.double() - b.double()).abs().max() / b.double().abs().max())
    assert err <= tol, err


def test_rms_norm(gold):
    c = CASES["rms"]
    x, r, w = (t(values(c["n"] * c["hidden"], 1).reshape(c["n"], -1)), t(values(c["n"] * c["hidden"], 2).reshape(c["n"], -1)),
               t(1.0 + values(c["hidden"], 3, 0.2)))
    close(plain_llama.rms_norm(x, w, c["eps"]), gold["rms_norm"], 2e-6)
    close(x + r, gold["fused_add_rms_norm_residual"], 1e-7)
    close(plain_llama.rms_norm(x + r, w, c["eps"]), gold["fused_add_rms_norm_x"], 2e-6)


def test_rotary(gold):
    c = CASES["rope"]
    n, nh, nkv, hd = c["n"], c["heads"], c["kv_heads"], c["head"]
    q, k = t(values(n * nh * hd, 4).reshape(n, nh, hd)), t(values(n * nkv * hd, 5).reshape(n, nkv, hd))
    inv = plain_llama.rope_inv_freq(dict(hidden_size=nh * hd, num_attention_heads=nh, head_dim=hd, rope_theta=c["theta"]))
    pos = torch.tensor(c["positions"])
    # float32 angles up to 1,000 rad: cos and sin of the two libraries differ in the last places
    close(plain_llama.rotary_neox(q, pos, inv).reshape(n, -1), gold["rotary_q"], 2e-5)
    close(plain_llama.rotary_neox(k, pos, inv).reshape(n, -1), gold["rotary_k"], 2e-5)


def test_gated_silu(gold):
    c = CASES["silu"]
    d = c["d"]
    x = t(values(c["n"] * 2 * d, 6, 4.0).reshape(c["n"], -1))
    eye, zero = torch.eye(d), torch.zeros(d, d)
    got = plain_llama.silu_gated_mlp(x, torch.cat([eye, zero], 1), torch.cat([zero, eye], 1), eye)
    close(got, gold["silu_and_mul"], 2e-6)


@pytest.mark.parametrize("which", ["v1", "v2"])
def test_attention_over_pages(gold, which):
    c = CASES["attn"]
    nh, nkv, hd, ctx = c["heads"], c["kv_heads"], c["head"], c["ctx"]
    q = t(values(len(ctx) * nh * hd, 30, 4.0).reshape(len(ctx), nh, hd))
    for s, L in enumerate(ctx):
        keys = t(values(L * nkv * hd, 10 + s).reshape(L, nkv, hd))
        vals = t(values(L * nkv * hd, 20 + s).reshape(L, nkv, hd))
        qs = torch.zeros(L, nh, hd)
        qs[-1] = q[s]                                  # the decoded token is the last of its sequence
        got = plain_llama.causal_attention(qs, keys, vals, 1.0 / math.sqrt(hd))[-1]
        close(got, gold["paged_attention_" + which][s], 2e-5)
