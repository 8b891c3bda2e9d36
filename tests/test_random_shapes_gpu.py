"""Kernels against their plain twins on many random shapes (seeded): the tcgen05 prefill attention against the
mma.sync one, the decode attention (planned splits and widths, and splits per request) against the generic kernel,
the weight-streaming product, its residual form and its prenormed input against float64.  Longer runs of the same loops found an order of calls in which a
decode launch was refused and a gated product of exactly 8 features that read zeros; the suite keeps a short run."""
import math
import os
import random

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SOAK = int(os.environ.get("LMSF_TEST_SOAK", "1"))     # a longer run of the same loops: LMSF_TEST_SOAK=10


def dev():
    return torch.device("cuda:0")


def _paged(rng, d, ctx_lens, nkv, bs, hd):
    """Pages in random order for requests of the given lengths: (cache, block table)."""
    pages_per = [(c + bs - 1) // bs for c in ctx_lens]
    n_pages = sum(pages_per) + 3
    cache = (torch.randn(n_pages, 2, nkv, bs, hd, device=d) * 0.5).to(torch.bfloat16)
    perm = torch.randperm(n_pages, device=d, dtype=torch.int32)
    bt = torch.full((len(ctx_lens), max(pages_per) + 1), -1, dtype=torch.int32, device=d)
    o = 0
    for i, p in enumerate(pages_per):
        bt[i, :p] = perm[o:o + p]
        o += p
    return cache, bt


@pytest.mark.parametrize("seed", [1, 2])
def test_prefill_attention_on_random_shapes(seed, monkeypatch):
    from lmsf_b200 import kernels
    rng = random.Random(seed)
    torch.manual_seed(seed)
    d = dev()
    i32 = lambda l: torch.tensor(l, dtype=torch.int32, device=d)
    for case in range(200 * SOAK):
        hd = rng.choice([64, 128])
        nkv = rng.choice([1, 2, 3, 4, 8])
        group = rng.choice([1, 2, 3, 4, 5, 8])
        nh = nkv * group
        bs = rng.choice([4, 8, 16, 32, 128])
        window = rng.choice([0, 0, 0, 70, 300, 1000])
        q_lens, ctx_lens = [], []
        for _ in range(rng.randint(1, 10)):
            kind = rng.random()
            q = rng.randint(2, 60) if kind < 0.3 else (rng.randint(60, 400) if kind < 0.8 else rng.randint(400, 1800))
            q_lens.append(q)
            ctx_lens.append(q + rng.choice([0, 0, rng.randint(1, 200), rng.randint(200, 2000)]))
        if rng.random() < 0.5:                 # few blocks: every block takes many units of work in turn
            monkeypatch.setenv("LMSF_TC_MAX_BLOCKS", str(rng.choice([1, 2, 3, 7, 20])))
        else:
            monkeypatch.delenv("LMSF_TC_MAX_BLOCKS", raising=False)
        cache, bt = _paged(rng, d, ctx_lens, nkv, bs, hd)
        q = (torch.randn(sum(q_lens), nh * hd, device=d) * 0.7).to(torch.bfloat16)
        cu = i32([0] + list(np.cumsum(q_lens)))
        cl = i32(ctx_lens)
        t128 = [(i, q0) for i, n in enumerate(q_lens) for q0 in range(0, n, 128)]
        t128.sort(key=lambda t: -(ctx_lens[t[0]] - q_lens[t[0]] + min(q_lens[t[0]], t[1] + 128)))
        t64 = [(i, q0) for i, n in enumerate(q_lens) for q0 in range(0, n, 64)]
        flag = torch.zeros(1, dtype=torch.int32, device=d)
        out, twin = torch.zeros_like(q), torch.zeros_like(q)
        scale = 1 / math.sqrt(hd)
        kernels.attention_prefill_tc(out, q, cache, bt, bs, i32([t[0] for t in t128]), i32([t[1] for t in t128]), len(t128),
                                     cu, cl, scale, window, nh, nkv, hd, flag)
        kernels.attention_prefill(twin, q, cache, bt, bs, i32([t[0] for t in t64]), i32([t[1] for t in t64]), len(t64),
                                  cu, cl, scale, window, nh, nkv, hd)
        what = (seed, case, hd, nkv, group, bs, window, q_lens, ctx_lens)
        assert flag.item() == 0, what
        assert torch.isfinite(out.float()).all().item(), what
        err = (out.float() - twin.float()).abs().max().item()
        assert err <= 2e-2 * max(twin.float().abs().max().item(), 1e-3), (err, what)


@pytest.mark.parametrize("seed", [1, 2])
def test_decode_attention_on_random_shapes(seed):
    from lmsf_b200 import kernels
    rng = random.Random(seed)
    torch.manual_seed(seed)
    d = dev()
    for case in range(300 * SOAK):
        hd = rng.choice([16, 32, 48, 64, 80, 96, 112, 128])
        nkv = rng.choice([1, 2, 4, 8])
        group = rng.choice([1, 2, 3, 4, 8, 17])
        nh = nkv * group
        bs = rng.choice([4, 8, 16, 32])
        window = rng.choice([0, 0, 0, 90, 700])
        n_req = rng.randint(1, 70)
        ctx_lens = [rng.randint(1, 600) for _ in range(n_req)]
        if rng.random() < 0.4:
            ctx_lens[rng.randrange(n_req)] = rng.randint(2000, 9000)
        r_w, r_s, alt = rng.random(), rng.random(), rng.choice([1, 37, 100])
        cache, bt = _paged(rng, d, ctx_lens, nkv, bs, hd)
        q = (torch.randn(n_req, nh * hd, device=d) * 0.7).to(torch.bfloat16)
        cu = torch.arange(n_req + 1, dtype=torch.int32, device=d)
        cl = torch.tensor(ctx_lens, dtype=torch.int32, device=d)
        scale = 1 / math.sqrt(hd)
        ref = torch.zeros_like(q)
        kernels.attention_generic(ref, q, cache, bt, bs, torch.arange(n_req, dtype=torch.int32, device=d),
                                  (cl - 1).to(torch.int32), scale, window, nh, nkv, hd)
        # the plan the attention part would make
        widths = kernels.decode_widths(hd, group)
        longest = max(ctx_lens)
        visible = min(longest, window) if window else longest
        mean = min(sum(ctx_lens) / n_req, visible)
        splits, warps = kernels.decode_plan(n_req, nkv, group, visible, hd, widths,
                                            mean_ctx=mean if mean * 4 <= visible * 3 else None)
        out = torch.zeros_like(q)
        scratch = torch.zeros(max(1, kernels.attention_decode_scratch_floats(n_req, nh, splits, hd)), dtype=torch.float32, device=d)
        kernels.attention_decode(out, q, cache, bt, bs, None, n_req, cu, cl, scale, window, nh, nkv, hd, splits, scratch, warps)
        # splits per request, for the device's slots or for a made-up number of them
        w2, slots = [(w[0], w[2][0]) for w in widths][int(r_w * len(widths))]
        if r_s < 0.3:
            slots = alt
        items = torch.empty((kernels.decode_items_capacity(n_req, nkv, group, slots), 4), dtype=torch.int32, device=d)
        kernels.decode_build_items(items, cl, None, n_req, window, nh, nkv, hd, slots)
        out2 = torch.zeros_like(q)
        scratch2 = torch.zeros(kernels.attention_decode_items_scratch_floats(items.shape[0], nh, hd), dtype=torch.float32, device=d)
        kernels.attention_decode_items(out2, q, cache, bt, bs, items, cu, cl, scale, window, nh, nkv, hd, w2, scratch2)
        tol = 2e-2 * max(ref.float().abs().max().item(), 1e-3)
        what = (seed, case, hd, nkv, group, bs, window, n_req, longest, splits, warps, w2, slots)
        assert (out.float() - ref.float()).abs().max().item() <= tol, what
        assert (out2.float() - ref.float()).abs().max().item() <= tol, what


@pytest.mark.parametrize("seed", [1, 2])
def test_weight_streaming_product_on_random_shapes(seed):
    from lmsf_b200 import kernels
    rng = random.Random(seed)
    torch.manual_seed(seed)
    d = dev()
    for case in range(600 * SOAK):
        M = rng.randint(1, 16)
        K = 8 * rng.randint(1, 700)
        fuse = rng.choice([None, None, "silu", "gelu_tanh"])
        n_out = rng.choice([rng.randint(1, 40), rng.randint(1, 3000), 16 * rng.randint(1, 400)])
        N = 2 * n_out if fuse else n_out
        f32 = rng.random() < 0.3
        x = (torch.randn(M, K, device=d) * 0.5).to(torch.bfloat16)
        w = (torch.randn(N, K, device=d) / math.sqrt(K)).to(torch.bfloat16)
        out = torch.full((M, n_out), float("nan"), device=d, dtype=torch.float32 if f32 else torch.bfloat16)
        kernels.gemm_skinny(out, x, w, fuse_act=fuse)
        y = x.double() @ w.double().t()
        if fuse:
            g, u = y[:, :n_out], y[:, n_out:]
            act = g / (1 + torch.exp(-g)) if fuse == "silu" else 0.5 * g * (1 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))
            y = act * u
        err = (out.double() - y).abs().max().item()
        assert err <= (2e-3 if f32 else 2e-2) * max(y.abs().max().item(), 1e-2), (seed, case, M, N, K, fuse, f32, err)
        if case % 3:
            continue
        # the norm split between two products: the residual form of this one (plain cases), then the same weights
        # again, transposed in role, as the product of the prenormed input
        if fuse is None:
            eps = 10.0 ** -rng.randint(5, 6)
            res0 = torch.randn(M, N, device=d) * 2
            nw = (1 + 0.3 * torch.randn(N, device=d)).to(torch.float32 if rng.random() < 0.5 else torch.bfloat16)
            parts = kernels.gemm_skinny_residual_parts(N)
            sumsq = torch.full((M, (parts + 3) // 4 * 4), float("nan"), device=d)[:, :parts]
            res, xg = res0.clone(), torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=d)
            kernels.gemm_skinny_residual(xg, x, w, res, nw, sumsq)
            delta = torch.empty(M, N, dtype=torch.bfloat16, device=d)
            kernels.gemm_skinny(delta, x, w)
            want_res = res0 + delta.float()
            what = (seed, case, M, N, K, "residual form")
            assert torch.equal(res, want_res), what
            r64 = want_res.double()
            assert torch.allclose(sumsq.double().sum(1), (r64 * r64).sum(1), rtol=1e-5), what
            assert (xg.double() - r64 * nw.double()).abs().max().item() <= 8e-3 * (r64 * nw.double()).abs().max().item(), what
            if N % 8 == 0:
                normed = r64 / torch.sqrt((r64 * r64).mean(1, keepdim=True) + eps) * nw.double()
                n2 = rng.choice([rng.randint(1, 40), 16 * rng.randint(1, 60)])
                act = rng.choice([None, "silu"])
                w2 = (torch.randn((2 if act else 1) * n2, N, device=d) / math.sqrt(N)).to(torch.bfloat16)
                y2 = normed @ w2.double().t()
                if act:
                    y2 = y2[:, :n2] / (1 + torch.exp(-y2[:, :n2])) * y2[:, n2:]
                out2 = torch.full((M, n2), float("nan"), dtype=torch.float32, device=d)
                kernels.gemm_skinny(out2, xg, w2, fuse_act=act, prenorm=(sumsq, eps, N))
                err = (out2.double() - y2).abs().max().item()
                assert err <= 2e-2 * max(y2.abs().max().item(), 1e-2), (seed, case, M, N, K, n2, act, "prenormed input", err)
