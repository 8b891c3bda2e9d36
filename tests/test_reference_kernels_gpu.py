"""This package's kernels against yinqiwen/lmsf's own CUDA kernels for the same operations.

The reference's kernel files are compiled unmodified for sm_100a (baseline/build_ref.py) and called through
their `extern "C"` launchers at sizes their dispatch takes (head sizes 64 and 128, pages of 16 keys).  Where the
two differ by design the bound says so: the reference rounds the residual sum and every rotary product to the
model's type, this package keeps them in float32 and rounds once; the reference's softmax divides by
(sum + 1e-6) (vllm/kernels/attention/attention_kernels.cu:309) and is built with --use_fast_math.
"""
import math
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


@pytest.fixture(scope="module")
def ref():
    from baseline import build_ref
    try:
        build_ref.ensure_built()
    except build_ref.ReferenceUnavailable as e:
        pytest.skip(f"the reference's kernels are not available: {e}")
    from baseline import ref_kernels
    return ref_kernels


DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
EPS_OF = {torch.float32: 2e-6, torch.bfloat16: 2.0 ** -7}      # a few units of rounding of the type


def rel_err(a, b):
    return float((a.double() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-30))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,hidden,eps", [(7, 4096, 1e-5), (33, 1000, 1e-6)])
def test_rms_norm_and_fused_add(ref, dtype, n, hidden, eps):
    from lmsf_b200 import kernels
    g = torch.Generator(device=DEV).manual_seed(n)
    x = torch.randn(n, hidden, device=DEV, generator=g).to(dtype)
    r = torch.randn(n, hidden, device=DEV, generator=g).to(dtype)
    w = (1.0 + 0.1 * torch.randn(hidden, device=DEV, generator=g)).to(dtype)
    want = torch.empty_like(x)
    ref.rms_norm(want, x, w, eps)
    got = torch.empty_like(x)
    kernels.add_rmsnorm(got, x, None, w, eps, 0)
    assert rel_err(got, want) <= 2 * EPS_OF[dtype]
    # residual add + norm
    x_ref, r_ref = x.clone(), r.clone()
    ref.fused_add_rms_norm(x_ref, r_ref, w, eps)
    res = r.float().clone()
    h = torch.empty_like(x)
    kernels.add_rmsnorm(h, x, res, w, eps, 2)
    assert rel_err(res, r_ref) <= EPS_OF[dtype]             # float32 sum here, rounded to the type there
    assert rel_err(h, x_ref) <= 3 * EPS_OF[dtype]


def ours_cache_to_ref(cache, ref_mod):
    """[pages, 2, kv_heads, slot, hd] -> ([pages, kv_heads, hd/x, slot, x], [pages, kv_heads, hd, slot])."""
    P, _, nkv, bs, hd = cache.shape
    x = 16 // cache.element_size()
    k = cache[:, 0].reshape(P, nkv, bs, hd // x, x).permute(0, 1, 3, 2, 4).contiguous()
    v = cache[:, 1].permute(0, 1, 3, 2).contiguous()
    return k, v


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,theta", [(8, 2, 128, 500000.0), (6, 6, 64, 10000.0)])
def test_rotary_and_cache_write(ref, dtype, nh, nkv, hd, theta):
    from lmsf_b200 import kernels
    bs, n_seq, max_pos = 16, 3, 600
    g = torch.Generator(device=DEV).manual_seed(nh)
    positions, token_seq, tables = [], [], []
    n_pages = 0
    lens = [37, 1, 130]
    starts = [400, 77, 0]
    max_blocks = -(-max_pos // bs)
    perm = torch.randperm(n_seq * max_blocks, generator=torch.Generator().manual_seed(1)).tolist()
    for s, (n, p0) in enumerate(zip(lens, starts)):
        positions += list(range(p0, p0 + n))
        token_seq += [s] * n
        tables.append(perm[s * max_blocks:(s + 1) * max_blocks])
    n_pages = n_seq * max_blocks
    T = len(positions)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV, generator=g).to(dtype)
    pos32 = torch.tensor(positions, dtype=torch.int32, device=DEV)
    tseq = torch.tensor(token_seq, dtype=torch.int32, device=DEV)
    bt = torch.tensor(tables, dtype=torch.int32, device=DEV)
    inv_freq = torch.tensor([theta ** (-(2.0 * i) / hd) for i in range(hd // 2)], dtype=torch.float32, device=DEV)

    # this package: one kernel rotates q in place and writes rotated k and v into the pages
    mine = qkv.clone()
    cache = torch.zeros(n_pages, 2, nkv, bs, hd, dtype=dtype, device=DEV)
    q, k, v = mine[:, :nh * hd], mine[:, nh * hd:(nh + nkv) * hd], mine[:, (nh + nkv) * hd:]
    kernels.rope_cache_write(q, k, v, pos32, tseq, bt, bs, cache, inv_freq, hd, True, nh, nkv, hd)

    # the reference: rotary_embedding in place on q and k, then reshape_and_cache by slot
    theirs = qkv.clone()
    tq, tk, tv = theirs[:, :nh * hd], theirs[:, nh * hd:(nh + nkv) * hd], theirs[:, (nh + nkv) * hd:]
    table = ref.cos_sin_cache(theta, hd, max_pos, dtype, DEV, inv_freq)
    ref.rotary_embedding(pos32.long(), tq, tk, table, hd, nh, nkv, True)
    kc, vc = ref.new_caches(n_pages, nkv, hd, bs, dtype, DEV)
    slots = torch.tensor([tables[s][p // bs] * bs + p % bs for s, p in zip(token_seq, positions)], dtype=torch.int64, device=DEV)
    ref.reshape_and_cache(tk, tv, kc, vc, slots, nkv, hd, bs)
    torch.cuda.synchronize()

    # float32: the same table values up to sincosf against torch's cos / sin at angles up to 600 rad;
    # bfloat16: the reference rounds cos, sin and each product to bfloat16
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert rel_err(q, tq) <= tol
    want_k, want_v = ours_cache_to_ref(cache, ref)
    assert rel_err(want_k, kc) <= tol
    assert torch.equal(want_v, vc)
    # pages that no token was written to stay zero in both
    assert float(want_k.abs().sum(dim=(1, 2, 3, 4)).eq(0).sum()) == float(kc.abs().sum(dim=(1, 2, 3, 4)).eq(0).sum())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,d", [(5, 14336), (40, 172)])
def test_silu_and_mul(ref, dtype, n, d):
    from lmsf_b200 import kernels
    g = torch.Generator(device=DEV).manual_seed(d)
    x = (2.0 * torch.randn(n, 2 * d, device=DEV, generator=g)).to(dtype)
    want = torch.empty(n, d, dtype=dtype, device=DEV)
    ref.silu_and_mul(want, x)
    got = torch.empty_like(want)
    kernels.gated_act(got, x, "silu")
    # bfloat16: the reference rounds silu(x) before the product
    assert rel_err(got, want) <= (1e-5 if dtype == torch.float32 else 2.0 ** -7)


def make_paged_case(dtype, n_seqs, nh, nkv, hd, ctx, bs=16, seed=0, sharp=False):
    g = torch.Generator(device=DEV).manual_seed(seed)
    max_blocks = -(-max(ctx) // bs)
    n_pages = n_seqs * max_blocks + 3
    cache = torch.randn(n_pages, 2, nkv, bs, hd, device=DEV, generator=g).to(dtype)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    bt = torch.tensor([perm[s * max_blocks:(s + 1) * max_blocks] for s in range(n_seqs)], dtype=torch.int32, device=DEV)
    q = torch.randn(n_seqs, nh * hd, device=DEV, generator=g).to(dtype)
    if sharp:
        # one far key per (request, kv head) dominates: a key that is skipped or read from a wrong page shows
        for s in range(n_seqs):
            for h in range(nkv):
                j = (7 * s + 13 * h + 5) % ctx[s]
                page, slot = int(bt[s, j // bs]), j % bs
                qh = q[s].view(nh, hd)[h * (nh // nkv)].float()
                cache[page, 0, h, slot] = (qh * (12.0 * math.sqrt(hd) / float(qh.norm()) ** 2)).to(dtype)   # score 12
    ctx_t = torch.tensor(ctx, dtype=torch.int32, device=DEV)
    return q, cache, bt, ctx_t


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd", [(8, 2, 128), (6, 6, 64)])
@pytest.mark.parametrize("which", ["v1", "v2"])
def test_paged_attention(ref, dtype, nh, nkv, hd, which):
    from lmsf_b200 import kernels
    ctx = [1, 17, 512, 513, 1300, 2048]
    n = len(ctx)
    for sharp in (False, True):
        q, cache, bt, ctx_t = make_paged_case(dtype, n, nh, nkv, hd, ctx, seed=3 + sharp, sharp=sharp)
        kc, vc = ours_cache_to_ref(cache, ref)
        want = torch.empty(n, nh, hd, dtype=dtype, device=DEV)
        used = ref.paged_attention(want, q.view(n, nh, hd), kc, vc, bt, ctx_t, max(ctx), 1.0 / math.sqrt(hd), nkv, force=which)
        assert used == which
        want = want.view(n, nh * hd)
        positions = (ctx_t - 1).contiguous()
        token_seq = torch.arange(n, dtype=torch.int32, device=DEV)
        got = torch.empty_like(q)
        kernels.attention_generic(got, q, cache, bt, 16, token_seq, positions, 1.0 / math.sqrt(hd), 0, nh, nkv, hd)
        tol = 1e-4 if dtype == torch.float32 else 2e-2      # --use_fast_math exponentials and the + 1e-6 there
        assert rel_err(got, want) <= tol, (sharp, "generic")
        if dtype == torch.bfloat16:
            cu_q = torch.arange(n + 1, dtype=torch.int32, device=DEV)
            for splits in (1, 4, 12):
                need = kernels.attention_decode_scratch_floats(n, nh, splits, hd)
                scratch = torch.zeros(max(need, 1), dtype=torch.float32, device=DEV)
                got2 = torch.empty_like(q)
                kernels.attention_decode(got2, q, cache, bt, 16, None, n, cu_q, ctx_t, 1.0 / math.sqrt(hd), 0, nh, nkv,
                                         hd, splits, scratch)
                assert rel_err(got2, want) <= tol, (sharp, splits)
    torch.cuda.synchronize()
