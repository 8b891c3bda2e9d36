"""Each CUDA kernel alone against a plain float32 PyTorch statement of the same operation, at sizes other
than the tiny models' (widths that are no power of two, head sizes in steps of 16, odd head counts)."""
import math

import numpy as np
import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev():
    return torch.device("cuda:0")


def tol(dtype):
    return dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,vocab", [(40, 50), (1000, 333), (4104, 17)])
def test_embedding(dtype, hidden, vocab):
    from lmsf_b200 import kernels
    g = torch.Generator().manual_seed(0)
    table = torch.randn(vocab, hidden, generator=g).to(DT[dtype]).to(dev())
    ids = torch.randint(0, vocab, (37,), generator=g, dtype=torch.int32).to(dev())
    out = torch.empty(37, hidden, dtype=DT[dtype], device=dev())
    flag = torch.zeros(1, dtype=torch.int32, device=dev())
    kernels.embedding(out, table, ids, flag)
    assert torch.equal(out, table[ids.long()]) and flag.item() == 0
    ids[5] = vocab                      # outside the table: zeros and a raised flag, no stray read
    kernels.embedding(out, table, ids, flag)
    assert flag.item() == 1 and torch.all(out[5] == 0) and torch.equal(out[6], table[ids[6].long()])


@pytest.mark.parametrize("dtype,wdtype", [("float32", "float32"), ("bfloat16", "bfloat16"), ("bfloat16", "float32")])
@pytest.mark.parametrize("hidden", [48, 1000, 5120, 11000])
def test_add_rmsnorm(dtype, wdtype, hidden):
    from lmsf_b200 import kernels
    g = torch.Generator().manual_seed(1)
    n, eps = 9, 3e-6
    x = (torch.randn(n, hidden, generator=g) * 3).to(DT[dtype])
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(DT[wdtype])
    res0 = torch.randn(n, hidden, generator=g)
    xd, wd = x.to(dev()), w.to(dev())
    # mode 0
    h = torch.empty_like(xd)
    kernels.add_rmsnorm(h, xd, None, wd, eps, 0)
    ref = P.rms_norm(x.float(), w.float(), eps)
    assert torch.allclose(h.float().cpu(), ref, **tol(DT[dtype]))
    # mode 1: the residual starts as x
    res = torch.empty(n, hidden, dtype=torch.float32, device=dev())
    kernels.add_rmsnorm(h, xd, res, wd, eps, 1)
    assert torch.equal(res.cpu(), x.float()) and torch.allclose(h.float().cpu(), ref, **tol(DT[dtype]))
    # mode 2: the sum is float32 and is what gets normalised
    res = res0.to(dev())
    kernels.add_rmsnorm(h, xd, res, wd, eps, 2)
    s = res0 + x.float()
    assert torch.equal(res.cpu(), s)
    assert torch.allclose(h.float().cpu(), P.rms_norm(s, w.float(), eps), **tol(DT[dtype]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d", [24, 172, 1000, 14336])
def test_gated_act(dtype, d):
    from lmsf_b200 import kernels
    g = torch.Generator().manual_seed(2)
    x = (torch.randn(7, 2 * d + 8, generator=g) * 2).to(DT[dtype]).to(dev())[:, :2 * d]   # a strided view
    out = torch.empty(7, d, dtype=DT[dtype], device=dev())
    kernels.gated_act(out, x, "silu")
    xf = x.float().cpu()
    ref = xf[:, :d] / (1 + torch.exp(-xf[:, :d])) * xf[:, d:]
    assert torch.allclose(out.float().cpu(), ref, **tol(DT[dtype]))
    kernels.gated_act(out, x, "gelu_tanh")
    ref = torch.nn.functional.gelu(xf[:, :d], approximate="tanh") * xf[:, d:]
    assert torch.allclose(out.float().cpu(), ref, **tol(DT[dtype]))
    with pytest.raises(kernels.KernelError):
        kernels.gated_act(out, x, "relu")


@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (3, 130, 67), (70, 65, 129), (129, 300, 1000)])
def test_gemm_simt_is_true_float32_and_row_independent(M, N, K):
    from lmsf_b200 import kernels
    g = torch.Generator().manual_seed(3)
    a, w = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g)
    out = torch.empty(M, N, device=dev())
    kernels.gemm_tn_simt(out, a.to(dev()), w.to(dev()))
    ref = (a.double() @ w.double().T)
    # float32 accumulation error grows like sqrt(K) ulps; TF32 would be off by ~1e-3 relative
    assert (out.cpu().double() - ref).abs().max() <= 2e-6 * math.sqrt(K) * ref.abs().max()
    one = torch.empty(1, N, device=dev())
    kernels.gemm_tn_simt(one, a[M - 1:].to(dev()), w.to(dev()))
    assert torch.equal(one[0], out[M - 1])              # a row does not depend on its batch
    # bfloat16 inputs, float32 output (the plain twin of the tensor-core products)
    ab, wb = a.bfloat16(), w.bfloat16()
    kernels.gemm_tn_simt(out, ab.to(dev()), wb.to(dev()))
    assert torch.allclose(out.cpu(), ab.float() @ wb.float().T, rtol=1e-4, atol=1e-4 * math.sqrt(K))


def _paged_setup(dtype, n_q_heads, n_kv_heads, hd, bs, ctx_lens, q_lens, seed, sharp=False, poison=False):
    """Random q and paged k, v for several requests; pages handed out in a scrambled order.  With `poison`,
    every slot that holds no key (the rest of a last page, spare pages) is NaN: a kernel must not let it in."""
    g = torch.Generator().manual_seed(seed)
    S = len(ctx_lens)
    n_pages = sum((c + bs - 1) // bs for c in ctx_lens) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    max_blocks = max((c + bs - 1) // bs for c in ctx_lens)
    bt = torch.full((S, max_blocks), -1, dtype=torch.int32)
    cache = torch.full((n_pages, 2, n_kv_heads, bs, hd), float('nan') if poison else 0.0)
    ks, vs = [], []
    for s, c in enumerate(ctx_lens):
        k, v = torch.randn(c, n_kv_heads, hd, generator=g), torch.randn(c, n_kv_heads, hd, generator=g)
        if sharp and c > 1:  # one far key stands out for the last queries: a lost key changes the result visibly
            k[1] *= 6.0
        k, v = k.to(DT[dtype]).float(), v.to(DT[dtype]).float()
        ks.append(k)
        vs.append(v)
        for i in range((c + bs - 1) // bs):
            page = perm.pop()
            bt[s, i] = page
            n = min(bs, c - i * bs)
            cache[page, 0, :, :n] = k[i * bs:i * bs + n].transpose(0, 1)
            cache[page, 1, :, :n] = v[i * bs:i * bs + n].transpose(0, 1)
    N = sum(q_lens)
    q = torch.randn(N, n_q_heads * hd, generator=g)
    if sharp:
        q = q * 2.0
    q = q.to(DT[dtype])
    token_seq = torch.repeat_interleave(torch.arange(S, dtype=torch.int32), torch.tensor(q_lens))
    positions = torch.cat([torch.arange(c - n, c, dtype=torch.int32) for c, n in zip(ctx_lens, q_lens)])
    return q, cache.to(DT[dtype]), bt, token_seq, positions, ks, vs


def _attention_reference(q, ks, vs, token_seq, positions, n_q_heads, n_kv_heads, hd, scale, window, softcap=0.0, slopes=None):
    out = torch.empty(q.shape[0], n_q_heads, hd, dtype=torch.float64)
    r = n_q_heads // n_kv_heads
    qf = q.double().reshape(-1, n_q_heads, hd)
    for t in range(q.shape[0]):
        s, p = int(token_seq[t]), int(positions[t])
        lo = max(0, p - window + 1) if window else 0
        for h in range(n_q_heads):
            k, v = ks[s][lo:p + 1, h // r].double(), vs[s][lo:p + 1, h // r].double()
            sc = (k @ qf[t, h]) * scale
            if softcap:
                sc = softcap * torch.tanh(sc / softcap)
            if slopes is not None:                        # a bias that grows with the distance to the query
                sc = sc + slopes[h] * (torch.arange(lo, p + 1, dtype=torch.float64) - p)
            w = torch.softmax(sc, dim=0)
            out[t, h] = w @ v
    return out.reshape(q.shape[0], -1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_constants_that_llama_leaves_at_their_defaults(dtype):
    """A cap on the attention scores (softcap * tanh(score / softcap)), a bias on them that grows with distance (both
    taken by the generic kernel) and a scale on the embeddings: parameters of the parts that another architecture
    would set."""
    from lmsf_b200 import kernels
    nh, nkv, hd, bs, cap = 4, 2, 64, 16, 7.5
    ctx_lens, q_lens = [90, 1, 40], [90, 1, 3]
    q, cache, bt, token_seq, positions, ks, vs = _paged_setup(dtype, nh, nkv, hd, bs, ctx_lens, q_lens, 6, sharp=True)
    out = torch.empty(q.shape, dtype=DT[dtype], device=dev())
    scale = 1.0 / math.sqrt(hd)
    kernels.attention_generic(out, q.to(dev()), cache.to(dev()), bt.to(dev()), bs, token_seq.to(dev()),
                              positions.to(dev()), scale, 0, nh, nkv, hd, softcap=cap)
    ref = _attention_reference(q.float(), ks, vs, token_seq, positions, nh, nkv, hd, scale, 0, softcap=cap)
    plain = _attention_reference(q.float(), ks, vs, token_seq, positions, nh, nkv, hd, scale, 0)
    tol_ = (1e-4 if dtype == "float32" else 2e-2) * ref.abs().max().item()
    assert (out.float().cpu().double() - ref).abs().max().item() <= tol_
    assert (plain - ref).abs().max().item() > 5 * tol_               # the cap matters on these scores
    # slope[head] * (key position - query position) on the scaled scores, with a window as well
    slopes = [0.5, 0.0625, 0.0, 1.25]
    for window in (0, 30):
        kernels.attention_generic(out, q.to(dev()), cache.to(dev()), bt.to(dev()), bs, token_seq.to(dev()), positions.to(dev()),
                                  scale, window, nh, nkv, hd, slopes=torch.tensor(slopes, device=dev()))
        ref = _attention_reference(q.float(), ks, vs, token_seq, positions, nh, nkv, hd, scale, window, slopes=slopes)
        plain = _attention_reference(q.float(), ks, vs, token_seq, positions, nh, nkv, hd, scale, window)
        tol_ = (1e-4 if dtype == "float32" else 2e-2) * ref.abs().max().item()
        assert (out.float().cpu().double() - ref).abs().max().item() <= tol_
        hs = slice(2 * hd, 3 * hd)                                    # the head with slope 0 is the plain one
        assert (plain[:, hs] - ref[:, hs]).abs().max().item() == 0 and (plain - ref).abs().max().item() > 5 * tol_
    with pytest.raises(kernels.KernelError):
        kernels.attention_generic(out, q.to(dev()), cache.to(dev()), bt.to(dev()), bs, token_seq.to(dev()), positions.to(dev()),
                                  scale, 0, nh, nkv, hd, slopes=torch.tensor(slopes[:3], device=dev()))
    g = torch.Generator().manual_seed(3)
    table = torch.randn(50, 72, generator=g).to(DT[dtype])
    ids = torch.tensor([3, 49, 0, 17], dtype=torch.int32)
    got = torch.empty(4, 72, dtype=DT[dtype], device=dev())
    flag = torch.zeros(1, dtype=torch.int32, device=dev())
    kernels.embedding(got, table.to(dev()), ids.to(dev()), flag, scale=8.5)
    want = (table[ids.long()].float() * 8.5).to(DT[dtype])
    assert torch.equal(got.cpu(), want) and flag.item() == 0
    kernels.embedding(got, table.to(dev()), torch.tensor([3, 50, 0, -1], dtype=torch.int32, device=dev()), flag, scale=8.5)
    assert flag.item() == 1 and got[1].abs().max().item() == 0 and got[3].abs().max().item() == 0
    assert torch.equal(got[0].cpu(), want[0])
    flag.zero_()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd,bs,window", [(6, 2, 16, 4, 0), (5, 5, 48, 8, 0), (8, 1, 80, 16, 0),
                                               (4, 2, 112, 32, 37), (2, 2, 256, 16, 0), (3, 1, 64, 16, 100)])
def test_attention_generic(dtype, nh, nkv, hd, bs, window):
    from lmsf_b200 import kernels
    ctx_lens, q_lens = [150, 1, 67, 300], [150, 1, 5, 1]          # a whole prompt, a first token, a portion, a decode
    q, cache, bt, token_seq, positions, ks, vs = _paged_setup(dtype, nh, nkv, hd, bs, ctx_lens, q_lens, 4, sharp=True)
    out = torch.empty(q.shape, dtype=DT[dtype], device=dev())
    scale = 1.0 / math.sqrt(hd)
    kernels.attention_generic(out, q.to(dev()), cache.to(dev()), bt.to(dev()), bs, token_seq.to(dev()),
                              positions.to(dev()), scale, window, nh, nkv, hd)
    ref = _attention_reference(q.float(), ks, vs, token_seq, positions, nh, nkv, hd, scale, window)
    err = (out.float().cpu().double() - ref).abs().max().item()
    # float32: scores reach |s| ~ 40 here, so their rounding (2^-24 |s| sqrt(hd)) shows in exp(s) as ~1e-4 relative
    assert err <= (1e-4 if dtype == "float32" else 2e-2) * ref.abs().max().item(), err


def test_attention_refuses_sizes_it_was_not_written_for():
    from lmsf_b200 import kernels
    d = dev()
    q = torch.zeros(1, 2 * 24, device=d)
    with pytest.raises((kernels.KernelError, ValueError)):
        kernels.attention_generic(torch.empty_like(q), q, torch.zeros(1, 2, 2, 4, 24, device=d),
                                  torch.zeros(1, 1, dtype=torch.int32, device=d), 4,
                                  torch.zeros(1, dtype=torch.int32, device=d), torch.zeros(1, dtype=torch.int32, device=d),
                                  1.0, 0, 2, 2, 24)
    q = torch.zeros(1, 272, device=d)
    with pytest.raises(kernels.KernelError):
        kernels.attention_generic(torch.empty_like(q), q, torch.zeros(1, 2, 1, 4, 272, device=d),
                                  torch.zeros(1, 1, dtype=torch.int32, device=d), 4,
                                  torch.zeros(1, dtype=torch.int32, device=d), torch.zeros(1, dtype=torch.int32, device=d),
                                  1.0, 0, 1, 1, 272)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd,rot,neox,bs", [(4, 2, 16, 16, True, 4), (5, 1, 48, 48, True, 8),
                                                  (3, 3, 64, 32, True, 16), (2, 1, 32, 32, False, 16)])
def test_rope_and_cache_write(dtype, nh, nkv, hd, rot, neox, bs):
    from lmsf_b200 import kernels
    g = torch.Generator().manual_seed(5)
    N, S, max_blocks = 11, 2, 80
    positions = torch.tensor([0, 1, 2, 3, 4, 5, 6, 300, 301, 302, 303], dtype=torch.int32)
    token_seq = torch.tensor([0] * 7 + [1] * 4, dtype=torch.int32)
    bt = torch.full((S, max_blocks), -1, dtype=torch.int32)
    pages = torch.randperm(50, generator=g).tolist()
    for t in range(N):
        s, b = int(token_seq[t]), int(positions[t]) // bs
        if bt[s, b] < 0:
            bt[s, b] = pages.pop()
    width = (nh + 2 * nkv) * hd
    qkv = torch.randn(N, width, generator=g).to(DT[dtype])
    inv = torch.tensor([10000.0 ** (-(2.0 * i) / rot) for i in range(rot // 2)], dtype=torch.float64)
    cache = torch.zeros(50, 2, nkv, bs, hd, dtype=DT[dtype], device=dev())
    qkv_d = qkv.to(dev()).clone()
    flag = torch.zeros(1, dtype=torch.int32, device=dev())
    kernels.rope_cache_write(qkv_d[:, :nh * hd], qkv_d[:, nh * hd:(nh + nkv) * hd], qkv_d[:, (nh + nkv) * hd:],
                             positions.to(dev()), token_seq.to(dev()), bt.to(dev()), bs, cache,
                             inv.float().to(dev()), rot, neox, nh, nkv, hd, flag)
    assert flag.item() == 0

    def rotate(x, heads):
        x = x.float().reshape(N, heads, hd)
        xr = x[..., :rot]
        if neox:
            y = P.rotary_neox(xr, positions, inv)
        else:                     # interleaved pairs (2i, 2i+1)
            ang = positions.float()[:, None] * inv.float()[None, :]
            c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
            a, b = xr[..., 0::2], xr[..., 1::2]
            y = torch.stack([a * c - b * s, b * c + a * s], dim=-1).reshape(N, heads, rot)
        return torch.cat([y, x[..., rot:]], dim=-1)

    q_ref, k_ref = rotate(qkv[:, :nh * hd], nh), rotate(qkv[:, nh * hd:(nh + nkv) * hd], nkv)
    v_ref = qkv[:, (nh + nkv) * hd:].float().reshape(N, nkv, hd)
    t_ = tol(DT[dtype])
    assert torch.allclose(qkv_d[:, :nh * hd].float().cpu().reshape(N, nh, hd), q_ref, **t_)
    c = cache.float().cpu()
    for t in range(N):
        page, slot = int(bt[int(token_seq[t]), int(positions[t]) // bs]), int(positions[t]) % bs
        assert torch.allclose(c[page, 0, :, slot], k_ref[t], **t_)
        assert torch.equal(c[page, 1, :, slot], v_ref[t])
    used = {int(b) for b in bt.flatten() if b >= 0}
    for p in range(50):
        if p not in used:
            assert torch.all(c[p] == 0)                 # nothing is written anywhere else
    # a token without a page raises the flag and writes nothing
    bt2 = bt.clone()
    bt2[1, 300 // bs] = -1
    kernels.rope_cache_write(qkv_d[:, :nh * hd], qkv_d[:, nh * hd:(nh + nkv) * hd], qkv_d[:, (nh + nkv) * hd:],
                             positions.to(dev()), token_seq.to(dev()), bt2.to(dev()), bs, cache,
                             inv.float().to(dev()), rot, neox, nh, nkv, hd, flag)
    assert flag.item() == 2


def test_sampling_greedy_and_temperature():
    from lmsf_b200 import kernels
    g = torch.Generator().manual_seed(6)
    for vocab in (7, 320, 50001):
        rows = 6
        logits = torch.randn(rows, vocab, generator=g) * 3
        logits[0, 3] = logits[0, 5] = 50.0                       # a tie: the lowest index wins
        d = logits.to(dev())
        out = torch.empty(rows, dtype=torch.int32, device=dev())
        kernels.sample(out, d)
        assert out.tolist() == [3] + [int(logits[r].argmax()) for r in range(1, rows)]
        temp = torch.tensor([0.0, 0.8, 0.8, 1.5, 0.3, 0.8], device=dev())
        seeds = [0, 1, 1, 2 ** 63 + 5, 77, 1]
        steps = [0, 0, 1, 9, 3, 0]
        seed_t = torch.from_numpy(np.asarray(seeds, dtype=np.uint64).view(np.int64)).to(dev())
        kernels.sample(out, d, temp, seed_t, torch.tensor(steps, dtype=torch.int32, device=dev()))
        got = out.tolist()
        assert got[0] == 3
        for r in range(1, rows):
            assert got[r] == P.sample_temperature(logits[r], float(temp[r]), seeds[r], steps[r]), (vocab, r)


@pytest.mark.parametrize("nh,nkv,hd,bs,window", [(8, 2, 128, 16, 0), (6, 2, 16, 8, 0), (5, 5, 48, 16, 0), (3, 1, 80, 32, 0),
                                               (20, 1, 64, 16, 0), (4, 2, 112, 16, 70), (4, 4, 96, 4, 200)])
@pytest.mark.parametrize("warps", [4, 2])
def test_attention_tensor_core_kernels(nh, nkv, hd, bs, window, warps, monkeypatch):
    """Decode (split over the keys, every split count; blocks of four warps and of two) and prefill (tiles of 64
    queries) against float64."""
    from lmsf_b200 import kernels
    monkeypatch.setenv("LMSF_DECODE_WARPS", str(warps))
    assert kernels.mma_attention_supported(torch.bfloat16, hd)
    # a long decode, a first token, a portion in the middle of a prompt, a whole prompt, a 2-token portion, a decode
    ctx_lens, q_lens = [1500, 1, 700, 130, 65, 64], [1, 1, 201, 130, 2, 1]
    q, cache, bt, token_seq, positions, ks, vs = _paged_setup("bfloat16", nh, nkv, hd, bs, ctx_lens, q_lens, 9, sharp=True)
    scale = 1.0 / math.sqrt(hd)
    ref = _attention_reference(q.float(), ks, vs, token_seq, positions, nh, nkv, hd, scale, window)
    d = dev()
    qd, cd, btd = q.to(d), cache.to(d), bt.to(d)
    cu = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32, device=d)
    cl = torch.tensor(ctx_lens, dtype=torch.int32, device=d)
    dec = [i for i, n in enumerate(q_lens) if n == 1]
    tiles = [(i, q0) for i, n in enumerate(q_lens) if n > 1 for q0 in range(0, n, 64)]
    tol_abs = 2e-2 * ref.abs().max().item()
    for splits in (1, 2, 5, 24):
        out = torch.zeros(q.shape, dtype=torch.bfloat16, device=d)
        scratch = torch.zeros(max(1, kernels.attention_decode_scratch_floats(len(q_lens), nh, splits, hd)),
                              dtype=torch.float32, device=d)
        kernels.attention_decode(out, qd, cd, btd, bs, torch.tensor(dec, dtype=torch.int32, device=d), len(dec), cu, cl,
                                 scale, window, nh, nkv, hd, splits, scratch)
        kernels.attention_prefill(out, qd, cd, btd, bs, torch.tensor([t[0] for t in tiles], dtype=torch.int32, device=d),
                                  torch.tensor([t[1] for t in tiles], dtype=torch.int32, device=d), len(tiles), cu, cl,
                                  scale, window, nh, nkv, hd)
        err = (out.float().cpu().double() - ref).abs()
        assert err.max().item() <= tol_abs, (splits, err.max().item(), int(err.argmax()) // (nh * hd))
    # the generic kernel is their plain twin: same inputs, same answer within bfloat16 rounding
    out2 = torch.empty_like(out)
    kernels.attention_generic(out2, qd, cd, btd, bs, token_seq.to(d), positions.to(d), scale, window, nh, nkv, hd)
    assert (out2.float() - out.float()).abs().max().item() <= tol_abs


@pytest.mark.parametrize("max_blocks", [2, 0])
def test_attention_tcgen05_runs_of_short_units(max_blocks, monkeypatch):
    """Many short prompts beside a long one: a block takes long runs of units of a single key tile, in which an
    item's queries are free again before its softmax warps have finished the unit before (the hand-over of the
    next unit's queries must wait for both), mixed with units of many tiles."""
    from lmsf_b200 import kernels
    nh, nkv, hd, bs = 8, 2, 128, 16
    if max_blocks:
        monkeypatch.setenv("LMSF_TC_MAX_BLOCKS", str(max_blocks))
    q_lens = [100] * 30 + [900] + [64] * 20 + [129] * 6
    ctx_lens = list(q_lens)
    ctx_lens[30] = 1300
    q, cache, bt, token_seq, positions, ks, vs = _paged_setup("bfloat16", nh, nkv, hd, bs, ctx_lens, q_lens, 21, sharp=True,
                                                              poison=True)
    scale = 1.0 / math.sqrt(hd)
    ref = _attention_reference(q.float(), ks, vs, token_seq, positions, nh, nkv, hd, scale, 0)
    d = dev()
    qd, cd, btd = q.to(d), cache.to(d), bt.to(d)
    cu = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32, device=d)
    cl = torch.tensor(ctx_lens, dtype=torch.int32, device=d)
    tiles = [(i, q0) for i, n in enumerate(q_lens) for q0 in range(0, n, 128)]
    flag = torch.zeros(1, dtype=torch.int32, device=d)
    for _ in range(3):
        out = torch.zeros(q.shape, dtype=torch.bfloat16, device=d)
        kernels.attention_prefill_tc(out, qd, cd, btd, bs, torch.tensor([t[0] for t in tiles], dtype=torch.int32, device=d),
                                     torch.tensor([t[1] for t in tiles], dtype=torch.int32, device=d), len(tiles), cu, cl,
                                     scale, 0, nh, nkv, hd, flag)
        assert flag.item() == 0
        err = (out.float().cpu().double() - ref).abs()
        assert err.max().item() <= 2e-2 * ref.abs().max().item(), (err.max().item(), int(err.argmax()) // (nh * hd))


@pytest.mark.parametrize("nh,nkv,hd,warps", [(8, 2, 128, 4), (8, 2, 128, 2), (6, 2, 64, 4), (5, 5, 48, 4), (20, 1, 96, 2)])
def test_attention_decode_with_splits_per_request(nh, nkv, hd, warps):
    """Decode attention over a list of work items: requests of 1 to 3,000 keys side by side, each split by its own
    length; the list for few and for many slots (one split each; up to 64 splits for the longest), with a prompt
    portion in the batch (the list names only the requests that decode).  Against float64, and the list itself."""
    from lmsf_b200 import kernels
    bs = 16
    ctx_lens, q_lens = [3000, 40, 1, 700, 300, 65, 64, 130, 17, 2048], [1, 1, 1, 1, 37, 1, 1, 1, 1, 1]
    q, cache, bt, token_seq, positions, ks, vs = _paged_setup("bfloat16", nh, nkv, hd, bs, ctx_lens, q_lens, 33, sharp=True,
                                                              poison=True)
    scale = 1.0 / math.sqrt(hd)
    ref = _attention_reference(q.float(), ks, vs, token_seq, positions, nh, nkv, hd, scale, 0)
    d = dev()
    qd, cd, btd = q.to(d), cache.to(d), bt.to(d)
    cu = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32, device=d)
    cl = torch.tensor(ctx_lens, dtype=torch.int32, device=d)
    dec = [i for i, n in enumerate(q_lens) if n == 1]
    dec_ids = torch.tensor(dec, dtype=torch.int32, device=d)
    rows = [int(cu[i]) for i in dec]
    group = nh // nkv
    per_split = nkv * ((group + 15) // 16)
    tol_abs = 2e-2 * ref.abs().max().item()
    for slots in (1, 9 * per_split, 40 * per_split, 592, 100000):
        capacity = kernels.decode_items_capacity(len(dec), nkv, group, slots)
        items = torch.full((capacity, 4), -7, dtype=torch.int32, device=d)
        kernels.decode_build_items(items, cl, dec_ids, len(dec), 0, nh, nkv, hd, slots)
        it = items.cpu().tolist()
        real = [e for e in it if e[0] >= 0]
        assert all(e == [-1, 0, 0, 0] for e in it[len(real):])
        assert len(real) <= len(dec) + slots // per_split      # pieces of about an even share of the keys, at least one a request
        k = 0
        for i in dec:                                          # every request: its splits in order, one after the other
            s_i = real[k][2]
            assert 1 <= s_i <= 64 and (s_i == 1 or ctx_lens[i] / s_i > 64)
            assert [e[:4] for e in real[k:k + s_i]] == [[i, j, s_i, k] for j in range(s_i)]
            k += s_i
        assert k == len(real)
        if slots == 1:
            assert len(real) == len(dec)
        if slots == 100000:
            assert real[0][2] == (3000 + 64) // 128            # the longest: pieces of 128 keys
        scratch = torch.zeros(kernels.attention_decode_items_scratch_floats(capacity, nh, hd), dtype=torch.float32, device=d)
        for _ in range(2):                                     # twice: the counters are left as they were found
            out = torch.zeros(q.shape, dtype=torch.bfloat16, device=d)
            kernels.attention_decode_items(out, qd, cd, btd, bs, items, cu, cl, scale, 0, nh, nkv, hd, warps, scratch)
            err = (out.float().cpu().double()[rows] - ref[rows]).abs()
            assert err.max().item() <= tol_abs, (slots, err.max().item(), int(err.argmax()) // (nh * hd))


def test_decode_attention_of_a_large_group_after_a_query_for_a_small_one():
    """A block's shared memory grows with the query heads it holds.  A launch for 17 heads per kv head, then the
    question how many blocks of a small group fit (which sets the kernel up for less), then the large group again:
    what the kernel is allowed is only ever raised."""
    from lmsf_b200 import kernels
    hd, nkv, bs, n_req, ctx_n = 64, 2, 16, 5, 300
    d = dev()
    pages = (ctx_n + bs - 1) // bs
    cache = torch.randn(n_req * pages, 2, nkv, bs, hd, device=d).to(torch.bfloat16)
    bt = torch.arange(n_req * pages, dtype=torch.int32, device=d).view(n_req, pages).contiguous()
    cu = torch.arange(n_req + 1, dtype=torch.int32, device=d)
    cl = torch.full((n_req,), ctx_n, dtype=torch.int32, device=d)
    token_seq = torch.arange(n_req, dtype=torch.int32, device=d)
    positions = (cl - 1).to(torch.int32)
    def run(group):
        nh = nkv * group
        q = torch.randn(n_req, nh * hd, device=d).to(torch.bfloat16)
        out, ref = torch.zeros_like(q), torch.zeros_like(q)
        scratch = torch.zeros(kernels.attention_decode_scratch_floats(n_req, nh, 2, hd), dtype=torch.float32, device=d)
        kernels.attention_decode(out, q, cache, bt, bs, None, n_req, cu, cl, 0.125, 0, nh, nkv, hd, 2, scratch, 4)
        kernels.attention_generic(ref, q, cache, bt, bs, token_seq, positions, 0.125, 0, nh, nkv, hd)
        assert (out.float() - ref.float()).abs().max().item() <= 2e-2 * ref.float().abs().max().item()
    run(17)
    kernels._DECODE_WIDTHS.pop((hd, 1), None)
    kernels.decode_widths(hd, 1)
    run(1)
    run(17)


def test_sampling_filters_and_penalties():
    from lmsf_b200 import kernels
    g = torch.Generator().manual_seed(7)
    d = dev()
    for vocab in (50, 1000, 32003):
        rows = 8
        logits = torch.randn(rows, vocab, generator=g) * 2.5
        temps = [0.7, 1.0, 0.9, 1.3, 0.8, 0.5, 1.0, 2.0]
        ks = [5, -1, 40, 1, -1, 3, vocab + 5, -1]
        ps = [1.0, 0.9, 0.5, 1.0, 0.2, 0.8, 1.0, 0.95]
        mps = [0.0, 0.0, 0.0, 0.0, 0.05, 0.1, 0.3, 0.0]
        seeds = [3, 4, 5, 6, 7, 8, 9, 2 ** 40 + 1]
        ld = logits.to(d)
        seed_t = torch.from_numpy(np.asarray(seeds, dtype=np.uint64).view(np.int64)).to(d)
        for step in range(6):
            out = torch.full((rows,), -1, dtype=torch.int32, device=d)
            steps = torch.full((rows,), step, dtype=torch.int32, device=d)
            kernels.sample_filtered(out, ld, torch.tensor(temps, device=d), seed_t, steps,
                                    torch.tensor(ks, dtype=torch.int32, device=d), torch.tensor(ps, device=d),
                                    torch.tensor(mps, device=d))
            got = out.tolist()
            for r in range(rows):
                want = P.sample_filtered(logits[r], temps[r], seeds[r], step, ks[r], ps[r], mps[r])
                assert got[r] == want, (vocab, step, r)
                kept = P.filter_logits(logits[r].double() / temps[r], ks[r], ps[r], mps[r])
                assert torch.isfinite(kept[got[r]])
        # only some rows, through row_ids: the others keep what they had
        out = torch.full((rows,), -7, dtype=torch.int32, device=d)
        kernels.sample_filtered(out, ld, torch.tensor(temps, device=d), seed_t,
                                torch.zeros(rows, dtype=torch.int32, device=d),
                                torch.tensor(ks, dtype=torch.int32, device=d), torch.tensor(ps, device=d),
                                torch.tensor(mps, device=d), torch.tensor([2, 5], dtype=torch.int32, device=d))
        got = out.tolist()
        assert [got[i] for i in (0, 1, 3, 4, 6, 7)] == [-7] * 6 and got[2] >= 0 and got[5] >= 0
    # penalties
    vocab = 300
    logits = torch.randn(2, vocab, generator=g) * 2
    prompt, output = [5, 9, 9, 200], [9, 17, 17, 17, 250]
    pres, freq, rep = 0.4, 0.3, 1.7
    want = P.apply_penalties(logits[1], prompt, output, pres, freq, rep)
    seen = sorted(set(prompt) | set(output))
    ld = logits.to(d).clone()
    kernels.apply_penalties(ld, torch.tensor([1] * len(seen), dtype=torch.int32, device=d),
                            torch.tensor(seen, dtype=torch.int32, device=d),
                            torch.tensor([output.count(t) for t in seen], dtype=torch.int32, device=d),
                            torch.tensor([0.0, pres], device=d), torch.tensor([0.0, freq], device=d),
                            torch.tensor([1.0, rep], device=d))
    assert torch.equal(ld[0].cpu(), logits[0]) and torch.allclose(ld[1].cpu(), want, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("M,N,K", [(1, 48, 64), (8, 4096, 4096), (5, 1000, 320), (16, 6144, 1024), (13, 28, 14336 // 7),
                                   (3, 16, 1976), (8, 2, 64), (7, 18, 72), (12, 16, 128)])    # gated: 8, 1, 9 and 8 pairs of rows
def test_gemm_skinny_against_its_plain_twin(M, N, K):
    from lmsf_b200 import kernels
    g = torch.Generator().manual_seed(11)
    d = dev()
    x = (torch.randn(M, K, generator=g)).bfloat16().to(d)
    w = (torch.randn(N, K, generator=g) * 0.1).bfloat16().to(d)
    ref = torch.empty(M, N, device=d)
    kernels.gemm_tn_simt(ref, x, w)                     # bfloat16 in, float32 FMA accumulation
    for odt in (torch.bfloat16, torch.float32):
        out = torch.empty(M, N, dtype=odt, device=d)
        kernels.gemm_skinny(out, x, w)
        tol_ = 1e-4 if odt == torch.float32 else 1e-2
        assert torch.allclose(out.float(), ref, rtol=tol_, atol=tol_ * ref.abs().max().item())
    if N % 2 == 0:                                      # gate rows first, up rows second
        out = torch.empty(M, N // 2, dtype=torch.bfloat16, device=d)
        kernels.gemm_skinny(out, x, w, fuse_act="silu")
        gte, up = ref[:, :N // 2], ref[:, N // 2:]
        want = gte / (1 + torch.exp(-gte)) * up
        assert torch.allclose(out.float(), want, rtol=1e-2, atol=1e-2 * want.abs().max().item())
    with pytest.raises(kernels.KernelError):
        kernels.gemm_skinny(torch.empty(17, N, dtype=torch.bfloat16, device=d),
                            torch.zeros(17, K, dtype=torch.bfloat16, device=d), w)


@pytest.mark.parametrize("M,N,K,N2", [(8, 4096, 512, 1024), (1, 48, 64, 32), (5, 1000, 320, 30), (16, 1032, 256, 512),
                                      (13, 5120, 128, 64), (3, 16, 1976, 18)])
@pytest.mark.parametrize("w_dtype", [torch.float32, torch.bfloat16])
def test_a_norm_split_between_the_products_around_it(M, N, K, N2, w_dtype):
    """The residual form (product, residual add, residual x norm weight, partial sums of squares) and a product that
    takes that as a prenormed input, plain and gated, and the finishing kernel, against float64; widths whose number
    of partial sums is no multiple of 4, of 8 or of 16 among them.  The residual itself is what the three separate
    steps give, bit for bit."""
    from lmsf_b200 import kernels
    g = torch.Generator().manual_seed(17)
    d = dev()
    eps = 1e-5
    x = torch.randn(M, K, generator=g).bfloat16().to(d)
    w = (torch.randn(N, K, generator=g) * 0.1).bfloat16().to(d)
    res0 = (torch.randn(M, N, generator=g) * 2).to(d)
    nw = (1 + 0.3 * torch.randn(N, generator=g)).to(w_dtype).to(d)
    w2 = (torch.randn(2 * N2, N, generator=g) * 0.05).bfloat16().to(d)
    parts = kernels.gemm_skinny_residual_parts(N)
    sumsq = torch.full((M, (parts + 3) // 4 * 4), float("nan"), device=d)[:, :parts]
    res = res0.clone()
    xg = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=d)
    kernels.gemm_skinny_residual(xg, x, w, res, nw, sumsq)
    # the three steps: product (bfloat16 out), add into the float32 residual, norm
    delta = torch.empty(M, N, dtype=torch.bfloat16, device=d)
    kernels.gemm_skinny(delta, x, w)
    res_ref = res0.clone()
    h_ref = torch.empty_like(delta)
    kernels.add_rmsnorm(h_ref, delta, res_ref, nw, eps, 2)
    assert torch.equal(res, res_ref)
    r64 = res_ref.double()
    assert torch.allclose(sumsq.double().sum(1), (r64 * r64).sum(1), rtol=1e-5)
    assert torch.allclose(xg.float().double(), r64 * nw.double(), rtol=1e-2, atol=1e-2)
    normed = r64 / torch.sqrt((r64 * r64).mean(1, keepdim=True) + eps) * nw.double()
    # the finishing kernel gives the norm's output
    h = torch.empty_like(xg)
    kernels.finish_rmsnorm(h, res, sumsq, nw, eps)
    assert torch.allclose(h.float().double(), normed, rtol=1e-2, atol=1e-2)
    assert (h.float() - h_ref.float()).abs().max().item() <= 2 ** -7 * h_ref.float().abs().max().item()
    # products of the prenormed input: plain (both output types) and gated
    want = normed @ w2.double().t()
    for odt in (torch.bfloat16, torch.float32):
        y = torch.full((M, 2 * N2), float("nan"), dtype=odt, device=d)
        kernels.gemm_skinny(y, xg, w2, prenorm=(sumsq, eps, N))
        assert (y.double() - want).abs().max().item() <= 1.5e-2 * want.abs().max().item()
    gte, up = want[:, :N2], want[:, N2:]
    y = torch.full((M, N2), float("nan"), dtype=torch.bfloat16, device=d)
    kernels.gemm_skinny(y, xg, w2, fuse_act="silu", prenorm=(sumsq, eps, N))
    want_g = gte / (1 + torch.exp(-gte)) * up
    assert (y.double() - want_g).abs().max().item() <= 2e-2 * want_g.abs().max().item()
    # as good as the unfused way: the same product of the ordinary norm's output
    y_ref = torch.empty(M, 2 * N2, dtype=torch.float32, device=d)
    kernels.gemm_skinny(y_ref, h_ref, w2)
    y_new = torch.empty_like(y_ref)
    kernels.gemm_skinny(y_new, xg, w2, prenorm=(sumsq, eps, N))
    e_ref, e_new = (y_ref.double() - want).abs().max().item(), (y_new.double() - want).abs().max().item()
    assert e_new <= 2 * e_ref + 1e-6 * want.abs().max().item(), (e_new, e_ref)


def test_attention_kernels_on_a_long_prompt_and_a_long_context():
    """6,000 tokens in one portion (47 key tiles per block: the rings of stages and the barriers' phases wrap many
    times) on both prefill kernels, and one decoded token over 16,000 keys in 1, 7 and 64 splits; a sample of rows
    is compared with float64."""
    from lmsf_b200 import kernels
    nh, nkv, hd, bs = 4, 2, 128, 16
    T = 6000
    q, cache, bt, token_seq, positions, ks, vs = _paged_setup("bfloat16", nh, nkv, hd, bs, [T, 16000], [T, 1], 21, sharp=True,
                                                              poison=True)
    scale = 1.0 / math.sqrt(hd)
    d = dev()
    qd, cd, btd = q.to(d), cache.to(d), bt.to(d)
    cu = torch.tensor([0, T, T + 1], dtype=torch.int32, device=d)
    cl = torch.tensor([T, 16000], dtype=torch.int32, device=d)
    rows = sorted(set([0, 1, 127, 128, 129, 2047, 4095, 4096, T - 2, T - 1, T] + list(range(3, T, 487))))
    sub = torch.tensor(rows)
    ref = _attention_reference(q.float()[sub], ks, vs, token_seq[sub], positions[sub], nh, nkv, hd, scale, 0)
    tol = 2e-2 * ref.abs().max().item()
    flag = torch.zeros(1, dtype=torch.int32, device=d)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=d)
    out_tc = torch.zeros(q.shape, dtype=torch.bfloat16, device=d)
    kernels.attention_prefill_tc(out_tc, qd, cd, btd, bs, i32([0] * ((T + 127) // 128)), i32(list(range(0, T, 128))),
                                 (T + 127) // 128, cu, cl, scale, 0, nh, nkv, hd, flag)
    assert flag.item() == 0
    out_mma = torch.zeros_like(out_tc)
    kernels.attention_prefill(out_mma, qd, cd, btd, bs, i32([0] * ((T + 63) // 64)), i32(list(range(0, T, 64))),
                              (T + 63) // 64, cu, cl, scale, 0, nh, nkv, hd)
    assert (out_tc[:T].float() - out_mma[:T].float()).abs().max().item() <= tol
    for splits in (1, 7, 64):
        out = out_tc.clone()
        scratch = torch.zeros(max(1, kernels.attention_decode_scratch_floats(2, nh, splits, hd)), dtype=torch.float32, device=d)
        kernels.attention_decode(out, qd, cd, btd, bs, i32([1]), 1, cu, cl, scale, 0, nh, nkv, hd, splits, scratch)
        err = (out.float().cpu().double()[sub] - ref).abs()
        assert err.max().item() <= tol, (splits, err.max().item(), rows[int(err.argmax()) // (nh * hd)])


@pytest.mark.parametrize("M,nh,nkv,hd,rot,neox,K", [(8, 4, 2, 128, 128, True, 512), (1, 3, 1, 64, 64, True, 200), (13, 2, 2, 64, 32, True, 96),
                                                    (5, 6, 3, 32, 32, False, 64), (16, 2, 1, 48, 24, False, 128), (7, 2, 2, 16, 0, True, 64)])
def test_fused_qkv_rotary_cache_write_equals_the_three_steps(M, nh, nkv, hd, rot, neox, K):
    """The q/k/v projection with rotation and cache write in its epilogue against the product, then the
    rotary / cache-write kernel: the same bits in q and in the pages."""
    from lmsf_b200 import kernels
    g = torch.Generator().manual_seed(31)
    d = dev()
    bs, n_pages, max_blocks = 8, 40, 6
    x = torch.randn(M, K, generator=g).bfloat16().to(d)
    w = (torch.randn((nh + 2 * nkv) * hd, K, generator=g) * 0.2).bfloat16().to(d)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, rot, 2).float() / rot))).to(d) if rot else None
    n_seqs = 3
    token_seq = torch.tensor([i % n_seqs for i in range(M)], dtype=torch.int32, device=d)
    # distinct positions per request; pages handed out at random
    positions = torch.tensor([(i // n_seqs) * 5 + (i % n_seqs) * 3 for i in range(M)], dtype=torch.int32, device=d)
    perm = torch.randperm(n_pages, generator=g).tolist()
    bt = torch.tensor([[perm.pop() for _ in range(max_blocks)] for _ in range(n_seqs)], dtype=torch.int32, device=d)
    q_size, kv_size = nh * hd, nkv * hd
    # the three steps
    qkv = torch.empty(M, q_size + 2 * kv_size, dtype=torch.bfloat16, device=d)
    kernels.gemm_skinny(qkv, x, w)
    cache_ref = torch.zeros(n_pages, 2, nkv, bs, hd, dtype=torch.bfloat16, device=d)
    flag = torch.zeros(1, dtype=torch.int32, device=d)
    q_ref = qkv[:, :q_size]
    kernels.rope_cache_write(q_ref, qkv[:, q_size:q_size + kv_size], qkv[:, q_size + kv_size:], positions, token_seq, bt, bs,
                             cache_ref, inv_freq, rot, neox, nh, nkv, hd, flag)
    # the one kernel
    cache = torch.zeros_like(cache_ref)
    q = torch.full((M, q_size), float("nan"), dtype=torch.bfloat16, device=d)
    kernels.gemm_skinny_qkv_rope(q, x, w, positions, token_seq, bt, bs, cache, inv_freq, rot, neox, nh, nkv, hd, flag)
    assert flag.item() == 0
    assert torch.equal(q.view(torch.int16), q_ref.contiguous().view(torch.int16))
    assert torch.equal(cache.view(torch.int16), cache_ref.view(torch.int16))
    # the same with a prenormed input: the factor of a row is applied before the sums are rounded
    sumsq = (torch.rand(M, 7, generator=g) * 50).to(d)
    sumsq_padded = torch.zeros(M, 8, device=d)
    sumsq_padded[:, :7] = sumsq
    pn = (sumsq_padded[:, :7], 1e-6, K)
    kernels.gemm_skinny(qkv, x, w, prenorm=pn)
    plain = torch.empty_like(qkv)
    kernels.gemm_skinny(plain, x, w)
    assert not torch.equal(plain, qkv)
    cache_ref.zero_()
    q_ref = qkv[:, :q_size]
    kernels.rope_cache_write(q_ref, qkv[:, q_size:q_size + kv_size], qkv[:, q_size + kv_size:], positions, token_seq, bt, bs,
                             cache_ref, inv_freq, rot, neox, nh, nkv, hd, flag)
    cache.zero_()
    kernels.gemm_skinny_qkv_rope(q, x, w, positions, token_seq, bt, bs, cache, inv_freq, rot, neox, nh, nkv, hd, flag, prenorm=pn)
    assert flag.item() == 0
    assert torch.equal(q.view(torch.int16), q_ref.contiguous().view(torch.int16))
    assert torch.equal(cache.view(torch.int16), cache_ref.view(torch.int16))
    # a token without a page raises the error word and writes nothing
    bt2 = bt.clone()
    bt2[int(token_seq[0]), int(positions[0]) // bs] = -1
    cache2 = torch.zeros_like(cache_ref)
    kernels.gemm_skinny_qkv_rope(q, x, w, positions, token_seq, bt2, bs, cache2, inv_freq, rot, neox, nh, nkv, hd, flag)
    assert flag.item() == 2
    flag.zero_()


@pytest.mark.parametrize("nh,nkv,hd,bs,window", [(8, 2, 128, 16, 0), (4, 4, 64, 16, 0), (6, 1, 128, 8, 0), (4, 2, 64, 32, 90),
                                               (2, 1, 128, 16, 300), (3, 1, 128, 4, 0), (6, 2, 64, 128, 0), (5, 1, 128, 256, 200),
                                               (2, 2, 64, 2, 70)])
@pytest.mark.parametrize("max_blocks", [0, 3])
def test_attention_tcgen05_prefill(nh, nkv, hd, bs, window, max_blocks, monkeypatch):
    """The tcgen05 prefill kernel against float64 and against its mma.sync twin: even and odd groups of heads,
    pages from 2 to 256 keys (tensor-map copies from 8 keys on, cp.async below), windows; slots that hold no key
    are NaN.  With three blocks only, every block takes many units of work in turn (with one and with two items,
    and empty ones), so the barriers' phases and the rings of stages run on from unit to unit."""
    from lmsf_b200 import kernels
    if max_blocks:
        monkeypatch.setenv("LMSF_TC_MAX_BLOCKS", str(max_blocks))
    assert kernels.tc_attention_supported(torch.bfloat16, hd)
    # a portion in the middle of a long prompt, a whole prompt, a 2-token portion, a portion of exactly one tile, a long one
    ctx_lens, q_lens = [700, 130, 65, 128, 1100], [201, 130, 2, 128, 1000]
    q, cache, bt, token_seq, positions, ks, vs = _paged_setup("bfloat16", nh, nkv, hd, bs, ctx_lens, q_lens, 13, sharp=True,
                                                              poison=True)
    scale = 1.0 / math.sqrt(hd)
    ref = _attention_reference(q.float(), ks, vs, token_seq, positions, nh, nkv, hd, scale, window)
    d = dev()
    qd, cd, btd = q.to(d), cache.to(d), bt.to(d)
    cu = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32, device=d)
    cl = torch.tensor(ctx_lens, dtype=torch.int32, device=d)
    tiles = [(i, q0) for i, n in enumerate(q_lens) for q0 in range(0, n, 128)]
    flag = torch.zeros(1, dtype=torch.int32, device=d)
    out = torch.zeros(q.shape, dtype=torch.bfloat16, device=d)
    kernels.attention_prefill_tc(out, qd, cd, btd, bs, torch.tensor([t[0] for t in tiles], dtype=torch.int32, device=d),
                                 torch.tensor([t[1] for t in tiles], dtype=torch.int32, device=d), len(tiles), cu, cl,
                                 scale, window, nh, nkv, hd, flag)
    assert flag.item() == 0
    err = (out.float().cpu().double() - ref).abs()
    assert err.max().item() <= 2e-2 * ref.abs().max().item(), (err.max().item(), int(err.argmax()) // (nh * hd))
    tiles64 = [(i, q0) for i, n in enumerate(q_lens) for q0 in range(0, n, 64)]
    out2 = torch.zeros_like(out)
    kernels.attention_prefill(out2, qd, cd, btd, bs, torch.tensor([t[0] for t in tiles64], dtype=torch.int32, device=d),
                              torch.tensor([t[1] for t in tiles64], dtype=torch.int32, device=d), len(tiles64), cu, cl,
                              scale, window, nh, nkv, hd)
    assert (out2.float() - out.float()).abs().max().item() <= 2e-2 * ref.abs().max().item()
