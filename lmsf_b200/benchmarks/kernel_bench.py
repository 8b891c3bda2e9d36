"""Times one kernel of the package alone, at a model's sizes, and reports it against the roofline.

    python -m lmsf_b200.benchmarks.kernel_bench --kernel decode_attention --batch 8 --ctx 2048
    python -m lmsf_b200.benchmarks.kernel_bench --kernel all

Timing: CUDA events around `--iters` launches after `--warmup` launches; between launches a buffer larger
than L2 is read, so every launch starts with an L2 that holds none of its data (and no dirty lines).  Peaks come from MEASURED_PEAKS.json at the
repository root when it exists.  Defaults are Llama-3-8B's layer sizes.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        with open(p) as f:
            return json.load(f)
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


class Timer:
    def __init__(self, device, flush=True):
        self.flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device) if flush else None

    def run(self, fn, warmup, iters):
        for _ in range(warmup):
            fn()
        times = []
        for _ in range(iters):
            if self.flush_buf is not None:
                self.flush_buf.max()           # a READ of 256 MB: L2 ends up full of clean lines of another buffer
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e-3)
        return statistics.median(times)


def reference_kernels():
    """The reference's own CUDA kernels (baseline/ref_kernels.py, built unmodified for sm_100a), or None where they
    are not available: the pairs below then carry no `ref_us`."""
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    try:
        from baseline import ref_kernels
        ref_kernels.lib()
        return ref_kernels
    except Exception:
        return None


def paged(args, dev, batch, ctx):
    """A cache of `batch` requests of `ctx` keys in scattered pages, and one query token each."""
    bs, nkv, hd = args.block_size, args.kv_heads, args.head_dim
    blocks = (ctx + bs - 1) // bs
    n_pages = batch * blocks
    cache = torch.randn(n_pages, 2, nkv, bs, hd, device=dev, dtype=torch.bfloat16)
    perm = torch.randperm(n_pages, device=dev, dtype=torch.int32).view(batch, blocks).contiguous()
    return cache, perm


def bench_decode_attention(args, dev, timer, pk):
    from lmsf_b200 import kernels
    B, ctx, nh, nkv, hd = args.batch, args.ctx, args.heads, args.kv_heads, args.head_dim
    cache, bt = paged(args, dev, B, ctx)
    q = torch.randn(B, nh * hd, device=dev, dtype=torch.bfloat16)
    out = torch.empty_like(q)
    cu = torch.arange(B + 1, dtype=torch.int32, device=dev)
    cl = torch.full((B,), ctx, dtype=torch.int32, device=dev)
    sm = torch.cuda.get_device_properties(dev).multi_processor_count
    splits, warps = kernels.decode_plan(B, nkv, nh // nkv, ctx, hd, kernels.decode_widths(hd, nh // nkv))
    if args.splits:
        splits = args.splits
    if args.warps:
        warps = args.warps
    scratch = torch.zeros(max(1, kernels.attention_decode_scratch_floats(B, nh, splits, hd)), dtype=torch.float32, device=dev)
    fn = lambda: kernels.attention_decode(out, q, cache, bt, args.block_size, None, B, cu, cl, 1 / math.sqrt(hd), 0,
                                          nh, nkv, hd, splits, scratch, warps)
    t = timer.run(fn, args.warmup, args.iters)
    nbytes = B * ctx * 2 * nkv * hd * 2
    res = dict(kernel="decode_attention", batch=B, ctx=ctx, splits=splits, warps=warps, us=t * 1e6, gbs=nbytes / t / 1e9,
               frac_hbm=nbytes / t / 1e9 / pk["hbm_gbs"])
    rk = reference_kernels()
    if rk is not None and hd in (64, 80, 96, 112, 128, 256) and args.block_size in (8, 16, 32):
        # the reference's paged_attention, v1 or v2 by its own rule, on the same keys in its own layout
        x = 8
        P, bs = cache.shape[0], args.block_size
        kc = cache[:, 0].reshape(P, nkv, bs, hd // x, x).permute(0, 1, 3, 2, 4).contiguous()
        vc = cache[:, 1].permute(0, 1, 3, 2).contiguous()
        o3, q3 = out.view(B, nh, hd), q.view(B, nh, hd)
        which = []
        parts = -(-ctx // rk.PARTITION_SIZE)
        ws = (torch.empty((B, nh, parts, hd), dtype=q.dtype, device=dev), torch.empty((B, nh, parts), device=dev),
              torch.empty((B, nh, parts), device=dev))
        rfn = lambda: which.append(rk.paged_attention(o3, q3, kc, vc, bt, cl, ctx, 1 / math.sqrt(hd), nkv, workspace=ws))
        res["ref_us"] = timer.run(rfn, args.warmup, args.iters) * 1e6
        res["ref_kernel"] = "paged_attention_" + which[-1]
    return res


def bench_prefill_attention(args, dev, timer, pk):
    from lmsf_b200 import kernels
    T, nh, nkv, hd = args.tokens, args.heads, args.kv_heads, args.head_dim
    cache, bt = paged(args, dev, 1, T)
    q = torch.randn(T, nh * hd, device=dev, dtype=torch.bfloat16)
    out = torch.empty_like(q)
    cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
    cl = torch.tensor([T], dtype=torch.int32, device=dev)
    n_tiles = (T + 63) // 64
    ts = torch.zeros(n_tiles, dtype=torch.int32, device=dev)
    tq = torch.arange(0, T, 64, dtype=torch.int32, device=dev).flip(0).contiguous()      # longest tiles first
    if args.tc:
        n_tiles = (T + 127) // 128
        ts = torch.zeros(n_tiles, dtype=torch.int32, device=dev)
        tq = torch.arange(0, T, 128, dtype=torch.int32, device=dev).flip(0).contiguous()     # longest tiles first
        fn = lambda: kernels.attention_prefill_tc(out, q, cache, bt, args.block_size, ts, tq, n_tiles, cu, cl,
                                                  1 / math.sqrt(hd), 0, nh, nkv, hd)
    else:
        fn = lambda: kernels.attention_prefill(out, q, cache, bt, args.block_size, ts, tq, n_tiles, cu, cl,
                                               1 / math.sqrt(hd), 0, nh, nkv, hd)
    t = timer.run(fn, args.warmup, args.iters)
    flops = 4 * nh * hd * T * T / 2
    return dict(kernel="prefill_attention_tcgen05" if args.tc else "prefill_attention", tokens=T, us=t * 1e6, tflops=flops / t / 1e12,
                frac_bf16=flops / t / 1e12 / pk["bf16_tflops"])


def bench_rmsnorm(args, dev, timer, pk):
    from lmsf_b200 import kernels
    n, H = args.tokens, args.hidden
    x = torch.randn(n, H, device=dev, dtype=torch.bfloat16)
    res = torch.randn(n, H, device=dev)
    w = torch.ones(H, device=dev, dtype=torch.bfloat16)
    h = torch.empty_like(x)
    t = timer.run(lambda: kernels.add_rmsnorm(h, x, res, w, 1e-5, 2), args.warmup, args.iters)
    nbytes = n * H * (2 + 4 + 4 + 2)
    out = dict(kernel="add_rmsnorm", tokens=n, us=t * 1e6, gbs=nbytes / t / 1e9, frac_hbm=nbytes / t / 1e9 / pk["hbm_gbs"])
    rk = reference_kernels()
    if rk is not None:                     # vllm_fused_add_rms_norm: residual in bfloat16, in place
        xr, rr = x.clone(), res.bfloat16()
        out["ref_us"] = timer.run(lambda: rk.fused_add_rms_norm(xr, rr, w, 1e-5), args.warmup, args.iters) * 1e6
    return out


def bench_gated_act(args, dev, timer, pk):
    from lmsf_b200 import kernels
    n, I = args.tokens, args.intermediate
    x = torch.randn(n, 2 * I, device=dev, dtype=torch.bfloat16)
    out = torch.empty(n, I, device=dev, dtype=torch.bfloat16)
    t = timer.run(lambda: kernels.gated_act(out, x, "silu"), args.warmup, args.iters)
    nbytes = n * I * 6
    res = dict(kernel="gated_act", tokens=n, us=t * 1e6, gbs=nbytes / t / 1e9, frac_hbm=nbytes / t / 1e9 / pk["hbm_gbs"])
    rk = reference_kernels()
    if rk is not None:
        res["ref_us"] = timer.run(lambda: rk.silu_and_mul(out, x), args.warmup, args.iters) * 1e6
    return res


def bench_rope_cache(args, dev, timer, pk):
    from lmsf_b200 import kernels
    n, nh, nkv, hd, bs = args.tokens, args.heads, args.kv_heads, args.head_dim, args.block_size
    qkv = torch.randn(n, (nh + 2 * nkv) * hd, device=dev, dtype=torch.bfloat16)
    blocks = (n + bs - 1) // bs
    cache = torch.zeros(blocks, 2, nkv, bs, hd, device=dev, dtype=torch.bfloat16)
    bt = torch.randperm(blocks, device=dev, dtype=torch.int32).view(1, blocks).contiguous()
    pos = torch.arange(n, dtype=torch.int32, device=dev)
    seq = torch.zeros(n, dtype=torch.int32, device=dev)
    inv = torch.tensor([500000.0 ** (-(2.0 * i) / hd) for i in range(hd // 2)], dtype=torch.float32, device=dev)
    fn = lambda: kernels.rope_cache_write(qkv[:, :nh * hd], qkv[:, nh * hd:(nh + nkv) * hd], qkv[:, (nh + nkv) * hd:], pos,
                                          seq, bt, bs, cache, inv, hd, True, nh, nkv, hd)
    t = timer.run(fn, args.warmup, args.iters)
    nbytes = n * hd * 2 * (2 * nh + 4 * nkv)          # q read+write, k and v read, k and v written to pages
    res = dict(kernel="rope_cache_write", tokens=n, us=t * 1e6, gbs=nbytes / t / 1e9, frac_hbm=nbytes / t / 1e9 / pk["hbm_gbs"])
    rk = reference_kernels()
    if rk is not None:                     # the reference's two kernels: rotary_embedding, then reshape_and_cache
        table = rk.cos_sin_cache(500000.0, hd, n, torch.bfloat16, dev, inv)
        kc, vc = rk.new_caches(blocks, nkv, hd, bs, torch.bfloat16, dev)
        pos64 = pos.long()
        slots = (bt[0].long()[pos64 // bs] * bs + pos64 % bs).contiguous()
        q_, k_, v_ = qkv[:, :nh * hd], qkv[:, nh * hd:(nh + nkv) * hd], qkv[:, (nh + nkv) * hd:]

        def rfn():
            rk.rotary_embedding(pos64, q_, k_, table, hd, nh, nkv, True)
            rk.reshape_and_cache(k_, v_, kc, vc, slots, nkv, hd, bs)
        res["ref_us"] = timer.run(rfn, args.warmup, args.iters) * 1e6
    return res


def bench_gemm(args, dev, timer, pk):
    from lmsf_b200.parts.linear import matmul_tn
    M, N, K = args.m, args.n, args.k
    x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
    t = timer.run(lambda: matmul_tn(x, w), args.warmup, args.iters)
    flops, nbytes = 2 * M * N * K, 2 * (M * K + N * K + M * N)
    return dict(kernel="gemm_bf16", m=M, n=N, k=K, us=t * 1e6, tflops=flops / t / 1e12, gbs=nbytes / t / 1e9,
                frac_bf16=flops / t / 1e12 / pk["bf16_tflops"], frac_hbm=nbytes / t / 1e9 / pk["hbm_gbs"])


def bench_gemm_skinny(args, dev, timer, pk):
    from lmsf_b200 import kernels
    M, N, K = args.m, args.n, args.k
    x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
    fuse = "silu" if args.fuse_act else None
    out = torch.empty(M, N // 2 if fuse else N, device=dev, dtype=torch.bfloat16)
    t = timer.run(lambda: kernels.gemm_skinny(out, x, w, fuse), args.warmup, args.iters)
    full = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    t_lib = timer.run(lambda: torch.mm(x, w.t(), out=full), args.warmup, args.iters)     # the library's plain product
    nbytes = 2 * (M * K + N * K + out.numel())
    return dict(kernel="gemm_skinny", m=M, n=N, k=K, fused_act=bool(fuse), us=t * 1e6, gbs=nbytes / t / 1e9,
                frac_hbm=nbytes / t / 1e9 / pk["hbm_gbs"], library_us=t_lib * 1e6)


def bench_sampling(args, dev, timer, pk):
    from lmsf_b200 import kernels
    rows, V = args.batch, args.vocab
    logits = torch.randn(rows, V, device=dev)
    out = torch.empty(rows, dtype=torch.int32, device=dev)
    temp = torch.full((rows,), 0.8, device=dev)
    seed = torch.arange(rows, dtype=torch.int64, device=dev)
    step = torch.zeros(rows, dtype=torch.int32, device=dev)
    t0 = timer.run(lambda: kernels.sample(out, logits), args.warmup, args.iters)
    t1 = timer.run(lambda: kernels.sample(out, logits, temp, seed, step), args.warmup, args.iters)
    nbytes = rows * V * 4
    return dict(kernel="sample", rows=rows, vocab=V, greedy_us=t0 * 1e6, temperature_us=t1 * 1e6,
                greedy_gbs=nbytes / t0 / 1e9, frac_hbm=nbytes / t0 / 1e9 / pk["hbm_gbs"])


def bench_sampling_filtered(args, dev, timer, pk):
    """Top-k 50 and top-p 0.9 over logits that are peaked like a trained model's (a few large values per row)."""
    from lmsf_b200 import kernels
    rows, V = args.batch, args.vocab
    logits = torch.randn(rows, V, device=dev)
    logits[:, :64] += torch.linspace(12.0, 4.0, 64, device=dev)
    out = torch.empty(rows, dtype=torch.int32, device=dev)
    temp = torch.full((rows,), 0.8, device=dev)
    seed = torch.arange(rows, dtype=torch.int64, device=dev)
    step = torch.zeros(rows, dtype=torch.int32, device=dev)
    top_k = torch.full((rows,), 50, dtype=torch.int32, device=dev)
    top_p = torch.full((rows,), 0.9, device=dev)
    min_p = torch.zeros(rows, device=dev)
    t = timer.run(lambda: kernels.sample_filtered(out, logits, temp, seed, step, top_k, top_p, min_p), args.warmup, args.iters)
    t_p = timer.run(lambda: kernels.sample_filtered(out, logits, temp, seed, step, None, top_p, None), args.warmup, args.iters)
    return dict(kernel="sample_filtered", rows=rows, vocab=V, top_k_top_p_us=t * 1e6, top_p_only_us=t_p * 1e6)


def bench_gemm_skinny_qkv(args, dev, timer, pk):
    """The merged q/k/v product of a decode step with the rotary encoding and the cache write in its epilogue."""
    from lmsf_b200 import kernels
    M, K, nh, nkv, hd, bs = args.m, args.hidden, args.heads, args.kv_heads, args.head_dim, args.block_size
    x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    w = torch.randn((nh + 2 * nkv) * hd, K, device=dev, dtype=torch.bfloat16) * 0.02
    q = torch.empty(M, nh * hd, device=dev, dtype=torch.bfloat16)
    cache = torch.zeros(M + 1, 2, nkv, bs, hd, device=dev, dtype=torch.bfloat16)
    bt = torch.arange(M, dtype=torch.int32, device=dev).view(M, 1)
    pos = torch.arange(M, dtype=torch.int32, device=dev) % bs
    seq = torch.arange(M, dtype=torch.int32, device=dev)
    inv = torch.tensor([500000.0 ** (-(2.0 * i) / hd) for i in range(hd // 2)], dtype=torch.float32, device=dev)
    flag = kernels.error_word(dev)
    fn = lambda: kernels.gemm_skinny_qkv_rope(q, x, w, pos, seq, bt, bs, cache, inv, hd, True, nh, nkv, hd, flag)
    t = timer.run(fn, args.warmup, args.iters)
    nbytes = 2 * (M * K + w.numel() + M * (nh + 2 * nkv) * hd)
    return dict(kernel="gemm_skinny_qkv_rope", m=M, n=w.shape[0], k=K, us=t * 1e6, gbs=nbytes / t / 1e9,
                frac_hbm=nbytes / t / 1e9 / pk["hbm_gbs"])


BENCHES = {"decode_attention": bench_decode_attention, "prefill_attention": bench_prefill_attention,
           "add_rmsnorm": bench_rmsnorm, "gated_act": bench_gated_act, "rope_cache_write": bench_rope_cache,
           "gemm": bench_gemm, "gemm_skinny": bench_gemm_skinny, "sampling": bench_sampling, "sampling_filtered": bench_sampling_filtered,
           "gemm_skinny_qkv": bench_gemm_skinny_qkv}


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--kernel", default="all", choices=["all", *BENCHES])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--intermediate", type=int, default=14336)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--warps", type=int, default=0, help="decode_attention: warps of a block, 2 or 4 (default: the plan's)")
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=28672)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--fuse-act", action="store_true", help="gemm_skinny: W = [gate; up], fused silu(gate) * up")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--tc", action="store_true", help="prefill_attention: the tcgen05 kernel instead of the mma.sync one")
    ap.add_argument("--skinny-defines", default="", help="comma-separated -D constants for gemm_skinny.cu")
    ap.add_argument("--kv-stages", type=int, default=0, help="pipeline depth of the attention kernels (default: the build's)")
    a = ap.parse_args()
    if a.skinny_defines:
        from lmsf_b200 import kernels
        kernels.SKINNY_DEFINES = tuple(a.skinny_defines.split(","))
    if a.kv_stages:
        from lmsf_b200 import kernels
        kernels.MMA_KV_STAGES = a.kv_stages
    dev = torch.device("cuda:0")
    pk = peaks()
    timer = Timer(dev, flush=not a.no_flush)
    names = list(BENCHES) if a.kernel == "all" else [a.kernel]
    with torch.inference_mode():
        for n in names:
            r = BENCHES[n](a, dev, timer, pk)
            print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in r.items()}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
