#!/usr/bin/env python3
"""Runs yinqiwen/lmsf's own CUDA kernels (built unmodified by baseline/build_ref.py) in float32 on small inputs
and writes their outputs to an .npz file.  It needs a GPU; the outputs are committed as
tests/golden/reference_kernels_f32.npz and tests/test_golden_reference_kernels.py compares the plain
implementation with them on the CPU.

    python tests/golden/make_reference_kernel_goldens.py OUT.npz
"""
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)
from golden_inputs import CASES, values  # noqa: E402

from baseline import ref_kernels as ref  # noqa: E402

DEV = "cuda:0"


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def main(out_path):
    out = {}
    c = CASES["rms"]
    x, r, w = (t(values(c["n"] * c["hidden"], 1).reshape(c["n"], -1)), t(values(c["n"] * c["hidden"], 2).reshape(c["n"], -1)),
               t(1.0 + values(c["hidden"], 3, 0.2)))
    y = torch.empty_like(x)
    ref.rms_norm(y, x, w, c["eps"])
    out["rms_norm"] = y.cpu().numpy()
    xi, ri = x.clone(), r.clone()
    ref.fused_add_rms_norm(xi, ri, w, c["eps"])
    out["fused_add_rms_norm_x"], out["fused_add_rms_norm_residual"] = xi.cpu().numpy(), ri.cpu().numpy()

    c = CASES["rope"]
    n, nh, nkv, hd = c["n"], c["heads"], c["kv_heads"], c["head"]
    q, k = t(values(n * nh * hd, 4).reshape(n, -1)), t(values(n * nkv * hd, 5).reshape(n, -1))
    table = ref.cos_sin_cache(c["theta"], hd, 1024, torch.float32, DEV)
    pos = torch.tensor(c["positions"], dtype=torch.int64, device=DEV)
    ref.rotary_embedding(pos, q, k, table, hd, nh, nkv, True)
    out["rotary_q"], out["rotary_k"] = q.cpu().numpy(), k.cpu().numpy()

    c = CASES["silu"]
    x = t(values(c["n"] * 2 * c["d"], 6, 4.0).reshape(c["n"], -1))
    y = torch.empty(c["n"], c["d"], device=DEV)
    ref.silu_and_mul(y, x)
    out["silu_and_mul"] = y.cpu().numpy()

    c = CASES["attn"]
    nh, nkv, hd, bs, ctx = c["heads"], c["kv_heads"], c["head"], c["block"], c["ctx"]
    n = len(ctx)
    max_blocks = -(-max(ctx) // bs)
    kc, vc = ref.new_caches(n * max_blocks, nkv, hd, bs, torch.float32, DEV)
    tables = []
    for s, L in enumerate(ctx):
        keys = t(values(L * nkv * hd, 10 + s).reshape(L, nkv * hd))
        vals = t(values(L * nkv * hd, 20 + s).reshape(L, nkv * hd))
        # pages in reverse order, written by the reference's own reshape_and_cache
        pages = [n * max_blocks - 1 - (s * max_blocks + b) for b in range(max_blocks)]
        tables.append(pages)
        slots = torch.tensor([pages[p // bs] * bs + p % bs for p in range(L)], dtype=torch.int64, device=DEV)
        ref.reshape_and_cache(keys, vals, kc, vc, slots, nkv, hd, bs)
    q = t(values(n * nh * hd, 30, 4.0).reshape(n, nh, hd))
    bt = torch.tensor(tables, dtype=torch.int32, device=DEV)
    cl = torch.tensor(ctx, dtype=torch.int32, device=DEV)
    for which in ("v1", "v2"):
        o = torch.empty_like(q)
        ref.paged_attention(o, q, kc, vc, bt, cl, max(ctx), 1.0 / math.sqrt(hd), nkv, force=which)
        out["paged_attention_" + which] = o.cpu().numpy()
    torch.cuda.synchronize()
    np.savez(out_path, **out)
    print("wrote", out_path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1])
