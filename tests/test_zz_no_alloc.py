"""The decode-attention entry point that allocates nothing (lmsf_attention_decode_static), called through
its exported C symbol as a program without torch's allocator would call it.  Such callers exist: a host
that gave all device memory to its own pool, a loop that must not stall on cudaMalloc's device-wide
synchronisation, a binding that has only the C ABI.  The test checks that the variant gives what the
ordinary entry point gives with caller-provided scratch, twice in a row with different inputs (the
static scratch keeps the first call's contents), and that it refuses what does not fit.

This file is collected last on purpose."""
import ctypes
import math
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbol(head_dim):
    from lmsf_b200.csrc.build import load_library
    lib = load_library("attention_mma.cu", (f"LMSF_HEAD_DIM={head_dim}",))
    f = lib.lmsf_attention_decode_static
    f.restype = c_int
    f.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_void_p, c_int,
                  c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_void_p]
    lib.lmsf_attention_decode_static_capacity.restype = c_longlong
    lib.lmsf_attention_mma_last_error.restype = ctypes.c_char_p
    return lib, f


def _case(nh, nkv, hd, bs, ctx_lens, seed):
    from test_kernels_gpu import _paged_setup
    q_lens = [1] * len(ctx_lens)
    q, cache, bt, _, _, _, _ = _paged_setup("bfloat16", nh, nkv, hd, bs, ctx_lens, q_lens, seed, sharp=True)
    d = torch.device("cuda:0")
    cu = torch.arange(len(ctx_lens) + 1, dtype=torch.int32, device=d)
    cl = torch.tensor(ctx_lens, dtype=torch.int32, device=d)
    return q.to(d), cache.to(d), bt.to(d), cu, cl


def test_static_scratch_variant_matches_the_ordinary_entry_point_twice_in_a_row():
    from lmsf_b200 import kernels
    nh, nkv, hd, bs = 8, 2, 64, 16
    lib, f = _symbol(hd)
    assert lib.lmsf_attention_decode_static_capacity() == 8 << 20
    stream = torch.cuda.current_stream().cuda_stream
    for ctx_lens, splits, seed in (([900, 65, 1, 400], 6, 1), ([130, 777, 300], 3, 2)):
        q, cache, bt, cu, cl = _case(nh, nkv, hd, bs, ctx_lens, seed)
        scale = 1.0 / math.sqrt(hd)
        want = torch.zeros_like(q)
        scratch = torch.zeros(kernels.attention_decode_scratch_floats(len(ctx_lens), nh, splits, hd),
                              dtype=torch.float32, device=q.device)
        kernels.attention_decode(want, q, cache, bt, bs, None, len(ctx_lens), cu, cl, scale, 0, nh, nkv, hd, splits, scratch)
        got = torch.zeros_like(q)
        rc = f(q.data_ptr(), q.stride(0), got.data_ptr(), got.stride(0), cache.data_ptr(), cache.stride(0), bs, nkv,
               bt.data_ptr(), bt.shape[1], None, len(ctx_lens), len(ctx_lens), cu.data_ptr(), cl.data_ptr(), scale, 0,
               nh, hd, splits, stream)
        assert rc == 0, lib.lmsf_attention_mma_last_error()
        torch.cuda.synchronize()
        assert torch.allclose(got.float(), want.float(), rtol=2e-2, atol=2e-2)
        assert torch.equal(got, want)          # the same kernels in the same order: not a bit may differ


def test_static_scratch_variant_refuses_what_does_not_fit():
    nh, nkv, hd, bs = 8, 2, 64, 16
    lib, f = _symbol(hd)
    q, cache, bt, cu, cl = _case(nh, nkv, hd, bs, [100, 50], 3)
    out = torch.zeros_like(q)
    # 2 requests would fit; claim 4096 rows of the table so that 4096 * 8 * 64 * 65 * 4 bytes > 8 MiB
    rc = f(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), cache.data_ptr(), cache.stride(0), bs, nkv,
           bt.data_ptr(), bt.shape[1], None, 2, 4096, cu.data_ptr(), cl.data_ptr(), 0.125, 0, nh, hd, 64,
           torch.cuda.current_stream().cuda_stream)
    assert rc == -1
    msg = lib.lmsf_attention_mma_last_error().decode()
    assert "static" in msg and "8388608" in msg
    torch.cuda.synchronize()
    assert torch.all(out == 0)                 # nothing ran
