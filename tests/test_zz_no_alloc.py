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
    """More than 8 key splits add their partial results up through the scratch (up to 8 meet in the shared memory
    of a thread-block cluster and never touch it), so the cases with 12, 24 and 16 splits are the ones in which
    the kernels really read and write the static array: a wrong device address, counters that a call did not
    leave at zero or partial results left over from the call before would change their output.  The calls differ
    in the number of requests, of heads and of splits, so each finds the array as another geometry left it; one
    call that stays inside a cluster (6 splits) runs in between."""
    from lmsf_b200 import kernels
    hd, bs = 64, 16
    lib, f = _symbol(hd)
    assert lib.lmsf_attention_decode_static_capacity() == 8 << 20
    stream = torch.cuda.current_stream().cuda_stream
    cases = ((8, 2, [900, 65, 1, 400], 12, 1), (4, 4, [130, 777, 300], 24, 2), (8, 2, [900, 65, 1, 400], 6, 3),
             (12, 3, [513, 2, 1030, 64, 257], 16, 4), (8, 2, [900, 65, 1, 400], 12, 1))
    for nh, nkv, ctx_lens, splits, seed in cases:
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
        assert torch.allclose(got.float(), want.float(), rtol=2e-2, atol=2e-2), (nh, splits)
        assert torch.equal(got, want), (nh, splits)     # the same kernels in the same order: not a bit may differ
        # and both agree with the plain twin that needs no scratch at all
        plain = torch.zeros_like(q)
        token_seq = torch.arange(len(ctx_lens), dtype=torch.int32, device=q.device)
        kernels.attention_generic(plain, q, cache, bt, bs, token_seq, (cl - 1).contiguous(), scale, 0, nh, nkv, hd)
        assert float((got.float() - plain.float()).abs().max()) <= 2e-2 * float(plain.float().abs().max()), (nh, splits)


def test_static_scratch_variant_refuses_more_served_requests_than_rows():
    """Without seq_ids the kernels index the scratch by the served request's number: more served requests than
    rows of the block table would run past what was sized."""
    nh, nkv, hd, bs = 8, 2, 64, 16
    lib, f = _symbol(hd)
    q, cache, bt, cu, cl = _case(nh, nkv, hd, bs, [100, 50], 3)
    out = torch.zeros_like(q)
    rc = f(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), cache.data_ptr(), cache.stride(0), bs, nkv,
           bt.data_ptr(), bt.shape[1], None, 2, 1, cu.data_ptr(), cl.data_ptr(), 0.125, 0, nh, hd, 12,
           torch.cuda.current_stream().cuda_stream)
    assert rc == -1 and "n_served" in lib.lmsf_attention_mma_last_error().decode()
    torch.cuda.synchronize()
    assert torch.all(out == 0)


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
