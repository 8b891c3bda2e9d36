"""ctypes faces of yinqiwen/lmsf's own CUDA launchers (built unmodified by `build_ref.py`).

Tensors are torch tensors used as plain device buffers; nothing of `lmsf_b200` is imported.  The
parameter structs repeat the reference's `extern "C"` declarations field for field:
RmsNormKernelParams (vllm/kernels/layernorm_kernels.cu:111-117), RotaryEmbeddingKernelParams
(pos_encoding_kernels.cu:82-93), RehshapeCacheKernelParams (cache_kernels.cu:236-245),
ActivationKernelParams (activation_kernels.cu:56-61), PagedAttentionV1Params / V2Params
(attention/attention_kernels.cu:660-673, :923-936).  Streams are passed as null like the reference
does (vllm/src/rms_norm.rs:68); with its `--default-stream per-thread` build that is the calling
thread's default stream, which orders itself with torch's default stream.

Layouts the reference uses (cache_kernels.cu:154-161): key cache [blocks, kv_heads, head/x, block, x]
with x = 16 bytes / element size, value cache [blocks, kv_heads, head, block].
"""
from __future__ import annotations

import ctypes
from ctypes import c_bool, c_float, c_int, c_void_p

import torch

from .build_ref import ensure_built

DATA_F16, DATA_BF16, DATA_F32 = 1, 2, 3            # ScalarType, vllm/kernels/cuda_ext.h:5-11
PARTITION_SIZE = 512                               # core/src/model_executor/layers/attention.rs (_PARTITION_SIZE)


def scalar_type(dt: torch.dtype) -> int:
    return {torch.float16: DATA_F16, torch.bfloat16: DATA_BF16, torch.float32: DATA_F32}[dt]


class RmsNormKernelParams(ctypes.Structure):
    _fields_ = [("stream", c_void_p), ("epsilon", c_float), ("hidden_size", c_int), ("num_tokens", c_int),
                ("dtype", c_int)]


class RotaryEmbeddingKernelParams(ctypes.Structure):
    _fields_ = [("stream", c_void_p), ("head_size", c_int), ("num_tokens", c_int), ("rot_dim", c_int),
                ("num_heads", c_int), ("num_kv_heads", c_int), ("query_stride", c_int), ("key_stride", c_int),
                ("is_neox", c_bool), ("scalar_type", c_int)]


class ReshapeCacheKernelParams(ctypes.Structure):
    _fields_ = [("value_stride", c_int), ("key_stride", c_int), ("num_tokens", c_int), ("num_heads", c_int),
                ("head_size", c_int), ("block_size", c_int), ("x", c_int), ("scalar_type", c_int)]


class ActivationKernelParams(ctypes.Structure):
    _fields_ = [("stream", c_void_p), ("d", c_int), ("num_tokens", c_int), ("dtype", c_int)]


class PagedAttentionV1Params(ctypes.Structure):
    _fields_ = [("block_size", c_int), ("num_seqs", c_int), ("num_heads", c_int), ("num_kv_heads", c_int),
                ("head_size", c_int), ("max_num_blocks_per_seq", c_int), ("q_stride", c_int),
                ("kv_block_stride", c_int), ("kv_head_stride", c_int), ("max_context_len", c_int),
                ("scale", c_float), ("scalar_type", c_int)]


class PagedAttentionV2Params(ctypes.Structure):
    _fields_ = [("block_size", c_int), ("num_seqs", c_int), ("num_heads", c_int), ("head_size", c_int),
                ("num_kv_heads", c_int), ("max_num_blocks_per_seq", c_int), ("q_stride", c_int),
                ("kv_block_stride", c_int), ("kv_head_stride", c_int), ("max_context_len", c_int),
                ("scale", c_float), ("scalar_type", c_int)]


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(ensure_built())
        _lib.vllm_rms_norm.argtypes = [c_void_p, c_void_p, c_void_p, RmsNormKernelParams]
        _lib.vllm_fused_add_rms_norm.argtypes = [c_void_p, c_void_p, c_void_p, RmsNormKernelParams]
        _lib.rotary_embedding.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, RotaryEmbeddingKernelParams]
        _lib.reshape_and_cache.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, ReshapeCacheKernelParams]
        _lib.vllm_silu_and_mul.argtypes = [c_void_p, c_void_p, ActivationKernelParams]
        _lib.paged_attention_v1.argtypes = [c_void_p] * 7 + [PagedAttentionV1Params]
        _lib.paged_attention_v2.argtypes = [c_void_p] * 10 + [PagedAttentionV2Params]
        for f in (_lib.vllm_rms_norm, _lib.vllm_fused_add_rms_norm, _lib.rotary_embedding, _lib.reshape_and_cache,
                  _lib.vllm_silu_and_mul, _lib.paged_attention_v1, _lib.paged_attention_v2):
            f.restype = None
    return _lib


def _c(t: torch.Tensor) -> torch.Tensor:
    assert t.is_cuda and t.is_contiguous(), "reference kernels take contiguous CUDA tensors"
    return t


def rms_norm(out, x, w, eps):
    """out = T(x * rsqrt(mean(x^2) + eps)) * w (layernorm_kernels.cu:13-37)."""
    n, h = x.shape
    lib().vllm_rms_norm(_c(out).data_ptr(), _c(x).data_ptr(), _c(w).data_ptr(),
                        RmsNormKernelParams(None, eps, h, n, scalar_type(x.dtype)))


def fused_add_rms_norm(x, residual, w, eps):
    """In place: residual = T(x + residual); x = T(residual * rsqrt(mean + eps)) * w (layernorm_kernels.cu:40-67)."""
    n, h = x.shape
    lib().vllm_fused_add_rms_norm(_c(x).data_ptr(), _c(residual).data_ptr(), _c(w).data_ptr(),
                                  RmsNormKernelParams(None, eps, h, n, scalar_type(x.dtype)))


def cos_sin_cache(base: float, rot_dim: int, max_pos: int, dtype, device, inv_freq=None):
    """[max_pos, rot_dim]: cos of position x inv_freq in float32, then sin, cast to dtype
    (vllm/src/pos_encoding.rs:8-36).  inv_freq may be given (scaled frequencies, which the reference lacks)."""
    if inv_freq is None:
        inv_freq = torch.tensor([1.0 / base ** (i / rot_dim) for i in range(0, rot_dim, 2)], dtype=torch.float32)
    inv_freq = inv_freq.to(device=device, dtype=torch.float32)
    t = torch.arange(max_pos, device=device, dtype=torch.float32)[:, None]
    fr = t * inv_freq[None, :]
    return torch.cat([fr.cos(), fr.sin()], dim=-1).to(dtype).contiguous()


def rotary_embedding(positions_i64, q, k, cache, head_size, num_heads, num_kv_heads, is_neox=True):
    """Rotates q [n, heads*head] and k [n, kv_heads*head] in place (row strides free, pos_encoding_kernels.cu:43-76)."""
    assert positions_i64.dtype == torch.int64 and q.stride(1) == 1 and k.stride(1) == 1
    p = RotaryEmbeddingKernelParams(None, head_size, q.shape[0], cache.shape[1], num_heads, num_kv_heads,
                                    q.stride(0), k.stride(0), is_neox, scalar_type(q.dtype))
    lib().rotary_embedding(positions_i64.data_ptr(), q.data_ptr(), k.data_ptr(), _c(cache).data_ptr(), p)


def reshape_and_cache(k, v, key_cache, value_cache, slot_mapping_i64, num_kv_heads, head_size, block_size):
    """Scatters the rows of k, v to slot = page * block_size + offset (cache_kernels.cu:186-232)."""
    assert slot_mapping_i64.dtype == torch.int64 and k.stride(1) == 1 and v.stride(1) == 1
    x = 16 // k.element_size()
    p = ReshapeCacheKernelParams(v.stride(0), k.stride(0), k.shape[0], num_kv_heads, head_size, block_size, x,
                                 scalar_type(k.dtype))
    lib().reshape_and_cache(k.data_ptr(), v.data_ptr(), _c(key_cache).data_ptr(), _c(value_cache).data_ptr(),
                            _c(slot_mapping_i64).data_ptr(), p)


def silu_and_mul(out, x):
    """out[t, i] = T(silu(x[t, i])) * x[t, d + i] (activation_kernels.cu:26-41)."""
    n, d = out.shape
    lib().vllm_silu_and_mul(_c(out).data_ptr(), _c(x).data_ptr(), ActivationKernelParams(None, d, n, scalar_type(x.dtype)))


def new_caches(num_blocks, num_kv_heads, head_size, block_size, dtype, device):
    x = 16 // torch.empty((), dtype=dtype).element_size()
    kc = torch.zeros((num_blocks, num_kv_heads, head_size // x, block_size, x), dtype=dtype, device=device)
    vc = torch.zeros((num_blocks, num_kv_heads, head_size, block_size), dtype=dtype, device=device)
    return kc, vc


def paged_attention(out, q, key_cache, value_cache, block_tables_i32, context_lens_i32, max_context_len, scale,
                    num_kv_heads, force=None, workspace=None):
    """Decode attention of one token per request, v1 or v2 chosen by the reference's own rule
    (core/src/model_executor/layers/attention.rs:255-257); `force` = "v1" / "v2" overrides it.
    q, out: [seqs, heads, head]; q may be a view whose rows are strided (the kernels take q_stride)."""
    n, nh, hd = q.shape
    assert q.is_cuda and q.stride(2) == 1 and q.stride(1) == hd
    parts = -(-max_context_len // PARTITION_SIZE)
    use_v1 = max_context_len <= 8192 and (parts == 1 or n * nh > 512)
    if force is not None:
        use_v1 = force == "v1"
    bs = value_cache.shape[3]
    common = dict(block_size=bs, num_seqs=n, num_heads=nh, num_kv_heads=num_kv_heads, head_size=hd,
                  max_num_blocks_per_seq=block_tables_i32.shape[1], q_stride=q.stride(0),
                  kv_block_stride=key_cache.stride(0), kv_head_stride=key_cache.stride(1),
                  max_context_len=max_context_len, scale=scale, scalar_type=scalar_type(q.dtype))
    if use_v1:
        lib().paged_attention_v1(_c(out).data_ptr(), q.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
                                 _c(block_tables_i32).data_ptr(), _c(context_lens_i32).data_ptr(), None,
                                 PagedAttentionV1Params(**common))
        return "v1"
    if workspace is None:
        workspace = (torch.empty((n, nh, parts, hd), dtype=q.dtype, device=q.device),
                     torch.empty((n, nh, parts), dtype=torch.float32, device=q.device),
                     torch.empty((n, nh, parts), dtype=torch.float32, device=q.device))
    tmp_out, exp_sums, max_logits = workspace
    lib().paged_attention_v2(_c(out).data_ptr(), exp_sums.data_ptr(), max_logits.data_ptr(), tmp_out.data_ptr(),
                             q.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
                             _c(block_tables_i32).data_ptr(), _c(context_lens_i32).data_ptr(), None,
                             PagedAttentionV2Params(**common))
    return "v2"
