"""Python faces of the CUDA kernels in `csrc/`.

Each function checks what the kernel cannot check (device, dtype, contiguity), takes the
launching stream from torch and raises `KernelError` with the library's own message when
the kernel refuses a size.  There is no CPU path: tensors that are not on a CUDA device
are an error.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional, Sequence, Tuple

import torch

from .csrc.build import load_library

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dt}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The handle of the current stream of the current device (asked at every launch: graphs are captured on
    another stream).  The raw getter saves building a Stream object, about 2 us a launch."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("lmsf_b200 kernels run on CUDA tensors only; got a tensor on " + str(t.device))
    return t.data_ptr()


def _i32(t: Optional[torch.Tensor], name: str) -> Optional[int]:
    if t is None:
        return None
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")
    return _ptr(t)


_FUNCS = {}


def _func(source: str, name: str, argtypes, defines: Tuple[str, ...] = ()):
    key = (source, name, defines)
    f = _FUNCS.get(key)
    if f is None:
        lib = load_library(source, defines)
        f = getattr(lib, name)
        f.argtypes = argtypes
        f.restype = c_int
        _FUNCS[key] = f
    return f


_LAUNCHES = 0


def launch_count() -> int:
    """Kernels of this package launched so far (launches replayed from a CUDA graph are added by the runner)."""
    return _LAUNCHES


def add_launches(n: int) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def _check(rc: int, source: str, prefix: str, defines: Tuple[str, ...] = ()):
    global _LAUNCHES
    if rc == 0:
        _LAUNCHES += 1
        return
    if rc < 0:
        lib = load_library(source, defines)
        getter = getattr(lib, prefix + "_last_error")
        getter.restype = ctypes.c_char_p
        raise KernelError(getter().decode())
    raise KernelError(f"CUDA error {rc} at the launch of a kernel of {source}")


# ----------------------------------------------------------------------------- embedding

def embedding(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, error_flag: Optional[torch.Tensor] = None,
              scale: float = 1.0):
    """out[t, :] = table[ids[t], :] (times `scale`, if it is not 1); out and table share one dtype."""
    n, hidden = out.shape
    if table.dtype != out.dtype or table.shape[1] != hidden or not (out.is_contiguous() and table.is_contiguous()):
        raise KernelError("embedding: out and table must be contiguous, of one dtype and one width")
    if scale != 1.0:
        f = _func("embedding.cu", "lmsf_embedding_scaled",
                  [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
        rc = f(_ptr(out), _ptr(table), _i32(ids, "ids"), n, hidden, table.shape[0], float(scale), dtype_code(out.dtype),
               _i32(error_flag, "error_flag"), _stream())
        _check(rc, "embedding.cu", "lmsf_embedding")
        return
    f = _func("embedding.cu", "lmsf_embedding",
              [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    rc = f(_ptr(out), _ptr(table), _i32(ids, "ids"), n, hidden, table.shape[0], dtype_code(out.dtype),
           _i32(error_flag, "error_flag"), _stream())
    _check(rc, "embedding.cu", "lmsf_embedding")


def patch_tokens(token_ids: torch.Tensor, dst: torch.Tensor, src: torch.Tensor, source: torch.Tensor):
    """token_ids[dst[i]] = source[src[i]] wherever dst[i] >= 0 (all int32, on the device)."""
    f = _func("embedding.cu", "lmsf_patch_tokens", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    rc = f(_i32(token_ids, "token_ids"), _i32(dst, "dst"), _i32(src, "src"), _i32(source, "source"), dst.numel(), _stream())
    _check(rc, "embedding.cu", "lmsf_embedding")


# ----------------------------------------------------------------------------- rmsnorm

def add_rmsnorm(h: torch.Tensor, x: torch.Tensor, res: Optional[torch.Tensor], w: torch.Tensor, eps: float, mode: int):
    """mode 0: h = norm(x) w.  mode 1: res = float(x); h = norm(res) w.  mode 2: res += float(x); h = norm(res) w.
    x, h: [n, hidden] float32 or bfloat16; res: float32; w: [hidden] of x's dtype or float32."""
    n, hidden = x.shape
    if h.shape != x.shape or h.dtype != x.dtype or not (x.is_contiguous() and h.is_contiguous()):
        raise KernelError("rmsnorm: h and x must be contiguous and alike")
    if res is not None and (res.dtype != torch.float32 or res.shape != x.shape or not res.is_contiguous()):
        raise KernelError("rmsnorm: the residual must be contiguous float32 of x's shape")
    if w.shape != (hidden,) or not w.is_contiguous():
        raise KernelError(f"rmsnorm: weight of shape {tuple(w.shape)} for width {hidden}")
    f = _func("rmsnorm.cu", "lmsf_add_rmsnorm",
              [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p])
    rc = f(_ptr(h), _ptr(x), _ptr(res), _ptr(w), n, hidden, float(eps), mode, dtype_code(x.dtype),
           dtype_code(w.dtype), _stream())
    _check(rc, "rmsnorm.cu", "lmsf_rmsnorm")


def finish_rmsnorm(h: torch.Tensor, res: torch.Tensor, sumsq: torch.Tensor, w: torch.Tensor, eps: float):
    """h = (res / rms) w, where sumsq[m] adds up to the sum of squares of row m of res: the second half of a norm whose
    first half `gemm_skinny_residual` did, for a product that cannot take a prenormed input."""
    n, hidden = res.shape
    if h.shape != res.shape or h.dtype != torch.bfloat16 or not (h.is_contiguous() and res.is_contiguous()) or res.dtype != torch.float32:
        raise KernelError("finish_rmsnorm: h must be bfloat16 and res float32, contiguous and of one shape")
    if sumsq.dtype != torch.float32 or sumsq.dim() != 2 or sumsq.shape[0] < n or sumsq.stride(1) != 1:
        raise KernelError("finish_rmsnorm: the sums of squares must be float32 [rows, parts]")
    if w.shape != (hidden,) or not w.is_contiguous():
        raise KernelError(f"finish_rmsnorm: weight of shape {tuple(w.shape)} for width {hidden}")
    f = _func("rmsnorm.cu", "lmsf_finish_rmsnorm",
              [c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_int, c_int, c_float, c_int, c_int, c_void_p])
    rc = f(_ptr(h), _ptr(res), _ptr(sumsq), sumsq.shape[1], sumsq.stride(0), _ptr(w), n, hidden, float(eps),
           dtype_code(h.dtype), dtype_code(w.dtype), _stream())
    _check(rc, "rmsnorm.cu", "lmsf_rmsnorm")


# ----------------------------------------------------------------------------- rope + cache write

def rope_cache_write(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor], positions: torch.Tensor,
                     token_seq: Optional[torch.Tensor], block_table: Optional[torch.Tensor], block_size: int,
                     cache: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], rot_dim: int, is_neox: bool,
                     n_q_heads: int, n_kv_heads: int, head_dim: int, error_flag: Optional[torch.Tensor] = None):
    """Rotates q in place; writes rotated k and v into `cache` [pages, 2, n_kv_heads, block_size, head_dim]
    at the page that `block_table[token_seq[t], positions[t] // block_size]` names.  q, k, v: [n, heads*head_dim]
    views whose last dimension is contiguous (row strides are free).  cache None: q only."""
    n = q.shape[0]
    for name, t, heads in (("q", q, n_q_heads), ("k", k, n_kv_heads), ("v", v, n_kv_heads)):
        if t is None:
            continue
        if t.dim() != 2 or t.shape[1] != heads * head_dim or t.stride(1) != 1 or t.shape[0] != n:
            raise KernelError(f"rope_cache: {name} must be [n, {heads * head_dim}] with a contiguous last dimension")
        if t.dtype != q.dtype:
            raise KernelError("rope_cache: q, k, v must share one dtype")
    page_stride = 0
    max_blocks = 0
    if cache is not None:
        if cache.dtype != q.dtype or not cache.is_contiguous() or tuple(cache.shape[1:]) != (2, n_kv_heads, block_size, head_dim):
            raise KernelError(f"rope_cache: cache of shape {tuple(cache.shape)} does not match "
                              f"[pages, 2, {n_kv_heads}, {block_size}, {head_dim}] of {q.dtype}")
        page_stride = cache.stride(0)
        max_blocks = block_table.shape[1]
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dim // 2):
        raise KernelError("rope_cache: inv_freq must hold rot_dim / 2 float32 values")
    f = _func("rope_cache.cu", "lmsf_rope_cache_write",
              [c_void_p, c_void_p, c_void_p, c_longlong, c_longlong, c_longlong, c_void_p, c_void_p, c_void_p, c_int,
               c_int, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
               c_void_p])
    rc = f(_ptr(q), _ptr(k), _ptr(v), q.stride(0), k.stride(0) if k is not None else 0,
           v.stride(0) if v is not None else 0, _i32(positions, "positions"), _i32(token_seq, "token_seq"),
           _i32(block_table, "block_table"), max_blocks, block_size, _ptr(cache), page_stride, _ptr(inv_freq),
           rot_dim, int(is_neox), n, n_q_heads, n_kv_heads, head_dim, dtype_code(q.dtype),
           _i32(error_flag, "error_flag"), _stream())
    _check(rc, "rope_cache.cu", "lmsf_rope_cache")


# ----------------------------------------------------------------------------- attention (generic)

def attention_generic(out: torch.Tensor, q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                      block_size: int, token_seq: torch.Tensor, positions: torch.Tensor, scale: float, window: int,
                      n_q_heads: int, n_kv_heads: int, head_dim: int, softcap: float = 0.0,
                      slopes: Optional[torch.Tensor] = None):
    """out[t] = softmax(scale q[t] K^T) V over the keys lo..positions[t] of token t's request, read from pages.
    q, out: [n, n_q_heads * head_dim] (last dimension contiguous); window <= 0 means all keys; softcap > 0 caps the
    scaled scores smoothly, softcap * tanh(score / softcap); slopes (float32 [n_q_heads]) adds
    slopes[head] * (key position - query position) to the scaled scores."""
    n = q.shape[0]
    if q.stride(1) != 1 or out.stride(1) != 1 or q.shape[1] != n_q_heads * head_dim or out.shape != q.shape:
        raise KernelError("attention: q and out must be [n, heads * head_dim] with a contiguous last dimension")
    if cache.dtype != q.dtype or out.dtype != q.dtype or not cache.is_contiguous() or \
            tuple(cache.shape[1:]) != (2, n_kv_heads, block_size, head_dim):
        raise KernelError(f"attention: cache of shape {tuple(cache.shape)} / {cache.dtype} does not match the heads")
    if slopes is not None and (slopes.dtype != torch.float32 or slopes.shape != (n_q_heads,) or not slopes.is_contiguous()):
        raise KernelError("attention: slopes must be float32 [n_q_heads]")
    f = _func("attention_generic.cu", "lmsf_attention_generic_scores",
              [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_int, c_void_p,
               c_void_p, c_float, c_float, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    rc = f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cache), cache.stride(0),
           _i32(block_table, "block_table"), block_table.shape[1], block_size, _i32(token_seq, "token_seq"),
           _i32(positions, "positions"), float(scale), float(softcap or 0.0), _ptr(slopes), int(window or 0), n, n_q_heads,
           n_kv_heads, head_dim, dtype_code(q.dtype), _stream())
    _check(rc, "attention_generic.cu", "lmsf_attention_generic")


# ----------------------------------------------------------------------------- gated activation

ACT_CODES = {"silu": 0, "swish": 0, "gelu_tanh": 1, "gelu_pytorch_tanh": 1}


def gated_act(out: torch.Tensor, x: torch.Tensor, act: str = "silu"):
    """out[t, i] = act(x[t, i]) * x[t, d + i]; x: [n, 2 d], out: [n, d] contiguous."""
    n, d = out.shape
    if x.shape != (n, 2 * d) or x.stride(1) != 1 or not out.is_contiguous() or x.dtype != out.dtype:
        raise KernelError("gated_act: x must be [n, 2d] and out [n, d] of one dtype")
    if act not in ACT_CODES:
        raise KernelError(f"gated_act: unknown activation {act!r} (known: {', '.join(sorted(ACT_CODES))})")
    f = _func("activation.cu", "lmsf_gated_act", [c_void_p, c_void_p, c_int, c_int, c_longlong, c_int, c_int, c_void_p])
    rc = f(_ptr(out), _ptr(x), n, d, x.stride(0), ACT_CODES[act], dtype_code(out.dtype), _stream())
    _check(rc, "activation.cu", "lmsf_activation")


def bias_add(x: torch.Tensor, bias: torch.Tensor):
    """x[t, :] += bias in place (sum in float32); x: [n, d] with a contiguous last dimension, bias: [d] of x's dtype."""
    n, d = x.shape
    if bias.shape != (d,) or bias.dtype != x.dtype or x.stride(1) != 1 or not bias.is_contiguous():
        raise KernelError(f"bias_add: x {tuple(x.shape)} / {x.dtype} and bias {tuple(bias.shape)} / {bias.dtype} do not match")
    f = _func("activation.cu", "lmsf_bias_add", [c_void_p, c_void_p, c_int, c_int, c_longlong, c_int, c_void_p])
    rc = f(_ptr(x), _ptr(bias), n, d, x.stride(0), dtype_code(x.dtype), _stream())
    _check(rc, "activation.cu", "lmsf_activation")


# ----------------------------------------------------------------------------- SIMT matrix product

def gemm_tn_simt(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor):
    """out[M, N] = a[M, K] w[N, K]^T, float32 FMA accumulation in ascending k (true 32-bit when a, w are float32)."""
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"gemm: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if a.dtype != w.dtype:
        raise KernelError("gemm: a and w must share one dtype")
    f = _func("gemm_simt.cu", "lmsf_gemm_tn_simt",
              [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int, c_int,
               c_void_p])
    rc = f(_ptr(out), _ptr(a), _ptr(w), M, N, K, a.stride(0), w.stride(0), out.stride(0), dtype_code(a.dtype),
           dtype_code(out.dtype), _stream())
    _check(rc, "gemm_simt.cu", "lmsf_gemm_simt")


# ----------------------------------------------------------------------------- weight-streaming product (M <= 16)

SKINNY_MAX_M = 16
# build-time constants of gemm_skinny.cu; experiments override them, e.g. LMSF_SKINNY_DEFINES=LMSF_SKINNY_STAGES=5
SKINNY_DEFINES: Tuple[str, ...] = tuple(d for d in os.environ.get("LMSF_SKINNY_DEFINES", "").split(",") if d)


def gemm_skinny_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and 0 < x.shape[0] <= SKINNY_MAX_M
            and x.shape[1] % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1 and w.stride(0) % 8 == 0
            and x.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0 and x.data_ptr() % 16 == 0)


def _prenorm_args(prenorm, M: int, what: str):
    """(sums of squares [>= M, parts] float32, eps, width) of a prenormed input -> the kernel's five arguments."""
    if prenorm is None:
        return None, 0, 0, 0.0, 0
    sumsq, eps, width = prenorm
    if sumsq.dtype != torch.float32 or sumsq.dim() != 2 or sumsq.shape[0] < M or sumsq.stride(1) != 1:
        raise KernelError(f"{what}: the sums of squares must be float32 [rows, parts]")
    return _ptr(sumsq), sumsq.shape[1], sumsq.stride(0), float(eps), int(width)


def gemm_skinny(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, fuse_act: Optional[str] = None, prenorm=None):
    """out[M, N] = x[M, K] w[N, K]^T for M <= 16 (bfloat16 in, bfloat16 or float32 out).  With fuse_act
    ("silu", "gelu_tanh") w is [2 N_out, K] (gate rows, then up rows) and out[M, N_out] = act(x gate^T) * (x up^T).
    prenorm = (sumsq, eps, width): x is a residual stream times a norm weight and the sums of row m are multiplied by
    1 / sqrt(sum(sumsq[m]) / width + eps) first (what `gemm_skinny_residual` leaves)."""
    M, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if fuse_act else N
    if not gemm_skinny_supported(x, w) or w.shape[1] != K or out.shape != (M, n_out) or out.stride(1) != 1:
        raise KernelError(f"gemm_skinny: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} are not taken")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_skinny: out must be bfloat16 or float32")
    if fuse_act is not None and fuse_act not in ACT_CODES:
        raise KernelError(f"gemm_skinny: unknown activation {fuse_act!r}")
    f = _func("gemm_skinny.cu", "lmsf_gemm_skinny",
              [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int, c_int,
               c_void_p, c_int, c_longlong, c_float, c_int, c_void_p], SKINNY_DEFINES)
    rc = f(_ptr(out), _ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(0), out.stride(0),
           ACT_CODES[fuse_act] if fuse_act else -1, int(out.dtype == torch.float32),
           *_prenorm_args(prenorm, M, "gemm_skinny"), _stream())
    _check(rc, "gemm_skinny.cu", "lmsf_gemm_skinny", SKINNY_DEFINES)


def gemm_skinny_residual_parts(n: int) -> int:
    """Partial sums of squares per row that `gemm_skinny_residual` leaves for n output features."""
    return (n + 15) // 16


def gemm_skinny_residual(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, res: torch.Tensor, norm_w: torch.Tensor,
                         sumsq: torch.Tensor):
    """A product, the residual add after it and the first half of the RMSNorm after that, for M <= 16 rows:
    res[M, N] (float32) += bfloat16(x w^T); out[M, N] (bfloat16) = res * norm_w; sumsq[m, b] = the sum of squares of
    row m's new residual values 16 b .. 16 b + 15.  `gemm_skinny(..., prenorm=(sumsq, eps, N))` is the other half."""
    M, K = x.shape
    N = w.shape[0]
    if not gemm_skinny_supported(x, w) or w.shape[1] != K or out.shape != (M, N) or out.stride(1) != 1 or out.dtype != torch.bfloat16:
        raise KernelError(f"gemm_skinny_residual: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} are not taken")
    if res.dtype != torch.float32 or res.shape != (M, N) or res.stride(1) != 1:
        raise KernelError("gemm_skinny_residual: the residual must be float32 of the output's shape")
    if norm_w.shape != (N,) or not norm_w.is_contiguous() or norm_w.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError("gemm_skinny_residual: the norm weight must be [N], float32 or bfloat16")
    if (sumsq.dtype != torch.float32 or sumsq.dim() != 2 or sumsq.shape[0] < M or sumsq.stride(1) != 1
            or sumsq.shape[1] != gemm_skinny_residual_parts(N)):
        raise KernelError("gemm_skinny_residual: the sums of squares must be float32 [rows, gemm_skinny_residual_parts(N)]")
    f = _func("gemm_skinny.cu", "lmsf_gemm_skinny_residual",
              [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_longlong,
               c_void_p, c_int, c_void_p, c_longlong, c_void_p], SKINNY_DEFINES)
    rc = f(_ptr(out), out.stride(0), _ptr(x), x.stride(0), _ptr(w), w.stride(0), M, N, K, _ptr(res), res.stride(0),
           _ptr(norm_w), int(norm_w.dtype == torch.float32), _ptr(sumsq), sumsq.stride(0), _stream())
    _check(rc, "gemm_skinny.cu", "lmsf_gemm_skinny", SKINNY_DEFINES)


def gemm_skinny_qkv_rope_supported(x: torch.Tensor, w: torch.Tensor, head_dim: int, rot_dim: int, is_neox: bool) -> bool:
    return (gemm_skinny_supported(x, w) and head_dim % 16 == 0
            and (rot_dim == 0 or (rot_dim % 16 == 0 if is_neox else rot_dim % 2 == 0)))


def gemm_skinny_qkv_rope(q_out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, positions: torch.Tensor, token_seq: torch.Tensor,
                         block_table: torch.Tensor, block_size: int, cache: torch.Tensor, inv_freq: Optional[torch.Tensor],
                         rot_dim: int, is_neox: bool, n_q_heads: int, n_kv_heads: int, head_dim: int,
                         error_flag: Optional[torch.Tensor] = None, prenorm=None):
    """The merged q, k, v projection of up to 16 single tokens (x [M, K] bfloat16, w [(heads + 2 kv heads) * head_dim, K])
    with the rotary encoding and the cache write in its epilogue: q_out [M, heads * head_dim] gets the rotated q, the
    pages of `cache` the rotated k and v.  The same values as gemm_skinny followed by rope_cache_write.  prenorm: as in
    `gemm_skinny`."""
    M, K = x.shape
    if (not gemm_skinny_qkv_rope_supported(x, w, head_dim, rot_dim if inv_freq is not None else 0, is_neox)
            or w.shape != ((n_q_heads + 2 * n_kv_heads) * head_dim, K) or q_out.shape != (M, n_q_heads * head_dim)
            or q_out.dtype != torch.bfloat16 or q_out.stride(1) != 1):
        raise KernelError(f"gemm_skinny_qkv_rope: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(q_out.shape)} are not taken")
    if not cache.is_contiguous() or tuple(cache.shape[1:]) != (2, n_kv_heads, block_size, head_dim) or cache.dtype != torch.bfloat16:
        raise KernelError(f"gemm_skinny_qkv_rope: cache of shape {tuple(cache.shape)} does not match the heads")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dim // 2):
        raise KernelError("gemm_skinny_qkv_rope: inv_freq must be float32 [rot_dim / 2]")
    f = _func("gemm_skinny.cu", "lmsf_gemm_skinny_qkv_rope",
              [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p,
               c_int, c_int, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
               c_void_p, c_int, c_longlong, c_float, c_int, c_void_p], SKINNY_DEFINES)
    rc = f(_ptr(q_out), q_out.stride(0), _ptr(x), x.stride(0), _ptr(w), w.stride(0), M, K, _i32(positions, "positions"),
           _i32(token_seq, "token_seq"), _i32(block_table, "block_table"), block_table.shape[1], block_size, _ptr(cache),
           cache.stride(0), _ptr(inv_freq) if inv_freq is not None else None, int(rot_dim), int(bool(is_neox)), n_q_heads,
           n_kv_heads, head_dim, _i32(error_flag, "error_flag"), *_prenorm_args(prenorm, M, "gemm_skinny_qkv_rope"), _stream())
    _check(rc, "gemm_skinny.cu", "lmsf_gemm_skinny", SKINNY_DEFINES)


# ----------------------------------------------------------------------------- the device's error word

_ERROR_WORDS = {}


def error_word(device) -> torch.Tensor:
    """The int32 word of a device in which kernels report errors that they cannot return (a wait that ran out,
    an id outside a table); the model runner reads and clears it after a step."""
    key = torch.device(device).index or 0
    w = _ERROR_WORDS.get(key)
    if w is None:
        w = _ERROR_WORDS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return w


# ----------------------------------------------------------------------------- sampling

def sample(out: torch.Tensor, logits: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           seed: Optional[torch.Tensor] = None, step: Optional[torch.Tensor] = None):
    """out[r] = greedy or temperature sample of logits[r] (float32).  temperature [rows] float32,
    seed [rows] int64 (bit pattern of an unsigned 64-bit seed), step [rows] int32; all None: greedy."""
    rows, vocab = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 with a contiguous last dimension")
    if out.dtype != torch.int32 or out.shape != (rows,) or not out.is_contiguous():
        raise KernelError("sample: out must be int32 [rows]")
    if temperature is not None and (temperature.dtype != torch.float32 or temperature.shape != (rows,)):
        raise KernelError("sample: temperature must be float32 [rows]")
    if seed is not None and (seed.dtype != torch.int64 or seed.shape != (rows,)):
        raise KernelError("sample: seed must be int64 [rows]")
    parts = 1 if vocab < 16384 else min(32, max(1, vocab // 8192))
    scratch = torch.empty(rows * parts * 2, dtype=torch.float64, device=logits.device) if parts > 1 else None
    f = _func("sampling.cu", "lmsf_sample",
              [c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p])
    rc = f(_ptr(out), _ptr(logits), logits.stride(0), rows, vocab, _ptr(temperature), _ptr(seed), _i32(step, "step"),
           parts, _ptr(scratch), _stream())
    _check(rc, "sampling.cu", "lmsf_sampling")
    if parts > 1:
        add_launches(1)


def apply_penalties(logits: torch.Tensor, rows: torch.Tensor, tokens: torch.Tensor, out_counts: torch.Tensor,
                    presence: torch.Tensor, frequency: torch.Tensor, repetition: torch.Tensor):
    """In place on float32 logits [n_rows, vocab]: for every listed (row, token) pair the repetition, frequency
    and presence penalties of that row; out_counts is how often the token occurs in the row's output so far
    (0: it occurs in the prompt only).  presence / frequency / repetition: float32 [n_rows]."""
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("apply_penalties: logits must be float32 with a contiguous last dimension")
    n = rows.numel()
    for t in (presence, frequency, repetition):
        if t.dtype != torch.float32 or t.shape != (logits.shape[0],):
            raise KernelError("apply_penalties: per-row penalties must be float32 [n_rows]")
    f = _func("sampling.cu", "lmsf_apply_penalties",
              [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    rc = f(_ptr(logits), logits.stride(0), _i32(rows, "rows"), _i32(tokens, "tokens"), _i32(out_counts, "out_counts"),
           n, _ptr(presence), _ptr(frequency), _ptr(repetition), _stream())
    _check(rc, "sampling.cu", "lmsf_sampling")


def sample_filtered(out: torch.Tensor, logits: torch.Tensor, temperature: torch.Tensor, seed: torch.Tensor,
                    step: torch.Tensor, top_k: Optional[torch.Tensor], top_p: Optional[torch.Tensor],
                    min_p: Optional[torch.Tensor], row_ids: Optional[torch.Tensor] = None):
    """Temperature sampling of the rows in row_ids (None: all) among the tokens kept by top_k (int32, <= 0 off),
    top_p (float32, 1 off) and min_p (float32, 0 off); per-row arrays are indexed by row."""
    rows, vocab = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or out.dtype != torch.int32 or out.shape != (rows,):
        raise KernelError("sample_filtered: logits float32 [rows, vocab], out int32 [rows]")
    n = rows if row_ids is None else row_ids.numel()
    f = _func("sampling.cu", "lmsf_sample_filtered",
              [c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
               c_void_p, c_void_p])
    rc = f(_ptr(out), _ptr(logits), logits.stride(0), n, vocab, _ptr(temperature), _ptr(seed), _i32(step, "step"),
           _i32(top_k, "top_k"), _ptr(top_p), _ptr(min_p), _i32(row_ids, "row_ids"), _stream())
    _check(rc, "sampling.cu", "lmsf_sampling")


# ----------------------------------------------------------------------------- tensor-core attention (bfloat16)

MMA_MAX_HEAD_DIM = 128


def mma_attention_supported(dtype: torch.dtype, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= MMA_MAX_HEAD_DIM


MMA_KV_STAGES = None   # pipeline depth of the attention kernels, a build-time constant of attention_mma.cu (None: its own choice)


def _mma_defines(head_dim: int) -> Tuple[str, ...]:
    if MMA_KV_STAGES is None:
        return (f"LMSF_HEAD_DIM={head_dim}",)
    return (f"LMSF_HEAD_DIM={head_dim}", f"LMSF_KV_STAGES={MMA_KV_STAGES}")


def _check_paged(q, out, cache, n_q_heads, n_kv_heads, head_dim, block_size, what):
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError(f"{what}: bfloat16 only")
    if q.stride(1) != 1 or out.stride(1) != 1 or q.shape[1] != n_q_heads * head_dim or out.shape != q.shape:
        raise KernelError(f"{what}: q and out must be [n, heads * head_dim] with a contiguous last dimension")
    if not cache.is_contiguous() or tuple(cache.shape[1:]) != (2, n_kv_heads, block_size, head_dim):
        raise KernelError(f"{what}: cache of shape {tuple(cache.shape)} does not match the heads")
    if (q.data_ptr() | out.data_ptr()) % 4 or (q.stride(0) | out.stride(0)) % 2 or cache.data_ptr() % 16:
        raise KernelError(f"{what}: q/out rows must be 4-byte aligned and the cache 16-byte aligned")




_DECODE_WIDTHS = {}


def decode_widths(head_dim: int, group: int = 1) -> Tuple[Tuple[int, float, Tuple[int, ...]], ...]:
    """The widths a decode block comes in, widest first; for each: its warps, the rate at which one block streams
    keys (its bytes in flight, in units of 64 KB) and, for cluster sizes 1..8, how many clusters of that many blocks
    the device holds at a time (it depends on the group of query heads per kv head, which sizes a block's shared
    memory).  Head sizes up to 64 have one width: four of its blocks fit an SM anyway."""
    key = (head_dim, min(16, max(1, group)))
    t = _DECODE_WIDTHS.get(key)
    if t is None:
        lib = load_library("attention_mma.cu", _mma_defines(head_dim))
        lib.lmsf_attention_decode_max_clusters.restype = c_int
        lib.lmsf_attention_decode_max_clusters.argtypes = [c_int, c_int, c_int]
        lib.lmsf_attention_decode_stream_bytes.restype = c_int
        lib.lmsf_attention_decode_stream_bytes.argtypes = [c_int]
        widths = []
        for warps in ((4,) if head_dim <= 64 else (4, 2)):
            clusters = tuple(max(1, lib.lmsf_attention_decode_max_clusters(s, key[1], warps)) for s in range(1, 9))
            widths.append((warps, lib.lmsf_attention_decode_stream_bytes(warps) / 65536.0, clusters))
        t = _DECODE_WIDTHS[key] = tuple(widths)
    return t


# The cost model of decode_plan, in units of the time in which a block with 64 KB in flight streams 32 KB (about
# 1.5 us on B200); fitted to B200 measurements of 8 and 40 kv heads, 2,048 to 8,000 keys, 16 to 128 requests, both
# widths, 1 to 8 splits, alone and inside decode steps.
DECODE_WAVE_COST = 6.0          # what a wave of blocks costs before and after its keys
DECODE_SPLIT_COST = 4.0         # adding the splits of a request up
DECODE_GLOBAL_MERGE_COST = 6.0  # more when more than 8 splits add up through global memory
DECODE_SATURATION = 240.0       # blocks with 64 KB in flight that saturate the memory
DECODE_BLOCK_COST = 1.3         # what a block costs the slot it runs in, beside its keys (tables, first loads, its part of the sum)
DECODE_MUST_GAIN = 0.95         # a narrower block or a further split is taken when the model gives it 5 % less


def decode_plan(n_served: int, n_kv_heads: int, group: int, max_ctx: int, head_dim: int,
                widths: Sequence[Tuple[int, float, Sequence[int]]], mean_ctx: Optional[float] = None) -> Tuple[int, int]:
    """(splits, warps): into how many blocks the keys of a request are split, and how wide the blocks are.  Up to 8
    splits form a thread-block cluster (they add up through its shared memory) and clusters[s - 1] such clusters
    run at a time; more splits add up through global memory.  The choice minimises the sum over the waves of
    (fixed cost + keys per split / rate), where a block streams at the rate of its own bytes in flight or, when more
    blocks are resident than saturate the memory, at its share of the device: few long requests want wide blocks
    and many splits, many requests narrow blocks, of which twice as many are resident, and no second, partly filled
    wave.  Every split keeps at least 128 keys.  mean_ctx: the requests' mean number of keys, when it is far below
    max_ctx (one long request among short ones): every request gets the same number of splits, so the longest one
    sets the time of a wave unless it is split as if it were nearly alone; the short requests' extra blocks find
    no keys and cost only their slots (64 requests of the 8B shape, one with 30,000 keys among 63 with 500, took
    0.8 ms a layer planned for 64 requests of 30,000 keys, the long request's 8 blocks streaming alone).  Measured on B200 (head size 128, 8 kv heads, 2,048 keys):
    5 requests take 20.5 us with 6 splits (45 clusters fit) and 30.7 us with 7 (37 fit); 48 requests 100 us at best
    with wide blocks (2 splits) and 95 us with narrow ones (1 split); a decode step of 20 requests 4.72 ms with wide
    blocks and one split, 4.42 ms with narrow ones and 3."""
    per_request = n_kv_heads * ((group + 15) // 16)
    n_blocks1 = n_served * per_request                            # blocks of the launch per split
    # the requests that matter for the time of a wave: all of them, or as many as would hold the keys at max_ctx each
    work_served = n_served if not mean_ctx else max(1, min(n_served, -(-int(n_served * mean_ctx) // max(1, max_ctx))))
    base = work_served * per_request
    tiles = -(-max_ctx // 64)
    cap = max(1, -(-max_ctx // 128))
    tile_work = head_dim / 128.0                  # a 64-key tile of k and v in units of 32 KB
    best = None
    for warps, rate, clusters in widths:
        slots = clusters[0]
        for s in list(range(1, 9)) + [12, 16, 24, 32, 48, 64]:
            if s > cap:
                break
            per_wave = clusters[s - 1] if s <= 8 else max(1, slots // s)      # (request, head group) pairs per wave
            work = -(-tiles // s) * tile_work
            cost = (DECODE_SPLIT_COST if s > 1 else 0.0) + (DECODE_GLOBAL_MERGE_COST if s > 8 else 0.0)
            cost += DECODE_BLOCK_COST * n_blocks1 * s / (per_wave * s)
            left = base
            while left > 0:
                n = min(left, per_wave) * s
                cost += DECODE_WAVE_COST + work / min(rate, DECODE_SATURATION / n)
                left -= per_wave
            # candidates come widest first and with few splits first; a later one must be better by 5 %: measured,
            # near-ties of the model go to either side by a per cent, and wide blocks with few splits never lose more
            if best is None or cost < best[0] * DECODE_MUST_GAIN:
                best = (cost, s, warps)
    return best[1], best[2]


DECODE_COUNTER_SLOTS = 65536     # counters of delivered splits at the start of the scratch (attention_mma.cu)


def attention_decode_scratch_floats(n_seqs_total: int, n_q_heads: int, n_splits: int, head_dim: int) -> int:
    return 0 if n_splits <= 1 else DECODE_COUNTER_SLOTS + n_seqs_total * n_q_heads * n_splits * (head_dim + 1)


def attention_decode(out: torch.Tensor, q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                     block_size: int, seq_ids: Optional[torch.Tensor], n_served: int, cu_q: torch.Tensor,
                     ctx_len: torch.Tensor, scale: float, window: int, n_q_heads: int, n_kv_heads: int,
                     head_dim: int, n_splits: int, scratch: Optional[torch.Tensor], warps: int = 0):
    """Attention of requests that bring ONE query token each (row cu_q[s] of q), over their ctx_len[s] keys
    in pages.  seq_ids: int32 [n_served] rows of the block table that are served (None: all, in order).
    scratch: float32, at least attention_decode_scratch_floats(...) values when n_splits > 1, all zero when it is
    first used (torch.zeros); the kernel leaves its counters zero, so one buffer serves every later call.
    warps: the width of the blocks, 4 or 2 (decode_plan chooses it with n_splits); 0 leaves it to the kernel."""
    _check_paged(q, out, cache, n_q_heads, n_kv_heads, head_dim, block_size, "attention_decode")
    n_total = block_table.shape[0]
    need = attention_decode_scratch_floats(n_total, n_q_heads, n_splits, head_dim)
    if need and (scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need):
        raise KernelError(f"attention_decode: {n_splits} splits need {need} float32 values of scratch")
    d = _mma_defines(head_dim)
    if warps not in (0, 2, 4):
        raise KernelError(f"attention_decode: blocks have 2 or 4 warps, not {warps}")
    f = _func("attention_mma.cu", "lmsf_attention_decode_width",
              [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_void_p, c_int,
               c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_void_p,
               c_void_p], d)
    rc = f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cache), cache.stride(0), block_size, n_kv_heads,
           _i32(block_table, "block_table"), block_table.shape[1], _i32(seq_ids, "seq_ids"), n_served, n_total,
           _i32(cu_q, "cu_q"), _i32(ctx_len, "ctx_len"), float(scale), int(window or 0), n_q_heads, head_dim,
           n_splits, warps, _ptr(scratch) if need else None, _stream())
    _check(rc, "attention_mma.cu", "lmsf_attention_mma", d)


def decode_items_capacity(n_served: int, n_kv_heads: int, group: int, slots: int) -> int:
    """Entries of the list of work items of a launch with splits per request: one per request and as many more as
    the device holds blocks for."""
    return n_served + slots // (n_kv_heads * ((group + 15) // 16)) + 1


def attention_decode_items_scratch_floats(capacity: int, n_q_heads: int, head_dim: int) -> int:
    return DECODE_COUNTER_SLOTS + capacity * n_q_heads * (head_dim + 1)


def decode_build_items(items: torch.Tensor, ctx_len: torch.Tensor, seq_ids: Optional[torch.Tensor], n_served: int,
                       window: int, n_q_heads: int, n_kv_heads: int, head_dim: int, slots: int):
    """Fills `items` (int32 [capacity, 4]) on the device: request s gets ceil(keys_s / T) splits, with T the smallest
    number of keys for which all blocks fit the `slots` blocks that the device holds at a time; entries that are
    left over are padding.  The attention of requests that differ much in length runs over this list
    (attention_decode_items): each block then has about the same number of keys."""
    if items.dtype != torch.int32 or items.dim() != 2 or items.shape[1] != 4 or not items.is_contiguous():
        raise KernelError("decode_build_items: items must be a contiguous int32 tensor [capacity, 4]")
    d = _mma_defines(head_dim)
    f = _func("attention_mma.cu", "lmsf_attention_decode_build_items",
              [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p], d)
    rc = f(_i32(ctx_len, "ctx_len"), _i32(seq_ids, "seq_ids"), n_served, int(window or 0), n_q_heads, n_kv_heads,
           int(slots), items.shape[0], _ptr(items), _stream())
    _check(rc, "attention_mma.cu", "lmsf_attention_mma", d)


def attention_decode_items(out: torch.Tensor, q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                           block_size: int, items: torch.Tensor, cu_q: torch.Tensor, ctx_len: torch.Tensor,
                           scale: float, window: int, n_q_heads: int, n_kv_heads: int, head_dim: int, warps: int,
                           scratch: torch.Tensor):
    """attention_decode with splits per request, over a list made by decode_build_items.  scratch: float32, at
    least attention_decode_items_scratch_floats(capacity, ...) values, zero when first used."""
    _check_paged(q, out, cache, n_q_heads, n_kv_heads, head_dim, block_size, "attention_decode_items")
    need = attention_decode_items_scratch_floats(items.shape[0], n_q_heads, head_dim)
    if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
        raise KernelError(f"attention_decode_items: a list of {items.shape[0]} entries needs {need} float32 values of scratch")
    d = _mma_defines(head_dim)
    f = _func("attention_mma.cu", "lmsf_attention_decode_items",
              [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_void_p, c_int,
               c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_void_p, c_void_p], d)
    rc = f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cache), cache.stride(0), block_size, n_kv_heads,
           _i32(block_table, "block_table"), block_table.shape[1], _ptr(items), items.shape[0], block_table.shape[0],
           _i32(cu_q, "cu_q"), _i32(ctx_len, "ctx_len"), float(scale), int(window or 0), n_q_heads, head_dim, int(warps),
           _ptr(scratch), _stream())
    _check(rc, "attention_mma.cu", "lmsf_attention_mma", d)


def attention_prefill(out: torch.Tensor, q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                      block_size: int, tile_seq: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int, cu_q: torch.Tensor,
                      ctx_len: torch.Tensor, scale: float, window: int, n_q_heads: int, n_kv_heads: int, head_dim: int):
    """Attention of prompt portions.  Tile i covers the query tokens tile_q0[i] .. tile_q0[i] + 63 (counted
    inside the portion) of request tile_seq[i]."""
    _check_paged(q, out, cache, n_q_heads, n_kv_heads, head_dim, block_size, "attention_prefill")
    d = _mma_defines(head_dim)
    f = _func("attention_mma.cu", "lmsf_attention_prefill",
              [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_void_p, c_int,
               c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_void_p], d)
    rc = f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cache), cache.stride(0), block_size, n_kv_heads,
           _i32(block_table, "block_table"), block_table.shape[1], _i32(tile_seq, "tile_seq"),
           _i32(tile_q0, "tile_q0"), n_tiles, _i32(cu_q, "cu_q"), _i32(ctx_len, "ctx_len"), float(scale),
           int(window or 0), n_q_heads, head_dim, _stream())
    _check(rc, "attention_mma.cu", "lmsf_attention_mma", d)


# ----------------------------------------------------------------------------- tcgen05 prefill attention

TC_HEAD_DIMS = (64, 128)
TC_Q_TILE = 128


def tc_attention_supported(dtype: torch.dtype, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and head_dim in TC_HEAD_DIMS


def attention_prefill_tc(out: torch.Tensor, q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                         block_size: int, tile_seq: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int, cu_q: torch.Tensor,
                         ctx_len: torch.Tensor, scale: float, window: int, n_q_heads: int, n_kv_heads: int, head_dim: int,
                         error_flag: Optional[torch.Tensor] = None):
    """Attention of prompt portions on tcgen05 tensor cores (head size 64 or 128).  Tile i covers the query
    tokens tile_q0[i] .. tile_q0[i] + 127 (counted inside the portion) of request tile_seq[i]."""
    _check_paged(q, out, cache, n_q_heads, n_kv_heads, head_dim, block_size, "attention_prefill_tc")
    d = _mma_defines(head_dim)[:1]
    f = _func("attention_tc.cu", "lmsf_attention_prefill_tc",
              [c_void_p, c_longlong, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_longlong, c_int, c_int,
               c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_void_p,
               c_void_p], d)
    rc = f(_ptr(q), q.stride(0), q.shape[0], _ptr(out), out.stride(0), _ptr(cache), cache.stride(0), cache.shape[0], block_size,
           n_kv_heads, _i32(block_table, "block_table"), block_table.shape[1], _i32(tile_seq, "tile_seq"),
           _i32(tile_q0, "tile_q0"), n_tiles, _i32(cu_q, "cu_q"), _i32(ctx_len, "ctx_len"), float(scale),
           int(window or 0), n_q_heads, head_dim, _i32(error_flag, "error_flag"), _stream())
    _check(rc, "attention_tc.cu", "lmsf_attention_tc", d)
