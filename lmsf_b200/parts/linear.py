"""Dense projections y = x W^T (+ b where the model has biases), weight stored [out, in] as in the checkpoint.

The reference's linear family (core/src/model_executor/layers/linear.rs:28-106, :325-497, :499-728)
wraps cuBLASLt and merges q, k, v (and gate, up) into one matrix by row ranges; the same merged
layouts are used here.  bfloat16 products of more than 16 rows go to the library (cuBLAS through torch.mm),
the place where the reference calls a library too; products of up to 16 rows (decode steps) run on
this package's weight-streaming kernel (csrc/gemm_skinny.cu); float32 products run on this package's own FFMA kernel so
that no reduced-precision mode can slip in and a row's result does not depend on the batch.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Union

import torch

from .. import kernels
from .base import NormAfter, Part, Prenormed, WeightSpec, register_part

# Library products must add up in float32: with torch's default a split-k bfloat16 product may add its partial sums
# in bfloat16, and a row's result would then depend on how many rows share the product (on how a prompt was cut).
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

_MM_HAS_OUT_DTYPE: Optional[bool] = None
USE_SKINNY = True     # bfloat16 products of up to 16 rows run on this package's weight-streaming kernel
SKINNY_TALL_FROM = 65536   # ... except 9 to 16 rows against this many output features and more


def _skinny_takes(x: torch.Tensor, w: torch.Tensor) -> bool:
    # (9 to 16 rows against a very tall matrix, the head: a stage of the kernel then holds as much of x as of w, and the
    # library is faster: 162 against 182 us for 128,256 x 4,096 at 16 rows)
    return USE_SKINNY and kernels.gemm_skinny_supported(x, w) and not (x.shape[0] > 8 and w.shape[0] >= SKINNY_TALL_FROM)


def matmul_tn(x: Union[torch.Tensor, Prenormed], w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
              bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [M, K] times w [N, K] transposed -> [M, N] in `out_dtype` (default: x's dtype), plus `bias` [N] if given
    (added by a kernel of its own after the product, as the reference adds it: layers/linear.rs:100-104).  x may be a
    `Prenormed`: the weight-streaming kernel divides its sums by the rows' root mean square."""
    if isinstance(x, Prenormed):
        dt = out_dtype or x.x.dtype
        if _skinny_takes(x.x, w) and dt in (torch.bfloat16, torch.float32):
            y = torch.empty((x.x.shape[0], w.shape[0]), dtype=dt, device=w.device)
            kernels.gemm_skinny(y, x.x, w, prenorm=(x.sumsq, x.eps, x.width))
        else:
            y = _product_tn(x.norm.finish(x), w, out_dtype)
    else:
        y = _product_tn(x, w, out_dtype)
    if bias is not None:
        kernels.bias_add(y, bias if bias.dtype == y.dtype else bias.to(y.dtype))
    return y


def _product_tn(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    global _MM_HAS_OUT_DTYPE
    out_dtype = out_dtype or x.dtype
    if x.dtype == torch.float32:
        out = torch.empty((x.shape[0], w.shape[0]), dtype=torch.float32, device=x.device)
        kernels.gemm_tn_simt(out, x, w)
        return out if out_dtype == torch.float32 else out.to(out_dtype)
    if _skinny_takes(x, w) and out_dtype in (torch.bfloat16, torch.float32):
        out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=x.device)
        kernels.gemm_skinny(out, x, w)
        return out
    if out_dtype == x.dtype:
        return torch.mm(x, w.t())
    if _MM_HAS_OUT_DTYPE is not False:
        try:
            y = torch.mm(x, w.t(), out_dtype=out_dtype)
            _MM_HAS_OUT_DTYPE = True
            return y
        except (TypeError, RuntimeError):
            if _MM_HAS_OUT_DTYPE:
                raise
            _MM_HAS_OUT_DTYPE = False
    out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=x.device)
    kernels.gemm_tn_simt(out, x, w)
    return out


def matmul_tn_residual(x: torch.Tensor, w: torch.Tensor, then: NormAfter) -> Optional[Prenormed]:
    """The product before a norm, for a few rows: then.res += x w^T, and the first half of then.norm on the new
    residual.  None when this product cannot do it (the caller then multiplies as usual and the norm runs whole)."""
    norm, res = then.norm, then.res
    weight = getattr(norm, "weight", None)
    if not (norm.splittable and _skinny_takes(x, w) and weight is not None and res.dtype == torch.float32
            and res.shape == (x.shape[0], w.shape[0]) and res.is_contiguous() and weight.shape == (w.shape[0],)):
        return None
    parts = kernels.gemm_skinny_residual_parts(w.shape[0])
    sumsq = torch.empty((x.shape[0], (parts + 3) // 4 * 4), dtype=torch.float32, device=x.device)[:, :parts]
    xg = torch.empty((x.shape[0], w.shape[0]), dtype=torch.bfloat16, device=x.device)
    kernels.gemm_skinny_residual(xg, x, w, res, weight, sumsq)
    return Prenormed(xg, sumsq, norm.eps, w.shape[0], norm, res)


@register_part("linear", "dense")
class Linear(Part):
    """out_features may be a list: the sources are stacked along the output dimension."""
    graph_safe = True

    def __init__(self, in_features: int, out_features: Union[int, Sequence[int]], out_dtype: Optional[str] = None,
                 bias: bool = False):
        self.in_features = int(in_features)
        self.has_bias = bool(bias)
        self.bias: Optional[torch.Tensor] = None
        self.out_splits: List[int] = [int(out_features)] if isinstance(out_features, int) else [int(o) for o in out_features]
        self.out_features = sum(self.out_splits)
        self.out_dtype = {None: None, "float32": torch.float32, "bfloat16": torch.bfloat16}[out_dtype]
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {"weight": WeightSpec([(o, self.in_features) for o in self.out_splits])}
        if self.has_bias:
            specs["bias"] = WeightSpec([(o,) for o in self.out_splits])
        return specs

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return matmul_tn(x, self.weight, self.out_dtype, self.bias)
