"""y = x W^T for the projections: picks the product kernel by operand types.

* bfloat16 x bfloat16: the tensor-core path. The reference's engine calls the vendor
  library for every projection (pegainfer-kernels/csrc/shared/linear.cu:312-362,
  ``cublasGemmEx`` with float32 accumulation); the same library call stands here until
  a hand-written tcgen05 kernel takes the shape (see ``set_bf16_gemm``).
* anything with a float32 operand: the hand-written float32-accumulate kernel on the
  ordinary pipes (no reduced-precision matrix mode), summed in ascending k.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from . import ops

# hook for a hand-written bf16 kernel: fn(out, x, w) -> bool (True when it took the shape)
_bf16_gemm: Optional[Callable[[torch.Tensor, torch.Tensor, torch.Tensor], bool]] = None


def set_bf16_gemm(fn: Optional[Callable[[torch.Tensor, torch.Tensor, torch.Tensor], bool]]) -> None:
    global _bf16_gemm
    _bf16_gemm = fn


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [M, K] (row stride free), w [N, K] -> [M, N] in ``out_dtype`` (default: x's)."""
    out_dtype = out_dtype or x.dtype
    M, N = x.shape[0], w.shape[0]
    if not x.is_cuda:
        raise ops.KernelError("linear: operands must be on a CUDA device; this package has no CPU path")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    if M == 0:
        return out
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        if _bf16_gemm is not None and _bf16_gemm(out, x, w):
            return out
        if out_dtype == torch.bfloat16:
            torch.mm(x, w.t(), out=out)
        else:
            out.copy_(torch.mm(x, w.t(), out_dtype=out_dtype))
        return out
    return ops.gemm_generic(out, x, w)
