"""RMSNorm part: out = x * rsqrt(mean(x^2) + eps) * (weight_offset + weight).

The reference's layer norms, per-head norms and final norm are all this operation with
the weight used as stored (pegainfer-kernels/csrc/shared/flashinfer_norm.cu:170-187); the
offset is a parameter so that a "1 + w" convention is a spec constant, not new code.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from .base import Norm
from .registry import register_norm
from .spec import NormSpec, ParamInfo


@register_norm("rms")
class RmsNorm(Norm):
    def __init__(self, spec: NormSpec) -> None:
        super().__init__(spec)
        self.weight: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamInfo]:
        return {"weight": ParamInfo((self.spec.size,), ("one_plus_normal", 0.02))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()

    def __call__(self, x: torch.Tensor, *, delta: Optional[torch.Tensor] = None,
                 row_idx: Optional[torch.Tensor] = None) -> torch.Tensor:
        rows = x.shape[0] if row_idx is None else row_idx.numel()
        out = torch.empty((rows, x.shape[1]), dtype=x.dtype, device=x.device)
        return ops.rmsnorm(out, x, self.weight, self.spec.eps, delta=delta, row_idx=row_idx,
                           weight_offset=self.spec.weight_offset)
