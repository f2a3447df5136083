"""Gated feed-forward (SwiGLU): down( act(gate x) * (up x) ).

gate and up are one fused [2*intermediate, hidden] matrix, as in the reference
(pegainfer-qwen3/src/weights/load.rs:136-154), so one product feeds the activation kernel
(pegainfer-qwen3/src/unified_forward.rs:557-595).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels.linear import linear, linear_silu_mul
from .base import FeedForward
from .registry import register_feed_forward
from .spec import GatedMlpSpec, ParamInfo


@register_feed_forward("gated_mlp")
class GatedMlp(FeedForward):
    def __init__(self, spec: GatedMlpSpec) -> None:
        super().__init__(spec)
        if spec.activation != "silu":
            raise ValueError(f"activation {spec.activation!r} has no kernel (silu only)")
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamInfo]:
        s = self.spec
        return {
            "gate_proj.weight": ParamInfo((s.intermediate_size, s.hidden_size)),
            "up_proj.weight": ParamInfo((s.intermediate_size, s.hidden_size)),
            "down_proj.weight": ParamInfo((s.hidden_size, s.intermediate_size)),
        }

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        if g.dtype != u.dtype:
            raise ValueError("gate_proj and up_proj must be stored in one dtype to be fused")
        self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"].contiguous()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        gate_up = linear(x, self.w_gate_up)
        return linear_silu_mul(gate_up, self.w_down)
