"""Gated feed-forward: down( act(gate x) * (up x) ), act chosen by the spec ("silu": SwiGLU, the
reference's; "gelu_tanh": the tanh form of GELU).

gate and up are one fused [2*intermediate, hidden] matrix, as in the reference
(pegainfer-qwen3/src/weights/load.rs:136-154), so one product feeds the activation kernel
(pegainfer-qwen3/src/unified_forward.rs:557-595).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import gemm_tcgen05, ops, policy
from ..kernels.linear import gate_up_silu_mul, linear, linear_silu_mul
from .base import FeedForward
from .registry import register_feed_forward
from .spec import GatedMlpSpec, ParamInfo

# rows from which the gate/up product with the activation in its epilogue is used (prompt portions)
FUSED_MIN_ROWS = 128


@register_feed_forward("gated_mlp")
class GatedMlp(FeedForward):
    def __init__(self, spec: GatedMlpSpec) -> None:
        super().__init__(spec)
        ops.act_code(spec.activation)      # refuses a name no kernel knows; the kernels take the code as an argument
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
        inter = self.spec.intermediate_size
        # Rows of the fused matrix: blocks of `block` gate rows followed by the up rows of the same
        # indices. With block = 64 a 128-row tile of the tensor-core products holds a gate block and
        # its up block side by side, and the activation is formed in those kernels' epilogues.
        self.block = gemm_tcgen05.ACT_BLOCK if (g.dtype == torch.bfloat16 and inter % gemm_tcgen05.ACT_BLOCK == 0) else inter
        nb = inter // self.block
        self.w_gate_up = torch.stack([g.view(nb, self.block, -1), u.view(nb, self.block, -1)], dim=1).reshape(2 * inter, -1).contiguous()
        self.w_down = tensors["down_proj.weight"].contiguous()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        inter = self.spec.intermediate_size
        if self.block == gemm_tcgen05.ACT_BLOCK and x.dtype == torch.bfloat16:
            if (x.shape[0] >= FUSED_MIN_ROWS or policy.batch_invariant()) and inter % (2 * gemm_tcgen05.ACT_BLOCK) == 0:
                act = torch.empty((x.shape[0], inter), dtype=x.dtype, device=x.device)
                if gemm_tcgen05.takes(act, x, self.w_gate_up):
                    tile = 256 if policy.batch_invariant() else gemm_tcgen05.portion_tile(x.shape[0], x.shape[1])
                    gemm_tcgen05.gemm_silu_mul(act, x, self.w_gate_up, tile, self.spec.activation)
                    return linear(act, self.w_down)
            else:
                act = gate_up_silu_mul(x, self.w_gate_up, self.spec.activation)     # decode: the weight stream forms the activation
                if act is not None:
                    return linear(act, self.w_down)
        gate_up = linear(x, self.w_gate_up)
        return linear_silu_mul(gate_up, self.w_down, self.block, self.spec.activation)
