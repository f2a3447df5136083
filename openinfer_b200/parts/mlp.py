"""Gated feed-forward: down( act(gate x) * (up x) ), act chosen by the spec ("silu": SwiGLU, the
reference's; "gelu_tanh": the tanh form of GELU).

gate and up are one fused [2*intermediate, hidden] matrix, as in the reference
(pegainfer-qwen3/src/weights/load.rs:136-154), so one product feeds the activation kernel
(pegainfer-qwen3/src/unified_forward.rs:557-595).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import gemm_tcgen05, native, ops
from ..kernels import lib as _lib
from ..kernels.linear import ensure_library
from .base import FeedForward
from .registry import register_feed_forward
from .spec import GatedMlpSpec, ParamInfo



@register_feed_forward("gated_mlp")
class GatedMlp(FeedForward):
    def __init__(self, spec: GatedMlpSpec) -> None:
        super().__init__(spec)
        self.act_code = ops.act_code(spec.activation)   # refuses a name no kernel knows; the kernels take the code
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
        """One native call (``oi_gated_mlp``): it picks, by the step's rows, the product that forms the activation in
        its epilogue (tcgen05 tiles from 128 rows, the weight stream up to 32) or the plain product and the
        stand-alone activation kernel, then the down projection."""
        s = self.spec
        M, inter = x.shape[0], s.intermediate_size
        L = _lib.load()
        codes = native.DTYPE_CODE
        if not x.is_contiguous():
            x = x.contiguous()
        if M > 32:
            ensure_library(x.device)
        out = torch.empty((M, s.hidden_size), dtype=x.dtype, device=x.device)
        act = torch.empty((M, inter), dtype=x.dtype, device=x.device)
        gate_up = None
        if L.oi_gated_mlp_needs_gate_up(codes[x.dtype], codes[self.w_gate_up.dtype], M, s.hidden_size, inter, self.block):
            gate_up = torch.empty((M, 2 * inter), dtype=x.dtype, device=x.device)
        _lib.check(L.oi_gated_mlp(out.data_ptr(), x.data_ptr(), codes[x.dtype], M, s.hidden_size, inter,
                                  self.w_gate_up.data_ptr(), codes[self.w_gate_up.dtype], self.w_down.data_ptr(),
                                  codes[self.w_down.dtype], self.act_code, self.block, act.data_ptr(), 0 if gate_up is None else gate_up.data_ptr(),
                                  _lib.current_stream()), "gated_mlp")
        return out
