"""Block arrangements. "prenorm": norm -> mixer -> add, norm -> feed-forward -> add
(pegainfer-qwen3/src/unified_forward.rs:383-611). Each residual add is carried out by
the norm that follows it (the reference fuses the same way: flashinfer_norm.cu:39-132,
pegainfer-qwen3/src/batch_decode.rs:210-236)."""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .base import Block, CacheBinding, Part
from .registry import build_feed_forward, build_mixer, build_norm, register_block
from .spec import BlockSpec


@register_block("prenorm")
class PreNormBlock(Block):
    def __init__(self, spec: BlockSpec) -> None:
        super().__init__(spec)
        self._mixer = build_mixer(spec.mixer)
        self.feed_forward = build_feed_forward(spec.feed_forward)
        self.input_norm = build_norm(spec.input_norm)
        self.post_norm = build_norm(spec.post_norm)

    @property
    def mixer(self):
        return self._mixer

    def sub_parts(self) -> Dict[str, Part]:
        s = self.spec
        return {
            s.input_norm_name: self.input_norm,
            s.mixer_name: self._mixer,
            s.post_norm_name: self.post_norm,
            s.feed_forward_name: self.feed_forward,
        }

    def forward(self, h: torch.Tensor, pending: Optional[torch.Tensor], ctx,
                binding: CacheBinding) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        x = self.input_norm(h, delta=pending)          # h += pending; x = norm(h)
        a = self._mixer.forward(x, ctx, binding)
        x = self.post_norm(h, delta=a)                 # h += a; x = norm(h)
        m = self.feed_forward.forward(x, ctx)
        return h, m
