"""Position encodings applied to queries and keys inside a mixer.

A position encoding is anything that can be given as a rotation table per position:
``rotation_tables`` returns float32 cos/sin [max_positions, rotary_dim/2], and the
fused kernel rotates the pair (d, d + rotary_dim/2) of each head with them (or, with the spec's
``interleaved``, the neighbours (2 d, 2 d + 1)). Scaled or
partial rotary variants only change the table; "none" returns no table.

"rope" is the reference's rotate-half encoding over the full head:
inv_freq[i] = 1 / theta^(2i / rotary_dim), angle = pos * inv_freq[i], both in float32
(pegainfer-core/src/weight_loader.rs:730-764). The reference rounds the table to
bfloat16; here it stays float32.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .base import PositionEncoding
from .registry import register_position_encoding
from .spec import PositionSpec

# tables are shared by all layers with the same constants on a device
_TABLES: Dict[Tuple, Tuple[torch.Tensor, torch.Tensor]] = {}


@register_position_encoding("rope")
class RotaryEncoding(PositionEncoding):
    def __init__(self, spec: PositionSpec) -> None:
        super().__init__(spec)
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {spec.rotary_dim}")
        if spec.max_positions <= 0:
            raise ValueError("max_positions must be positive")

    def rotation_tables(self, device: torch.device):
        s = self.spec
        key = (s.rotary_dim, float(s.theta), s.max_positions, str(device))
        if key not in _TABLES:
            half = s.rotary_dim // 2
            idx = torch.arange(half, dtype=torch.float32)
            inv_freq = 1.0 / torch.pow(torch.tensor(float(s.theta), dtype=torch.float32),
                                       idx * 2.0 / s.rotary_dim)
            ang = torch.arange(s.max_positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
            _TABLES[key] = (torch.cos(ang).contiguous().to(device), torch.sin(ang).contiguous().to(device))
        return _TABLES[key]


@register_position_encoding("none")
class NoPositionEncoding(PositionEncoding):
    def rotation_tables(self, device: torch.device) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        return None
