"""Interfaces of the parts a layer is made of.

A part owns its parameters and knows its sizes and constants from its spec; it does
not know which model it is in. All of them work on flattened rows: ``x`` is
``[tokens, hidden]`` for the whole batch of a step, and everything about which row
belongs to which request, at which position, lives in the ``StepContext``.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Tuple

import torch

from ..cache.manager import KvHandle, KvNeed, StateNeed
from .spec import ParamInfo


@dataclasses.dataclass(frozen=True)
class CacheBinding:
    """What one call of a block (one entry of the run order) holds in the cache manager.

    ``kv`` is the page group and layer the mixer reads; ``owns_kv`` is False when the
    entry reads the cache of an earlier call and must not write. ``states`` are the
    ids of its per-request state tensors, in the order of ``Mixer.state_needs()``.
    """

    kv: Optional[KvHandle] = None
    owns_kv: bool = True
    states: Tuple[int, ...] = ()


class Part:
    """Base of all parts: named parameters, loaded once."""

    def __init__(self, spec) -> None:
        self.spec = spec

    def parameters(self) -> Dict[str, ParamInfo]:
        """Local tensor name -> what is expected of it. The checkpoint name is the
        prefix the enclosing block gives this part, followed by the local name."""
        return {}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Take the tensors named by ``parameters()`` (already on the device, in the
        dtype the loader settled). May fuse or re-lay them out."""

    def prepare(self, device: torch.device, dtype: torch.dtype) -> None:
        """Build what is derived rather than loaded (tables), once, after ``load``."""


class Norm(Part):
    def __call__(self, x: torch.Tensor, *, delta: Optional[torch.Tensor] = None,
                 row_idx: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Normalised rows. ``delta``: x <- x + delta first (x is updated in place).
        ``row_idx``: only these rows of x, in this order (x is then left as it is)."""
        raise NotImplementedError


class Mixer(Part):
    """Mixes information across positions of a request (attention, a recurrence, ...)."""

    # True when ``forward`` reads the step's metadata only through the context's DEVICE
    # tensors, so that a recorded launch sequence (a CUDA graph) can be replayed for another
    # step of the same shape. A mixer that reads the host lists must leave this False.
    graph_safe = False

    def kv_need(self) -> Optional[KvNeed]:
        """Paged keys and values this mixer wants, or None."""
        return None

    def state_needs(self) -> List[StateNeed]:
        """Per-request state tensors of fixed size this mixer wants."""
        return []

    def forward(self, x: torch.Tensor, ctx, binding: CacheBinding) -> torch.Tensor:
        """[tokens, hidden] -> [tokens, hidden]. Must only depend, for a row, on earlier
        rows of the same request in this step and on what earlier steps left in the
        cache / state of that request."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def rotation_tables(self, device: torch.device):
        """(cos, sin) float32 tables [max_positions, rotary_dim / 2], or None when queries
        and keys are not rotated."""
        raise NotImplementedError


class Block(Part):
    """One layer: arranges a mixer, a feed-forward and norms around the residual stream.

    The residual stream travels as a pair (h, pending): ``pending`` is a branch output
    not yet added to ``h``; the next norm adds it while it reads the row (one pass over
    memory instead of two). ``forward`` returns the new pair.
    """

    def forward(self, h: torch.Tensor, pending: Optional[torch.Tensor], ctx,
                binding: CacheBinding) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        raise NotImplementedError

    def sub_parts(self) -> Dict[str, Part]:
        """Tensor-name prefix (relative to the block's own name) -> part."""
        return {}

    @property
    def mixer(self) -> Optional[Mixer]:
        return None
