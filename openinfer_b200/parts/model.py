"""A model assembled from a ``ModelSpec``: embedding, blocks run in the spec's order,
final norm, head. It knows nothing about the architecture the spec came from.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..cache.manager import CacheManager
from ..kernels import ops
from ..kernels.linear import linear
from .base import Block, CacheBinding
from .registry import build_block, build_norm
from .spec import LayerCall, ModelSpec, ParamInfo


class Model:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype) -> None:
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"model dtype must be float32 or bfloat16, got {dtype}")
        self.spec = spec
        self.dtype = dtype
        self.blocks: List[Block] = [build_block(b) for b in spec.blocks]
        self.final_norm = build_norm(spec.final_norm)
        self.calls: List[LayerCall] = spec.calls()
        for i, c in enumerate(self.calls):
            if not (0 <= c.layer < len(self.blocks)):
                raise ValueError(f"run order entry {i} names layer {c.layer}, of {len(self.blocks)}")
            if c.read_cache_of is not None:
                if not (0 <= c.read_cache_of < i):
                    raise ValueError(f"run order entry {i} reads the cache of entry {c.read_cache_of}, which is not earlier")
                if self.calls[c.read_cache_of].read_cache_of is not None:
                    raise ValueError(f"run order entry {i} reads the cache of an entry that owns none")
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self.bindings: List[CacheBinding] = []
        self.device: Optional[torch.device] = None

    # ------------------------------------------------------------------ tensors
    def expected_tensors(self) -> Dict[str, ParamInfo]:
        s = self.spec
        out: Dict[str, ParamInfo] = {s.embedding_name: ParamInfo((s.vocab_size, s.hidden_size))}
        for block, bspec in zip(self.blocks, s.blocks):
            for prefix, part in block.sub_parts().items():
                for local, info in part.parameters().items():
                    out[bspec.name + prefix + local] = info
        for local, info in self.final_norm.parameters().items():
            out[s.final_norm_name + local] = info
        if s.head_name is not None:
            out[s.head_name] = ParamInfo((s.vocab_size, s.hidden_size))
        return out

    def load(self, tensors: Dict[str, torch.Tensor], device: torch.device) -> None:
        """Hand every part its tensors (already on ``device``), then build derived tables."""
        s = self.spec
        self.device = torch.device(device)
        self.embedding = tensors[s.embedding_name].contiguous()
        self.head = self.embedding if s.head_name is None else tensors[s.head_name].contiguous()
        for block, bspec in zip(self.blocks, s.blocks):
            for prefix, part in block.sub_parts().items():
                full = bspec.name + prefix
                part.load({local: tensors[full + local] for local in part.parameters()})
                part.prepare(self.device, self.dtype)
        self.final_norm.load({local: tensors[s.final_norm_name + local] for local in self.final_norm.parameters()})

    def weight_bytes(self) -> int:
        """Bytes of the tensors a decode step reads once (the embedding table only when it
        is also the head)."""
        seen, total = set(), 0

        def add(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()

        add(self.head)
        for block in self.blocks:
            for part in block.sub_parts().values():
                for v in vars(part).values():
                    if isinstance(v, torch.Tensor):
                        add(v)
        add(getattr(self.final_norm, "weight", None))
        return total

    # ------------------------------------------------------------------ cache
    def bind_cache(self, cache: CacheManager) -> None:
        """Register what every entry of the run order needs from the cache manager."""
        self.bindings = []
        for c in self.calls:
            mixer = self.blocks[c.layer].mixer
            if mixer is None:
                self.bindings.append(CacheBinding())
                continue
            if c.read_cache_of is not None:
                src = self.bindings[c.read_cache_of]
                if src.kv is None:
                    raise ValueError("run order entry reads the cache of an entry without keys and values")
                src_need = self.blocks[self.calls[c.read_cache_of].layer].mixer.kv_need()
                need = mixer.kv_need()
                if need is None or (need.num_kv_heads, need.head_dim) != (src_need.num_kv_heads, src_need.head_dim):
                    raise ValueError("a layer can only read the cache of a layer with the same kv heads and head size")
                kv, owns = src.kv, False
            else:
                need = mixer.kv_need()
                kv, owns = (cache.add_kv_layer(need) if need is not None else None), True
            states = tuple(cache.add_state(n) for n in mixer.state_needs())
            self.bindings.append(CacheBinding(kv=kv, owns_kv=owns, states=states))

    # ------------------------------------------------------------------ forward
    def forward(self, ctx) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """Run all rows of the step through the blocks. Returns the residual stream as
        (h, pending): pending is the last branch output, not yet added."""
        h = torch.empty((ctx.num_tokens, self.spec.hidden_size), dtype=self.dtype, device=self.device)
        ops.embedding(h, self.embedding, ctx.token_ids)
        if self.spec.embedding_scale != 1.0:
            ops.scale_cap(h, scale=self.spec.embedding_scale)
        pending = None
        for call, binding in zip(self.calls, self.bindings):
            h, pending = self.blocks[call.layer].forward(h, pending, ctx, binding)
        return h, pending

    def logits(self, h: torch.Tensor, pending: Optional[torch.Tensor], row_idx: torch.Tensor) -> torch.Tensor:
        """Float32 logits [rows, vocab] of the wanted rows only: gather + final norm in one
        kernel, then the head (pegainfer-qwen3/src/prefill.rs:440-477)."""
        x = self.final_norm(h, delta=pending, row_idx=row_idx)
        out = linear(x, self.head, out_dtype=torch.float32)
        if self.spec.logit_soft_cap > 0.0:
            ops.scale_cap(out, cap=self.spec.logit_soft_cap)
        return out
