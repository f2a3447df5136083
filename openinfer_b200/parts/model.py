"""A model assembled from a ``ModelSpec``: embedding, blocks run in the spec's order,
final norm, head. It knows nothing about the architecture the spec came from.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

import ctypes
import os

from ..cache.manager import CacheManager
from ..kernels import attention as attn_kernels
from ..kernels import lib as _lib
from ..kernels import native, ops
from ..kernels.linear import ensure_library, linear
from .base import Block, CacheBinding
from .registry import build_block, build_norm
from .spec import LayerCall, ModelSpec, ParamInfo

# A model whose every part is one of this package's own runs all layers of a step in ONE native call (oi_forward).
# Off (OI_NATIVE_STEP=0, or ``Model.native_step = False``): the parts are called one by one from Python, which is
# also what a model with a registered part of its own does. Both launch the same kernels with the same arguments.
NATIVE_STEP = os.environ.get("OI_NATIVE_STEP", "1") != "0"


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
        self.native_step = NATIVE_STEP
        self._native = None          # (ModelDesc, what it points to), made at the first step
        self._native_checked = False

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

    def run(self, ctx, row_idx: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """All rows of the step through the model; float32 logits of the rows ``row_idx`` names (None: none wanted)."""
        desc = self._native_description(ctx) if self.native_step else None
        if desc is not None:
            return self._run_native(desc, ctx, row_idx)
        h, pending = self.forward(ctx)
        return self.logits(h, pending, row_idx) if row_idx is not None else None

    # ------------------------------------------------------------------ the native step
    def _native_description(self, ctx):
        """The model as the native step sees it (csrc/oi_api.h, OiModelDesc), or None if some part is not one of
        this package's own. Pointers to the weights and to every layer's pages: made once, when the cache stands."""
        if self._native_checked:
            return self._native
        self._native_checked = True
        from .attention import Attention
        from .block import PreNormBlock
        from .mlp import GatedMlp
        from .norm import RmsNorm

        def own(obj, cls):
            return type(obj) is cls

        if not own(self.final_norm, RmsNorm) or not all(
                own(b, PreNormBlock) and own(b.mixer, Attention) and own(b.feed_forward, GatedMlp)
                and own(b.input_norm, RmsNorm) and own(b.post_norm, RmsNorm) for b in self.blocks):
            return None
        codes = native.DTYPE_CODE
        cache = ctx.cache
        layers = (native.LayerDesc * len(self.calls))()
        keys: List[tuple] = []        # distinct attention geometries: a step plans each once
        reps: List[tuple] = []        # (call index) that stands for each geometry
        for i, (call, binding) in enumerate(zip(self.calls, self.bindings)):
            b = self.blocks[call.layer]
            at, ff, s = b.mixer, b.feed_forward, b.mixer.spec
            k_cache, v_cache, page_stride = cache.kv_views(binding.kv)
            qkv_rows = at.q_dim + 2 * at.kv_dim if binding.owns_kv else at.q_dim
            cos, sin = at.tables if at.tables is not None else (None, None)
            key = (binding.kv.group, s.num_heads, s.num_kv_heads, s.head_dim, s.window, qkv_rows, cos is not None,
                   None if at.q_norm_w is None else at.q_norm_w.dtype)
            if key not in keys:
                keys.append(key)
                reps.append(i)
            qn = s.qk_norm
            L = layers[i]
            L.input_norm_w, L.input_norm_dtype = b.input_norm.weight.data_ptr(), codes[b.input_norm.weight.dtype]
            L.input_eps, L.input_offset = b.input_norm.spec.eps, b.input_norm.spec.weight_offset
            L.post_norm_w, L.post_norm_dtype = b.post_norm.weight.data_ptr(), codes[b.post_norm.weight.dtype]
            L.post_eps, L.post_offset = b.post_norm.spec.eps, b.post_norm.spec.weight_offset
            L.w_qkv, L.w_qkv_dtype, L.qkv_rows = at.w_qkv.data_ptr(), codes[at.w_qkv.dtype], qkv_rows
            L.w_o, L.w_o_dtype = at.w_o.data_ptr(), codes[at.w_o.dtype]
            L.w_gate_up, L.w_gate_up_dtype = ff.w_gate_up.data_ptr(), codes[ff.w_gate_up.dtype]
            L.w_down, L.w_down_dtype = ff.w_down.data_ptr(), codes[ff.w_down.dtype]
            L.inter, L.act, L.act_block = ff.spec.intermediate_size, ff.act_code, ff.block
            L.attn_step = keys.index(key)
            a = L.attn
            a.k_cache, a.v_cache = k_cache.data_ptr(), v_cache.data_ptr()
            a.q_norm_w = 0 if at.q_norm_w is None else at.q_norm_w.data_ptr()
            a.k_norm_w = 0 if at.k_norm_w is None else at.k_norm_w.data_ptr()
            a.norm_dtype = 0 if at.q_norm_w is None else codes[at.q_norm_w.dtype]
            a.cos_tab, a.sin_tab = (0, 0) if cos is None else (cos.data_ptr(), sin.data_ptr())
            a.rot_half, a.max_pos = (0, 0) if cos is None else (cos.shape[1], cos.shape[0])
            a.nq, a.nkv, a.hd, a.window = s.num_heads, s.num_kv_heads, s.head_dim, int(s.window) if s.window else 0
            a.scale, a.eps, a.w_offset = s.softmax_scale, (qn.eps if qn else 0.0), (qn.weight_offset if qn else 0.0)
            a.write_kv, a.rope_mode = (1 if binding.owns_kv else 0), 1
            a.interleaved = 1 if getattr(s.position, "interleaved", False) else 0
        sp = self.spec
        desc = native.ModelDesc(
            layers=layers, embedding=self.embedding.data_ptr(), final_norm_w=self.final_norm.weight.data_ptr(),
            head=self.head.data_ptr(), num_layers=len(self.calls), hidden=sp.hidden_size, vocab=sp.vocab_size,
            dtype=codes[self.dtype], embedding_dtype=codes[self.embedding.dtype],
            final_norm_dtype=codes[self.final_norm.weight.dtype], head_dtype=codes[self.head.dtype],
            embedding_scale=sp.embedding_scale, final_eps=self.final_norm.spec.eps,
            final_offset=self.final_norm.spec.weight_offset, logit_soft_cap=sp.logit_soft_cap,
            max_qkv_rows=max(L.qkv_rows for L in layers), max_q_dim=max(L.attn.nq * L.attn.hd for L in layers),
            max_inter=max(L.inter for L in layers))
        desc.keep = layers
        self._native = (desc, keys, reps)
        return self._native

    def _run_native(self, native_desc, ctx, row_idx: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        desc, keys, reps = native_desc
        T, H, dev, dt = ctx.num_tokens, self.spec.hidden_size, self.device, self.dtype
        lib = _lib.load()
        if T > 32:
            ensure_library(dev)

        def buf(cols, dtype=dt, rows=T):
            return torch.empty((rows, cols), dtype=dtype, device=dev)

        h, x, qkv, attn = buf(H), buf(H), buf(desc.max_qkv_rows), buf(desc.max_q_dim)
        branch_a, branch_m, act = buf(H), buf(H), buf(desc.max_inter)
        gate_up = buf(2 * desc.max_inter) if self._gate_up_needed(lib, desc, T) else None
        steps = (native.AttnStep * len(keys))()
        kept = []
        for j, (key, i) in enumerate(zip(keys, reps)):
            call, binding = self.calls[i], self.bindings[i]
            at = self.blocks[call.layer].mixer
            k_cache, _, page_stride = ctx.cache.kv_views(binding.kv)
            L = desc.keep[i]
            cos = at.tables[0] if at.tables is not None else None
            s = attn_kernels.attention_step(ctx, ctx.groups[binding.kv.group], qkv.view(-1)[: T * L.qkv_rows].view(T, L.qkv_rows),
                                            attn.view(-1)[: T * at.q_dim].view(T, at.q_dim), k_cache, page_stride,
                                            L.attn.nq, L.attn.nkv, L.attn.hd, at.spec.window, cos=cos, q_norm_w=at.q_norm_w)
            kept.append(s)
            ctypes.memmove(ctypes.byref(steps[j]), ctypes.byref(s), ctypes.sizeof(native.AttnStep))
        xs = ssq = None
        if T <= 32 and dt == torch.bfloat16:   # decode-sized steps may run without norm kernels inside the layer stack
            xs = buf(H)
            ssq = torch.empty((32, -(-H // 128) * 8), dtype=torch.float32, device=dev)   # [row][tile of 128 columns, K slice]
        n_want = 0 if row_idx is None else row_idx.numel()
        wanted = buf(H, rows=n_want) if n_want else None
        logits = buf(self.spec.vocab_size, dtype=torch.float32, rows=n_want) if n_want else None
        step = native.StepDesc(
            token_ids=ctx.token_ids.data_ptr(), attn_steps=steps, want_rows=row_idx.data_ptr() if n_want else 0,
            h=h.data_ptr(), x=x.data_ptr(), qkv=qkv.data_ptr(), attn=attn.data_ptr(), branch_a=branch_a.data_ptr(),
            branch_m=branch_m.data_ptr(), act=act.data_ptr(), gate_up=0 if gate_up is None else gate_up.data_ptr(),
            wanted=wanted.data_ptr() if n_want else 0, logits=logits.data_ptr() if n_want else 0,
            xs=0 if xs is None else xs.data_ptr(), ssq=0 if ssq is None else ssq.data_ptr(),
            ssq_stride=0 if ssq is None else ssq.stride(0), tokens=T, num_attn_steps=len(keys), num_want=n_want)
        _lib.check(lib.oi_forward(ctypes.byref(desc), ctypes.byref(step), _lib.current_stream()), "forward")
        return logits

    def _gate_up_needed(self, lib, desc, T: int) -> bool:
        """Whether some layer's feed-forward needs the gate|up scratch rows at this step size (asked once per size)."""
        cache = self.__dict__.setdefault("_gate_up_by_rows", {})
        if T not in cache:
            codes = native.DTYPE_CODE
            cache[T] = any(lib.oi_gated_mlp_needs_gate_up(codes[self.dtype], L.w_gate_up_dtype, T, self.spec.hidden_size,
                                                          L.inter, L.act_block) for L in desc.keep)
        return cache[T]

    def logits(self, h: torch.Tensor, pending: Optional[torch.Tensor], row_idx: torch.Tensor) -> torch.Tensor:
        """Float32 logits [rows, vocab] of the wanted rows only: gather + final norm in one
        kernel, then the head (pegainfer-qwen3/src/prefill.rs:440-477)."""
        x = self.final_norm(h, delta=pending, row_idx=row_idx)
        out = linear(x, self.head, out_dtype=torch.float32)
        if self.spec.logit_soft_cap > 0.0:
            ops.scale_cap(out, cap=self.spec.logit_soft_cap)
        return out
