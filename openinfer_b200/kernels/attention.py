"""Dispatch of paged attention to the kernel that takes the shape.

The general kernel (one warp per token and head) takes every supported shape in both
storage types; tuned kernels register themselves for the shapes they cover. A shape no
kernel takes raises, it never computes something else.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops


def paged_attention(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    page_stride: int, ctx, group, nq: int, nkv: int, hd: int, scale: float,
                    window: Optional[int], rope: Optional["RopeFusion"] = None) -> torch.Tensor:
    """q [tokens, nq*hd] (row stride free) -> out [tokens, nq*hd], over the pages that
    ``group.block_table`` lists for each request of the step. With ``rope`` (only after
    ``decode_takes_rope`` said yes) q is the RAW fused projection and the decode kernel does the
    q/k norm, the rotation and the cache write itself."""
    if rope is None:
        for impl in _TUNED:
            if impl(q, out, k_cache, v_cache, page_stride, ctx, group, nq, nkv, hd, scale, window):
                return out
    step = attention_step(ctx, group, q, out, k_cache, page_stride, nq, nkv, hd, window,
                          cos=rope.cos if rope is not None else None, q_norm_w=rope.q_norm_w if rope is not None else None)
    if rope is not None:
        if not step.fuse_rope:
            raise ops.KernelError("paged_attention: the fused rotation was promised and then refused")
        mine = native.AttnStep()          # the caller's own positions and slots, not the step's
        ctypes.memmove(ctypes.byref(mine), ctypes.byref(step), ctypes.sizeof(native.AttnStep))
        mine.positions, mine.slot_mapping = rope.positions.data_ptr(), rope.slots.data_ptr()
        mine.keep = (step, rope)
        step = mine
    layer = attention_layer(q, out, k_cache, v_cache, nq, nkv, hd, scale, window,
                            q_norm_w=rope.q_norm_w if rope else None, k_norm_w=rope.k_norm_w if rope else None,
                            eps=rope.eps if rope else 0.0, weight_offset=rope.weight_offset if rope else 0.0,
                            cos=rope.cos if rope else None, sin=rope.sin if rope else None,
                            write_kv=bool(rope.write_kv) if rope else False, rope_mode=1 if rope else 0)
    run_attention(step, layer)
    return out


def run_attention(step: "native.AttnStep", layer: "native.AttnLayer") -> None:
    """One layer's attention in native code (``oi_attention_layer``): the norm + rotation + cache write kernel when the
    layer asks for it and the decode kernel does not do that itself, then the kernel(s) that take the step's shape."""
    _lib.check(_lib.load().oi_attention_layer(ctypes.byref(step), ctypes.byref(layer), _lib.current_stream()), "attention")


def attention_layer(qkv: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, nq: int, nkv: int,
                    hd: int, scale: float, window: Optional[int], *, q_norm_w=None, k_norm_w=None, eps: float = 0.0,
                    weight_offset: float = 0.0, cos=None, sin=None, write_kv: bool = True, rope_mode: int = 1,
                    interleaved: bool = False) -> "native.AttnLayer":
    """The description of one layer's attention call (csrc/oi_api.h, OiAttnLayer)."""
    _check_layer_operands(qkv, out, k_cache, v_cache, q_norm_w, k_norm_w, cos, sin, hd)
    norm_dtype = 0
    if q_norm_w is not None:
        norm_dtype = 1 if q_norm_w.dtype == torch.bfloat16 else 0
    return native.AttnLayer(
        qkv=qkv.data_ptr(), out=out.data_ptr(), k_cache=k_cache.data_ptr(), v_cache=v_cache.data_ptr(),
        q_norm_w=0 if q_norm_w is None else q_norm_w.data_ptr(), k_norm_w=0 if k_norm_w is None else k_norm_w.data_ptr(),
        cos_tab=0 if cos is None else cos.data_ptr(), sin_tab=0 if sin is None else sin.data_ptr(),
        q_row_stride=qkv.stride(0), out_row_stride=out.stride(0), dtype=native.DTYPE_CODE[qkv.dtype],
        nq=nq, nkv=nkv, hd=hd, window=int(window) if window else 0, scale=float(scale), eps=float(eps),
        w_offset=float(weight_offset), norm_dtype=norm_dtype, rot_half=0 if cos is None else cos.shape[1],
        max_pos=0 if cos is None else cos.shape[0], interleaved=1 if interleaved else 0, write_kv=1 if write_kv else 0,
        rope_mode=rope_mode)


def _check_layer_operands(qkv, out, k_cache, v_cache, q_norm_w, k_norm_w, cos, sin, hd) -> None:
    for t in (qkv, out, k_cache, v_cache, q_norm_w, k_norm_w, cos, sin):
        if t is not None and not t.is_cuda:
            raise ops.KernelError("a kernel was given a tensor that is not on a CUDA device; this package has no CPU path")
    if qkv.dtype not in native.DTYPE_CODE or out.dtype != qkv.dtype or k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype:
        raise ops.KernelError(f"attention: q, out and the cache must share one dtype (float32 or bfloat16), got "
                              f"{qkv.dtype}, {out.dtype}, {k_cache.dtype}")
    if qkv.stride(1) != 1 or out.stride(1) != 1:
        raise ops.KernelError("attention: q and out must be contiguous along the head dimension")
    if (q_norm_w is None) != (k_norm_w is None):
        raise ops.KernelError("attention: q and k norm weights come together or not at all")
    for w in (q_norm_w, k_norm_w):
        if w is not None and (w.numel() != hd or not w.is_contiguous() or w.dtype not in native.DTYPE_CODE):
            raise ops.KernelError("attention: a norm weight must have head_dim contiguous float32 or bfloat16 elements")
    if q_norm_w is not None and q_norm_w.dtype != k_norm_w.dtype:
        raise ops.KernelError("attention: q and k norm weights must share a dtype")
    if cos is not None and (cos.dtype != torch.float32 or sin is None or sin.shape != cos.shape
                            or not (cos.is_contiguous() and sin.is_contiguous())):
        raise ops.KernelError("attention: cos/sin must be contiguous float32 tables of one shape")


# tuned implementations: fn(...) -> bool, True when it ran
_TUNED = []


def register_tuned(fn) -> None:
    _TUNED.append(fn)


# ---------------------------------------------------------------------------
# tensor-core kernels (bfloat16, head_dim 32 / 64 / 128): host-side planning of work items
# ---------------------------------------------------------------------------
import dataclasses  # noqa: E402
import ctypes  # noqa: E402
from ctypes import c_float, c_int, c_longlong, c_void_p  # noqa: E402

import numpy as np  # noqa: E402

from . import lib as _lib  # noqa: E402
from . import native, policy  # noqa: E402

_P, _I, _L, _F = c_void_p, c_int, c_longlong, c_float


# prompt tiles through the tcgen05 / TMEM / TMA kernel where it covers the shape (head_dim 128, a group
# that divides 128, pages of 16/32/64/... keys); the mma.sync kernel otherwise
USE_TCGEN05 = True

ROWS_PER_CTA = 64          # query rows (tokens x group) of a small tile
ROWS_PER_CTA_LARGE = 128   # of a large tile, used when some portion fills one
KEYS_PER_TILE = 64
MAX_SPLITS = 16            # slices of a prompt tile's keys
MIN_TILES_PER_SPLIT = 2    # such a slice is at least 128 keys long
DECODE_WARPS = 4           # slices of a decode row per CTA (one per warp)
DECODE_CTAS_PER_SM = 2
DECODE_MAX_SPLITS = 32     # 8 CTAs of 4 slices: what a cluster merges in the kernel (batch 1 at context 2048: 313 tok/s
                           # against 299 with 64 slices and the second kernel)
DECODE_MERGE_IN_KERNEL_MAX_SPLITS = 32   # up to 8 CTAs of a row form a cluster and merge their slices themselves
DECODE_LONG_SPLITS = 64     # rows of DECODE_LONG_CONTEXT keys and more get up to this many slices (the most the merge kernel
                            # takes) when 32 a row leave SMs without a CTA; their partial results go through global memory
                            # and the second kernel. Qwen3-8B sizes, batch 1: context 8,192 280 tok/s against 284 with 32
                            # slices, 16,384 261 against 251, 32,768 230 against 204; batch 2 at 16,384 496 against 481
DECODE_LONG_CONTEXT = 12288
DECODE_VERY_LONG_CONTEXT = 24576   # and from here up to 128: batch 1 at 32,768 keys 240 against 229, at 65,536 206 against 188
DECODE_VERY_LONG_SPLITS = 128
DECODE_MIN_KEYS_PER_SPLIT = 32
DECODE_MAX_GROUP = 16
_SM_COUNT = None


def _sm_count(device) -> int:
    global _SM_COUNT
    if _SM_COUNT is None:
        _SM_COUNT = torch.cuda.get_device_properties(device).multi_processor_count
    return _SM_COUNT


@dataclasses.dataclass
class RopeFusion:
    """What the decode kernel needs to do the q/k norm, the rotation and the cache write itself."""
    q_norm_w: Optional[torch.Tensor]
    k_norm_w: Optional[torch.Tensor]
    eps: float
    weight_offset: float
    cos: torch.Tensor
    sin: torch.Tensor
    positions: torch.Tensor
    slots: torch.Tensor
    write_kv: bool


@dataclasses.dataclass
class AttentionPlan:
    tile_items: torch.Tensor      # int32 [n, 4]: request, first token of the tile, slice, slices
    num_tile_items: int
    decode_items: torch.Tensor    # int32 [n, 4]: request, 0, first slice of the CTA, slices
    num_decode_items: int
    row_splits: torch.Tensor      # int32 [tokens]
    rows_per_cta: int             # 64 or 128 query rows per tile
    tile_split: bool              # some prompt tile was cut into slices (merged after the tile kernel)
    max_splits: int
    part_o: Optional[torch.Tensor]
    part_lse: Optional[torch.Tensor]
    decode_merge_in_kernel: bool = False


def decode_splits(num_rows: int, nkv: int, sm_count: int, max_kv_len: Optional[int], capacity: Optional[int] = None,
                  long_ok: bool = True) -> int:
    """Slices per decode row: as many as fill the GPU once (two CTAs of four slices per SM), a
    multiple of four, each at least 32 keys long when the lengths are known. ``capacity``: the keys a row
    may hold when the lengths are not known (a recorded step: the width of its block table). ``long_ok`` False: no
    more slices than a cluster merges, whatever the lengths (steps that also bring prompt portions: the scratch of
    slices merged by the second kernel is indexed by the step's rows, and the GPU is busy anyway)."""
    if policy.batch_invariant():
        return policy.INVARIANT_DECODE_SPLITS      # the same cutting whatever else is in the step
    pairs = max(1, num_rows * nkv)
    ns = DECODE_WARPS * max(1, (DECODE_CTAS_PER_SM * sm_count) // pairs)
    # a recorded step serves the lengths in the upper half of its table's capacity
    longest = max_kv_len if max_kv_len is not None else (capacity // 2 if capacity is not None else None)
    limit = DECODE_MAX_SPLITS
    if long_ok and longest is not None and longest >= DECODE_LONG_CONTEXT:
        limit = DECODE_VERY_LONG_SPLITS if longest >= DECODE_VERY_LONG_CONTEXT else DECODE_LONG_SPLITS
    ns = min(ns, limit)
    if ns > DECODE_MAX_SPLITS:
        ns = 1 << (ns.bit_length() - 1)    # beyond what a cluster merges: 64 or 128 (72 slices measured slower than 64)
    if max_kv_len is not None:
        ns = min(ns, max(DECODE_WARPS, (max_kv_len // DECODE_MIN_KEYS_PER_SPLIT) // DECODE_WARPS * DECODE_WARPS))
    return ns


def tile_rows(q_lens, group: int, decode_kernel: bool = True) -> int:
    """Query rows per tile: 128 when some prompt portion fills such a tile, else 64."""
    if policy.batch_invariant():
        return ROWS_PER_CTA_LARGE
    big = [n for n in q_lens if not (decode_kernel and n == 1 and group <= DECODE_MAX_GROUP)]
    if group <= ROWS_PER_CTA and any(n * group >= ROWS_PER_CTA_LARGE for n in big):
        return ROWS_PER_CTA_LARGE
    return ROWS_PER_CTA if group <= ROWS_PER_CTA else ROWS_PER_CTA_LARGE


def plan_items(q_lens, kv_lens, group: int, nkv: int, window: Optional[int], sm_count: int,
               decode_kernel: bool = True, rows_per_cta: Optional[int] = None, whole_tiles_kernel: bool = False):
    """Work items of one step.

    Requests that bring one token go to the decode kernel (when the group fits its 16 rows):
    each row's keys are cut into ``decode_splits`` slices, four per CTA. The others are cut
    into query tiles (``rows_per_cta`` rows = rows // group tokens times `group` heads) for the tile kernel;
    when that grid would leave SMs idle and there are no decode rows, a tile's keys are cut
    into slices too, merged by a second kernel (``whole_tiles_kernel``: keep tiles whole unless they would not even
    fill half of the SMs; for the fast tile kernel).
    Returns (tile_items [n, 4], decode_items [n, 4], row_splits [tokens], max_splits, tile_split)."""
    rows_per_cta = rows_per_cta or tile_rows(q_lens, group, decode_kernel)
    tpt = rows_per_cta // group
    starts = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int64)
    row_splits = np.ones(int(starts[-1]), dtype=np.int32)
    use_decode = decode_kernel and group <= DECODE_MAX_GROUP
    decode_reqs = [b for b, n in enumerate(q_lens) if n == 1] if use_decode else []
    decode_set = set(decode_reqs)
    tiles = []
    for b, (n, kv) in enumerate(zip(q_lens, kv_lens)):
        if b in decode_set:
            continue
        for t0 in range(0, n, tpt):
            toks = min(tpt, n - t0)
            pos0 = kv - n + t0
            lo = (max(0, pos0 - window + 1) if window else 0) & ~(KEYS_PER_TILE - 1)
            span_tiles = -(-(pos0 + toks - lo) // KEYS_PER_TILE)
            tiles.append((b, t0, toks, span_tiles))
    max_splits = 1
    decode_items = []
    if decode_reqs:
        ns = decode_splits(len(decode_reqs), nkv, sm_count, max(kv_lens[b] for b in decode_reqs), long_ok=not tiles)
        max_splits = ns
        for b in decode_reqs:
            row_splits[starts[b]] = ns
            decode_items.extend((b, 0, s0, ns) for s0 in range(0, ns, DECODE_WARPS))
    want = 1
    idle_below = sm_count // 2 if whole_tiles_kernel else 2 * sm_count
    if tiles and not decode_reqs and len(tiles) * nkv < idle_below and not policy.batch_invariant():
        want = min(MAX_SPLITS, -(-2 * sm_count // (len(tiles) * nkv)))
    tile_items = []
    tile_split = False
    # tiles with the most keys first: the long ones must not be the last to start
    tiles.sort(key=lambda t: -t[3])
    for b, t0, toks, span_tiles in tiles:
        ns = max(1, min(want, span_tiles // MIN_TILES_PER_SPLIT))
        if ns > 1:
            tile_split = True
            max_splits = max(max_splits, ns)
            row_splits[starts[b] + t0: starts[b] + t0 + toks] = ns
        tile_items.extend((b, t0, s, ns) for s in range(ns))
    return (np.asarray(tile_items, dtype=np.int32).reshape(-1, 4), np.asarray(decode_items, dtype=np.int32).reshape(-1, 4),
            row_splits, max_splits, tile_split)


def plan_items_static_decode(num_requests: int, group: int, nkv: int, sm_count: int, capacity: Optional[int] = None):
    """Items of a decode step whose launch is recorded once and replayed (a CUDA graph): one
    query token per request, and a number of key slices that depends on the batch size only;
    the kernels find each slice's bounds from the request's current length."""
    empty = np.zeros((0, 4), dtype=np.int32)
    if group <= DECODE_MAX_GROUP:
        ns = decode_splits(num_requests, nkv, sm_count, None, capacity)
        items = np.asarray([(b, 0, s0, ns) for b in range(num_requests) for s0 in range(0, ns, DECODE_WARPS)],
                           dtype=np.int32).reshape(-1, 4)
        return empty, items, np.full(num_requests, ns, dtype=np.int32), ns, False
    ns = 1
    if num_requests * nkv < 2 * sm_count and not policy.batch_invariant():
        ns = min(MAX_SPLITS, -(-2 * sm_count // (num_requests * nkv)))
    items = np.asarray([(b, 0, s, ns) for b in range(num_requests) for s in range(ns)], dtype=np.int32).reshape(-1, 4)
    return items, empty, np.full(num_requests, ns, dtype=np.int32), ns, ns > 1


_PLAN_RING = ops.UploadRing()


def _plan_for(ctx, group_step, group: int, nq: int, nkv: int, hd: int, window, device) -> AttentionPlan:
    key = ("attention_mma_plan", id(group_step), group, nkv, window)
    plan = ctx.scratch.get(key)
    if plan is None:
        if getattr(ctx, "static_decode", False):
            rows = ROWS_PER_CTA if (group <= ROWS_PER_CTA and not policy.batch_invariant()) else ROWS_PER_CTA_LARGE
            table = getattr(group_step, "block_table", None)
            capacity = int(table.shape[1]) * ctx.cache.page_size if table is not None and table.dim() == 2 else None
            t_items, d_items, row_splits, max_splits, tile_split = plan_items_static_decode(
                ctx.num_requests, group, nkv, _sm_count(device), capacity)
        else:
            rows = tile_rows(ctx.q_lens_host, group)
            page = ctx.cache.page_size
            # the tcgen05 kernel takes slices too, but is fast enough per tile that cutting its tiles only pays when
            # they would not even fill half of the SMs (measured: a 2,048-token prompt at Qwen3-0.6B sizes, 256 tiles,
            # 4.1 ms whole against 4.6 ms cut in two with their partial results merged by a second kernel)
            fast_tiles = (USE_TCGEN05 and hd == 128 and rows == ROWS_PER_CTA_LARGE and ROWS_PER_CTA_LARGE % group == 0
                          and page >= 16 and page & (page - 1) == 0)
            t_items, d_items, row_splits, max_splits, tile_split = plan_items(
                ctx.q_lens_host, ctx.kv_lens_host, group, nkv, window, _sm_count(device), rows_per_cta=rows,
                whole_tiles_kernel=fast_tiles)
        packed = np.concatenate([t_items.reshape(-1), d_items.reshape(-1), row_splits]).astype(np.int32, copy=False)
        dev = _PLAN_RING.upload(packed, device)   # pinned memory read by a kernel: the host does not wait for the stream
        nt, nd = t_items.shape[0], d_items.shape[0]
        part_o = part_lse = None
        # decode rows merge their slices inside the kernel when their CTAs fit a cluster; prompt tiles
        # are only ever cut when there are no decode rows
        in_kernel = nd > 0 and max_splits <= DECODE_MERGE_IN_KERNEL_MAX_SPLITS
        if max_splits > 1 and not in_kernel:
            part_o = torch.empty(ctx.num_tokens * nq * max_splits * hd, dtype=torch.float32, device=device)
            part_lse = torch.empty(ctx.num_tokens * nq * max_splits, dtype=torch.float32, device=device)
        plan = AttentionPlan(dev[: nt * 4].view(nt, 4), nt, dev[nt * 4: (nt + nd) * 4].view(nd, 4), nd,
                             dev[(nt + nd) * 4:], rows, tile_split, max_splits, part_o, part_lse, in_kernel)
        ctx.scratch[key] = plan
    return plan


def _tcgen05_takes(plan, q, out, k_cache, page_size, nq, nkv, hd, page_stride) -> bool:
    group = nq // nkv
    return (USE_TCGEN05 and hd == 128 and plan.rows_per_cta == ROWS_PER_CTA_LARGE
            and ROWS_PER_CTA_LARGE % group == 0 and page_size >= 16 and page_size & (page_size - 1) == 0
            and q.stride(0) % 8 == 0 and out.stride(0) % 8 == 0 and page_stride % 8 == 0
            and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0 and k_cache.data_ptr() % 16 == 0)


def tcgen05_status() -> int:
    """0, or the code of the bounded wait that ran out in the tcgen05 attention kernel since the
    last call (synchronises the device)."""
    v = c_int(0)
    _lib.check(_lib.load().oi_attention_tcgen05_status(ctypes.byref(v)), "attention_tcgen05_status")
    return v.value


FUSE_ROPE_IN_DECODE = True


def decode_takes_rope(qkv: torch.Tensor, ctx, group_step, nq: int, nkv: int, hd: int, window, cos, q_norm_w,
                      page_stride: int) -> bool:
    """Whether this step's attention is the decode kernel alone (every request brings one token) and
    that kernel can take the norm, rotation and cache write into itself."""
    if not FUSE_ROPE_IN_DECODE or cos is None or qkv.dtype != torch.bfloat16 or hd not in (32, 64, 128):
        return False
    if policy.batch_invariant():
        return False
    if nq // nkv > DECODE_MAX_GROUP or qkv.stride(0) % 8 or page_stride % 8 or qkv.data_ptr() % 16:
        return False
    rot_half = cos.shape[1]
    if rot_half == 0 or rot_half % 2 or 2 * rot_half > hd:
        return False
    if q_norm_w is not None and q_norm_w.dtype not in (torch.bfloat16, torch.float32):
        return False
    if not (getattr(ctx, "static_decode", False) or all(n == 1 for n in ctx.q_lens_host)):
        return False
    plan = _plan_for(ctx, group_step, nq // nkv, nq, nkv, hd, window, qkv.device)
    # Measured at Qwen3-8B sizes: 3.59 -> 3.56 ms per step at batch 8, where all CTAs of the kernel run at once;
    # at batch 64 (two waves of CTAs, each with the rotation in front) the separate kernel is 1.6 % faster.
    one_wave = plan.num_decode_items * nkv <= DECODE_CTAS_PER_SM * _sm_count(qkv.device)
    return plan.num_tile_items == 0 and plan.num_decode_items > 0 and one_wave


def attention_step(ctx, group_step, qkv: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, page_stride: int,
                   nq: int, nkv: int, hd: int, window, cos=None, q_norm_w=None) -> "native.AttnStep":
    """What every attention call of one geometry shares in this step (csrc/oi_api.h, OiAttnStep): the step's metadata
    on the device, which kernels take it, and their work items. Made once per step and geometry."""
    key = ("attention_step", id(group_step), nq, nkv, hd, window, qkv.dtype, qkv.stride(0), out.stride(0), cos is not None)
    step = ctx.scratch.get(key)
    if step is not None:
        return step
    group = nq // nkv
    bt = group_step.block_table
    # the tensor-core kernels: bfloat16, head_dim 32, 64 or 128
    tensor_core = (qkv.dtype == torch.bfloat16 and hd in (32, 64, 128) and group <= ROWS_PER_CTA_LARGE
                   and qkv.stride(0) % 2 == 0 and page_stride % 8 == 0)
    def ptr(obj, name):     # a step that only runs kernels which do not read a tensor may leave it out
        t = getattr(obj, name, None)
        return 0 if t is None else t.data_ptr()

    step = native.AttnStep(
        slot_mapping=ptr(group_step, "slot_mapping"), block_table=bt.data_ptr(), kv_lens=group_step.kv_lens.data_ptr(),
        cu_seqlens=ctx.cu_seqlens.data_ptr(), token_req=ptr(ctx, "token_req"), positions=ptr(ctx, "positions"),
        bt_stride=bt.stride(0), tokens=ctx.num_tokens, page_size=ctx.cache.page_size, num_pages=k_cache.shape[0],
        page_stride=int(page_stride), tensor_core=1 if tensor_core else 0)
    if tensor_core:
        plan = _plan_for(ctx, group_step, group, nq, nkv, hd, window, qkv.device)
        step.keep = plan       # the plan's device tensors live as long as the description
        step.tile_items, step.num_tile_items = plan.tile_items.data_ptr(), plan.num_tile_items
        step.decode_items, step.num_decode_items = plan.decode_items.data_ptr(), plan.num_decode_items
        step.row_splits = plan.row_splits.data_ptr()
        step.rows_per_cta, step.tile_split, step.max_splits = plan.rows_per_cta, 1 if plan.tile_split else 0, plan.max_splits
        step.merge_in_kernel = 1 if plan.decode_merge_in_kernel else 0
        step.part_o = 0 if plan.part_o is None else plan.part_o.data_ptr()
        step.part_lse = 0 if plan.part_lse is None else plan.part_lse.data_ptr()
        step.use_tcgen05 = 1 if (plan.num_tile_items and _tcgen05_takes(plan, qkv, out, k_cache, ctx.cache.page_size, nq, nkv,
                                                                       hd, page_stride)) else 0
        step.fuse_rope = 1 if decode_takes_rope(qkv, ctx, group_step, nq, nkv, hd, window, cos, q_norm_w, page_stride) else 0
    ctx.scratch[key] = step
    return step


def attention_mma(q, out, k_cache, v_cache, page_stride, ctx, group_step, nq, nkv, hd, scale, window) -> bool:
    """The tensor-core kernels alone, when they cover the shape (bfloat16, head_dim 32, 64 or 128): q is ready and the
    cache is written. Returns whether they ran."""
    step = attention_step(ctx, group_step, q, out, k_cache, page_stride, nq, nkv, hd, window)
    if not step.tensor_core:
        return False
    run_attention(step, attention_layer(q, out, k_cache, v_cache, nq, nkv, hd, scale, window, write_kv=False, rope_mode=0))
    return True
