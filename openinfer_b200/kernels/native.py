"""The library's host-side step code as seen from Python: the structures of ``csrc/oi_api.h`` and the
set-up of the vendor-library product.

The fields below mirror the C structures one for one, in order. Python fills them in (a model's
description once after loading, a step's description every step) and native code launches the kernels.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import lib as _lib

# options of oi_configure
OPT_BATCH_INVARIANT, OPT_DECODE_GEMM, OPT_PREFILL_GEMM, OPT_FORCE_SLICES, OPT_PAIR_MIN_ROWS, OPT_FUSE_NORM = range(6)
DECODE_GEMM_CODES = {"stream": 0, "skinny": 1, "library": 2}
PREFILL_GEMM_CODES = {"library": 0, "pair": 1}

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


class StreamEpilogue(Structure):
    _fields_ = [
        ("ssq_in", c_void_p), ("ssq_units", c_int), ("ssq_stride", c_int), ("inv_width", c_float), ("eps", c_float),
        ("residual", c_void_p), ("ld_residual", c_longlong), ("norm_w", c_void_p), ("norm_w_bf16", c_int),
        ("w_offset", c_float), ("xs", c_void_p), ("ld_xs", c_longlong), ("ssq_out", c_void_p),
    ]


class AttnStep(Structure):
    _fields_ = [
        ("slot_mapping", c_void_p), ("block_table", c_void_p), ("kv_lens", c_void_p), ("cu_seqlens", c_void_p),
        ("token_req", c_void_p), ("positions", c_void_p),
        ("bt_stride", c_int), ("tokens", c_int), ("page_size", c_int), ("num_pages", c_int),
        ("page_stride", c_longlong),
        ("tensor_core", c_int), ("use_tcgen05", c_int), ("fuse_rope", c_int),
        ("tile_items", c_void_p), ("decode_items", c_void_p), ("row_splits", c_void_p),
        ("num_tile_items", c_int), ("num_decode_items", c_int), ("rows_per_cta", c_int), ("tile_split", c_int),
        ("max_splits", c_int), ("merge_in_kernel", c_int),
        ("part_o", c_void_p), ("part_lse", c_void_p),
    ]


class AttnLayer(Structure):
    _fields_ = [
        ("qkv", c_void_p), ("out", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p),
        ("q_norm_w", c_void_p), ("k_norm_w", c_void_p), ("cos_tab", c_void_p), ("sin_tab", c_void_p),
        ("q_row_stride", c_int), ("out_row_stride", c_int), ("dtype", c_int),
        ("nq", c_int), ("nkv", c_int), ("hd", c_int), ("window", c_int),
        ("scale", c_float), ("eps", c_float), ("w_offset", c_float),
        ("norm_dtype", c_int), ("rot_half", c_int), ("max_pos", c_int),
        ("interleaved", c_int), ("write_kv", c_int), ("rope_mode", c_int),
    ]


class LayerDesc(Structure):
    _fields_ = [
        ("input_norm_w", c_void_p), ("post_norm_w", c_void_p), ("w_qkv", c_void_p), ("w_o", c_void_p),
        ("w_gate_up", c_void_p), ("w_down", c_void_p),
        ("attn", AttnLayer),
        ("input_norm_dtype", c_int), ("post_norm_dtype", c_int), ("w_qkv_dtype", c_int), ("w_o_dtype", c_int),
        ("w_gate_up_dtype", c_int), ("w_down_dtype", c_int),
        ("input_eps", c_float), ("input_offset", c_float), ("post_eps", c_float), ("post_offset", c_float),
        ("qkv_rows", c_int), ("attn_step", c_int), ("inter", c_int), ("act", c_int), ("act_block", c_int),
    ]


class ModelDesc(Structure):
    _fields_ = [
        ("layers", POINTER(LayerDesc)), ("embedding", c_void_p), ("final_norm_w", c_void_p), ("head", c_void_p),
        ("num_layers", c_int), ("hidden", c_int), ("vocab", c_int), ("dtype", c_int),
        ("embedding_dtype", c_int), ("final_norm_dtype", c_int), ("head_dtype", c_int),
        ("embedding_scale", c_float), ("final_eps", c_float), ("final_offset", c_float), ("logit_soft_cap", c_float),
        ("max_qkv_rows", c_int), ("max_q_dim", c_int), ("max_inter", c_int),
    ]


class StepDesc(Structure):
    _fields_ = [
        ("token_ids", c_void_p), ("attn_steps", POINTER(AttnStep)), ("want_rows", c_void_p),
        ("h", c_void_p), ("x", c_void_p), ("qkv", c_void_p), ("attn", c_void_p), ("branch_a", c_void_p),
        ("branch_m", c_void_p), ("act", c_void_p), ("gate_up", c_void_p), ("wanted", c_void_p), ("logits", c_void_p),
        ("xs", c_void_p), ("ssq", c_void_p), ("ssq_stride", c_int),
        ("tokens", c_int), ("num_attn_steps", c_int), ("num_want", c_int),
    ]


def declare(lib) -> None:
    """Argument types of the host-step entry points (called by ``lib.load``)."""
    P, I, L = c_void_p, c_int, c_longlong
    lib.oi_library_gemm_ready.argtypes, lib.oi_library_gemm_ready.restype = [], c_int
    lib.oi_library_gemm_init.argtypes, lib.oi_library_gemm_init.restype = [ctypes.c_char_p, P, L], c_int
    lib.oi_library_gemm.argtypes, lib.oi_library_gemm.restype = [P, I, L, P, L, P, L, I, I, I, P], c_int
    lib.oi_configure.argtypes, lib.oi_configure.restype = [I, I], c_int
    lib.oi_option.argtypes, lib.oi_option.restype = [I], c_int
    lib.oi_stream_slices.argtypes, lib.oi_stream_slices.restype = [I, I], c_int
    lib.oi_linear.argtypes, lib.oi_linear.restype = [P, I, L, P, I, L, P, I, L, I, I, I, P], c_int
    lib.oi_gated_mlp.argtypes, lib.oi_gated_mlp.restype = [P, P, I, I, I, I, P, I, P, I, I, I, P, P, P], c_int
    lib.oi_gated_mlp_needs_gate_up.argtypes, lib.oi_gated_mlp_needs_gate_up.restype = [I, I, I, I, I, I], c_int
    lib.oi_attention_layer.argtypes, lib.oi_attention_layer.restype = [POINTER(AttnStep), POINTER(AttnLayer), P], c_int
    lib.oi_forward.argtypes, lib.oi_forward.restype = [POINTER(ModelDesc), POINTER(StepDesc), P], c_int
    lib.oi_launches.argtypes, lib.oi_launches.restype = [], ctypes.c_ulonglong
    lib.oi_launch_fence.argtypes, lib.oi_launch_fence.restype = [], c_int
    lib.oi_gemm_stream_fused.argtypes = [P, I, L, P, L, P, L, I, I, I, I, I, POINTER(StreamEpilogue), P]
    lib.oi_gemm_stream_fused.restype = c_int


def configure_from_environment(lib) -> None:
    """Options that the environment sets for measurements: which kernel takes the decode products
    (OI_DECODE_GEMM = stream | skinny | library), the plain prompt products (OI_PREFILL_GEMM = library | pair),
    a fixed number of K slices (OI_GEMM_C) and the rows from which pairs of CTAs are used (OI_PAIR_MIN_ROWS)."""
    env = os.environ
    if env.get("OI_DECODE_GEMM"):
        lib.oi_configure(OPT_DECODE_GEMM, DECODE_GEMM_CODES[env["OI_DECODE_GEMM"]])
    if env.get("OI_PREFILL_GEMM"):
        lib.oi_configure(OPT_PREFILL_GEMM, PREFILL_GEMM_CODES[env["OI_PREFILL_GEMM"]])
    if env.get("OI_GEMM_C"):
        lib.oi_configure(OPT_FORCE_SLICES, int(env["OI_GEMM_C"]))
    if env.get("OI_FUSE_NORM"):
        lib.oi_configure(OPT_FUSE_NORM, int(env["OI_FUSE_NORM"]))
    if env.get("OI_PAIR_MIN_ROWS"):
        lib.oi_configure(OPT_PAIR_MIN_ROWS, int(env["OI_PAIR_MIN_ROWS"]))


_workspace: Optional[torch.Tensor] = None
LIBRARY_WORKSPACE_BYTES = 32 << 20


def _cublaslt_path() -> Optional[str]:
    """Where torch's own copy of cuBLASLt lies (it is normally loaded already; this is the fallback)."""
    try:
        import nvidia.cublas as pkg     # the wheel torch depends on: a data package, no code
        for folder in list(getattr(pkg, "__path__", [])) + [os.path.dirname(getattr(pkg, "__file__", "") or "")]:
            cand = os.path.join(folder, "lib", "libcublasLt.so.12")
            if os.path.isfile(cand):
                return cand
    except Exception:
        pass
    for cand in ("/usr/local/cuda/lib64/libcublasLt.so.12", "/usr/local/cuda/lib64/libcublasLt.so"):
        if os.path.isfile(cand):
            return cand
    return None


def init_library_gemm(device: torch.device) -> bool:
    """Hand the vendor-library product its scratch memory (once per process). Returns whether the library is
    usable; without it every product runs on this package's own kernels."""
    global _workspace
    lib = _lib.load()
    if lib.oi_library_gemm_ready() and _workspace is not None:
        return True
    _workspace = torch.empty(LIBRARY_WORKSPACE_BYTES, dtype=torch.uint8, device=device)
    path = _cublaslt_path()
    rc = lib.oi_library_gemm_init(path.encode() if path else None, _workspace.data_ptr(), _workspace.numel())
    return rc == 0
