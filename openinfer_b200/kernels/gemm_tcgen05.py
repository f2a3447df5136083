"""Wrapper of the hand-written tcgen05 / TMEM / TMA product for bfloat16 operands."""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_longlong, c_void_p

import torch

from . import lib as _lib
from . import ops
from .lib import KernelError


ACT_BLOCK = 64    # the fused gate/up matrix: blocks of 64 gate rows followed by the 64 up rows of the same indices


def takes(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the kernel accepts these operands (bfloat16 in, bfloat16 or float32 out, TMA alignment)."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype not in (torch.bfloat16, torch.float32):
        return False
    K = x.shape[1]
    return (K % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1 and x.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


PAIR = 0          # tile_n value that selects 256 x 256 tiles computed by pairs of CTAs (cta_group::2)
ROW_TILE = 256    # rows of the widest row tile of the prompt products (a pair of CTAs): steps whose rows are a multiple fill every tile


def portion_tile(rows: int, K: int = 1 << 30) -> int:
    """The tile a prompt portion of ``rows`` tokens is computed with (what the native dispatch of the fused gate/up
    product uses). Short sums (K <= 2048) of fewer than 2,048 rows stay with single CTAs: a tile's products are then
    no longer than its epilogue, which the pairs' larger tile does not hide (fused gate/up, N 6144, K 1024, single
    against pair, us: 512 rows 11.3 / 13.1; 1,024 rows 17.6 / 18.8; 2,048 rows 25.7 / 25.3; 4,152 rows 46.0 / 43.8;
    K 2048 at 2,048 rows 43.1 / 41.4). Measured on B200 at 2,048 rows (us, library / pair / one CTA per tile):
    QKV 6144 x 4096: 72 / 76 / 84; O 4096 x 4096: 49 / 51 / 51; down 4096 x 12288: 136 / 148 / 165;
    gate|up 24576 x 4096: 279 / 285 / 313 (and 285 includes the activation, which costs the library path a further
    32 us kernel): the plain products of prompt portions stay with the library unless OI_PREFILL_GEMM=pair."""
    from . import native
    return PAIR if rows >= _lib.load().oi_option(native.OPT_PAIR_MIN_ROWS) and (K > 2048 or rows >= 2048) else 256


def gemm(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, tile_n: int = 256) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T on the tcgen05 tensor cores (float32 accumulation in TMEM).
    ``tile_n``: 256 or 128 columns per 128-row tile of one CTA, or ``PAIR``."""
    if not (x.is_cuda and w.is_cuda and out.is_cuda):
        raise KernelError("gemm_tcgen05: operands must be on a CUDA device; this package has no CPU path")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or not takes(out, x, w):
        raise KernelError(f"gemm_tcgen05: operands not accepted: x={tuple(x.shape)} w={tuple(w.shape)} out={tuple(out.shape)}")
    L = _lib.load()
    if tile_n == PAIR:
        return _pair(L, out, x, w, 0)
    _lib.check(L.oi_gemm_tcgen05(out.data_ptr(), 1 if out.dtype == torch.bfloat16 else 0, out.stride(0), x.data_ptr(),
                                 x.stride(0), w.data_ptr(), w.stride(0), M, N, K, tile_n, 0,
                                 _lib.current_stream()), "gemm_tcgen05")
    return out


def _pair(L, out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, silu_mul: int) -> torch.Tensor:
    M, K = x.shape
    _lib.check(L.oi_gemm_tcgen05_pair(out.data_ptr(), 1 if out.dtype == torch.bfloat16 else 0, out.stride(0), x.data_ptr(),
                                      x.stride(0), w.data_ptr(), w.stride(0), M, w.shape[0], K, silu_mul,
                                      _lib.current_stream()), "gemm_tcgen05_pair")
    return out


def gemm_silu_mul(out: torch.Tensor, x: torch.Tensor, w_gate_up: torch.Tensor, tile_n: int = 256,
                  act: str = "silu") -> torch.Tensor:
    """out[M, I] = act(x Wg^T) * (x Wu^T) in one kernel (act: "silu" or "gelu_tanh"). ``w_gate_up`` is [2 I, K] with rows in blocks
    of 64 gate rows followed by the 64 up rows of the same indices (I a multiple of 128: a tile of the
    kernel holds two such pairs)."""
    M, K = x.shape
    N = w_gate_up.shape[0]
    if N % (2 * ACT_BLOCK) or out.shape != (M, N // 2) or out.dtype != torch.bfloat16 or not takes(out, x, w_gate_up):
        raise KernelError(f"gemm_silu_mul: operands not accepted: x={tuple(x.shape)} w={tuple(w_gate_up.shape)} out={tuple(out.shape)}")
    L = _lib.load()
    code = ops.act_code(act)
    if tile_n == PAIR:
        return _pair(L, out, x, w_gate_up, code)
    _lib.check(L.oi_gemm_tcgen05(out.data_ptr(), 1, out.stride(0), x.data_ptr(), x.stride(0), w_gate_up.data_ptr(),
                                 w_gate_up.stride(0), M, N, K, tile_n, code, _lib.current_stream()),
               "gemm_tcgen05 (fused activation)")
    return out


def status() -> int:
    """0, or the role whose bounded wait ran out since the last call (synchronises the device)."""
    L = _lib.load()
    v = c_int(0)
    _lib.check(L.oi_gemm_tcgen05_status(ctypes.byref(v)), "gemm_tcgen05_status")
    return v.value
