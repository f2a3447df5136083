"""y = x W^T for the projections: picks the product kernel by operand types and shape.

* bfloat16 x bfloat16, up to 32 rows (decode): the hand-written weight-streaming kernel on the
  5th-generation tensor cores (``gemm_stream.cu``: TMA -> shared memory -> tcgen05.mma with the
  weight rows on the M side), which reads nothing but weights before the kernel ahead of it on
  the stream has finished and therefore starts its stream under that kernel's tail.
* bfloat16 x bfloat16 otherwise: a registered hand-written kernel (``set_bf16_gemm``) if it takes
  the shape, else the vendor library. The reference's engine calls the vendor library for every
  projection (pegainfer-kernels/csrc/shared/linear.cu:312-362, ``cublasGemmEx`` with float32
  accumulation).
* anything with a float32 operand: the hand-written float32-accumulate kernel on the
  ordinary pipes (no reduced-precision matrix mode), summed in ascending k.
"""
from __future__ import annotations

import os as _os
from typing import Callable, Optional

import torch

from . import gemm_tcgen05 as _tc
from . import lib as _lib
from . import ops, policy

# which hand-written kernel takes the decode products: "stream" (tcgen05), "skinny" (mma.sync), "library"
DECODE_GEMM = _os.environ.get("OI_DECODE_GEMM", "stream")
_FORCE_C = int(_os.environ.get("OI_GEMM_C", "0"))

DECODE_MAX_ROWS = 32     # rows up to which the streaming kernel takes a product (32: the most its clusters take)
SKINNY_MAX_ROWS = 16
# Forming silu(gate) * up while the skinny kernel stages its activations repeats the exponentials
# once per 64-row tile of the weight (64 times at N = 4096): measured 44.7 us for the fused down
# projection against 25 + 3.2 us for the two kernels. The fused path stays available and tested.
FUSE_SILU_MUL = False
_SM_COUNT = None

# hook for a hand-written bf16 kernel: fn(out, x, w) -> bool (True when it took the shape)
_bf16_gemm: Optional[Callable[[torch.Tensor, torch.Tensor, torch.Tensor], bool]] = None


def set_bf16_gemm(fn: Optional[Callable[[torch.Tensor, torch.Tensor, torch.Tensor], bool]]) -> None:
    global _bf16_gemm
    _bf16_gemm = fn


def _sm_count(device) -> int:
    global _SM_COUNT
    if _SM_COUNT is None:
        _SM_COUNT = torch.cuda.get_device_properties(device).multi_processor_count
    return _SM_COUNT


def stream_cluster_size(N: int, K: int, sm_count: int) -> int:
    """How many K slices (CTAs per cluster) the streaming kernel uses: one when the tiles of 128
    weight rows alone fill the GPU, else the fewest slices that give every SM a CTA, each slice at
    least two k blocks long. Measured on B200 at M = 8 (us, inside a CUDA graph): N 6144 K 4096:
    14.2 with 4 slices (16.1 with 2, 17.0 with 8); N 4096 K 4096: 11.1 with 8 (11.8 with 4);
    N 4096 K 12288: 20.9 with 8 (22.1 with 4); N 24576 and N 151936: one slice (34.4 and 188). At M = 32 the
    same choices stand (12.8, 9.0, 18.9, 34.9, 198 us against the library's 12.1, 10.0, 21.3, 35.1, 209), and the
    decode step of batch 32 gains 5 % over the library's products (6556 against 6252 tok/s)."""
    tiles = -(-N // 128)
    num_kb = -(-K // 64)
    c = 1
    while c < 8 and tiles * c < sm_count and num_kb // (2 * c) >= 2:
        c *= 2
    return c


def _operands_ok(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor) -> bool:
    if out.dtype not in (torch.bfloat16, torch.float32):
        return False
    if x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        return False
    return not (x.stride(0) % 8 or w.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16)


def _stream(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, act: int = 0) -> bool:
    """The tcgen05 weight-streaming kernel, when it takes the shape. ``act``: 0, or the code of the gate
    activation to form from gate and up rows (``ops.act_code``)."""
    M, N, K = x.shape[0], w.shape[0], w.shape[1]
    if K % 8 or not _operands_ok(out, x, w) or (act and N % 128):
        return False
    c = stream_cluster_size(N, K, _sm_count(x.device))
    if _FORCE_C:
        c = _FORCE_C
    num_kb = -(-K // 64)
    while c > 1 and (c - 1) * (-(-num_kb // c)) >= num_kb:
        c //= 2
    L = _lib.load()
    _lib.check(L.oi_gemm_stream(out.data_ptr(), 1 if out.dtype == torch.bfloat16 else 0, out.stride(0), x.data_ptr(),
                                x.stride(0), w.data_ptr(), w.stride(0), M, N, K, c, int(act),
                                _lib.current_stream()), "gemm_stream")
    return True


def gate_up_silu_mul(x: torch.Tensor, w_gate_up: torch.Tensor, act: str = "silu") -> Optional[torch.Tensor]:
    """act(x Wg^T) * (x Wu^T) for up to 32 rows of x in ONE weight-streaming kernel, or None when it
    does not take the operands. ``w_gate_up`` [2 I, K]: blocks of 64 gate rows followed by the 64 up
    rows of the same indices."""
    M = x.shape[0]
    if policy.batch_invariant():
        return None
    if (DECODE_GEMM != "stream" or not 0 < M <= DECODE_MAX_ROWS or x.dtype != torch.bfloat16
            or w_gate_up.dtype != torch.bfloat16):
        return None
    out = torch.empty((M, w_gate_up.shape[0] // 2), dtype=x.dtype, device=x.device)
    return out if _stream(out, x, w_gate_up, act=ops.act_code(act)) else None


def stream_status() -> int:
    """0, or which bounded wait of the streaming kernel ran out since the last call (synchronises)."""
    from ctypes import byref, c_int
    v = c_int(0)
    _lib.check(_lib.load().oi_gemm_stream_status(byref(v)), "gemm_stream_status")
    return v.value


def skinny_cluster_size(N: int, K: int, sm_count: int) -> int:
    """How many K slices (CTAs per cluster) the skinny kernel uses, 0 if it does not take the
    shape (each slice's activations must fit in shared memory beside the 48 KB of weight rings)."""
    valid = [c for c in (1, 2, 4, 8) if K % (32 * c) == 0 and 49152 + 32 * (K // c + 64) + 4096 <= 200 * 1024]
    if not valid:
        return 0
    # measured on B200 at M = 8: four slices are best for the short products (N 4096..6144)
    for c in (4, 2, 8, 1):
        if c in valid:
            return c
    return valid[-1]


def _skinny(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, silu_mul: int, act: int = 1) -> bool:
    """The mma.sync weight-streaming kernel, when it takes the shape."""
    M, N, K = x.shape[0], w.shape[0], w.shape[1]
    if M > SKINNY_MAX_ROWS or not _operands_ok(out, x, w):
        return False
    c = skinny_cluster_size(N, K, _sm_count(x.device))
    if c == 0:
        return False
    if _FORCE_C and K % (32 * _FORCE_C) == 0 and 49152 + 32 * (K // _FORCE_C + 64) + 4096 <= 200 * 1024:
        c = _FORCE_C
    L = _lib.load()
    _lib.check(L.oi_gemm_skinny(out.data_ptr(), 1 if out.dtype == torch.bfloat16 else 0, out.stride(0), x.data_ptr(),
                                x.stride(0), w.data_ptr(), w.stride(0), M, N, K, int(silu_mul), int(act), c,
                                _lib.current_stream()), "gemm_skinny")
    return True


def linear_silu_mul(gate_up: torch.Tensor, w: torch.Tensor, block: Optional[int] = None, act: str = "silu") -> torch.Tensor:
    """(act(gate) * up) W^T for a fused [M, 2K] gate|up buffer (blocks of ``block`` gates then
    their ups; default all gates, then all ups) and w [N, K]."""
    M, K = gate_up.shape[0], w.shape[1]
    block = K if block is None else block
    if FUSE_SILU_MUL and gate_up.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 0 < M <= SKINNY_MAX_ROWS:
        out = torch.empty((M, w.shape[0]), dtype=gate_up.dtype, device=gate_up.device)
        if _skinny(out, gate_up, w, block, ops.act_code(act)):
            return out
    a = torch.empty((M, K), dtype=gate_up.dtype, device=gate_up.device)
    ops.silu_mul(a, gate_up, block, act)
    return linear(a, w)


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [M, K] (row stride free), w [N, K] -> [M, N] in ``out_dtype`` (default: x's)."""
    out_dtype = out_dtype or x.dtype
    M, N = x.shape[0], w.shape[0]
    if not x.is_cuda:
        raise ops.KernelError("linear: operands must be on a CUDA device; this package has no CPU path")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    if M == 0:
        return out
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        if policy.batch_invariant():
            # one kernel for every step shape: a row's sums are formed in the same order whatever else is in the step
            if not _tc.takes(out, x, w):
                raise ops.KernelError("linear: batch-invariant products need 16-byte aligned bfloat16 operands with K % 8 == 0")
            _tc.gemm(out, x, w, 256)
            return out
        if _bf16_gemm is not None and _bf16_gemm(out, x, w):
            return out
        if M <= DECODE_MAX_ROWS:
            if DECODE_GEMM == "stream" and _stream(out, x, w):
                return out
            if DECODE_GEMM in ("stream", "skinny") and _skinny(out, x, w, 0):
                return out
        if M >= _tc.PAIR_MIN_ROWS and _tc.PREFILL_GEMM == "pair" and _tc.takes(out, x, w):
            _tc.gemm(out, x, w, _tc.PAIR)
            return out
        if out_dtype == torch.bfloat16:
            torch.mm(x, w.t(), out=out)
        else:
            out.copy_(torch.mm(x, w.t(), out_dtype=out_dtype))
        return out
    return ops.gemm_generic(out, x, w)
