"""y = x W^T for the projections. Which kernel takes a product is decided in native code
(``oi_linear``, csrc/host_step.cu) by operand types, shape and options:

* bfloat16 x bfloat16, up to 32 rows (decode): the hand-written weight-streaming kernel on the
  5th-generation tensor cores (``gemm_stream.cu``: TMA -> shared memory -> tcgen05.mma with the
  weight rows on the M side), which reads nothing but weights before the kernel ahead of it on
  the stream has finished and therefore starts its stream under that kernel's tail.
* bfloat16 x bfloat16 otherwise: the vendor library (cuBLASLt, called from the package's own native
  code, ``library_gemm.cu``), or the hand-written pair kernel of ``gemm_tcgen05.cu`` with
  ``OI_PREFILL_GEMM=pair`` and wherever the library cannot be loaded. The reference's engine calls
  the vendor library for every projection (pegainfer-kernels/csrc/shared/linear.cu:312-362,
  ``cublasGemmEx`` with float32 accumulation).
* anything with a float32 operand: the hand-written float32-accumulate kernel on the
  ordinary pipes (no reduced-precision matrix mode), summed in ascending k.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from . import lib as _lib
from . import native, ops, policy

DECODE_MAX_ROWS = 32     # rows up to which the streaming kernel takes a product (32: the most its clusters take)
SKINNY_MAX_ROWS = 16
# Forming act(gate) * up while the skinny kernel stages its activations repeats the exponentials
# once per 64-row tile of the weight (64 times at N = 4096): measured 44.7 us for the fused down
# projection against 25 + 3.2 us for the two kernels. The fused path stays available and tested.
FUSE_SILU_MUL = False

# hook for a hand-written bf16 kernel: fn(out, x, w) -> bool (True when it took the shape)
_bf16_gemm: Optional[Callable[[torch.Tensor, torch.Tensor, torch.Tensor], bool]] = None
_library_tried = False


def set_bf16_gemm(fn: Optional[Callable[[torch.Tensor, torch.Tensor, torch.Tensor], bool]]) -> None:
    global _bf16_gemm
    _bf16_gemm = fn


def ensure_library(device) -> None:
    """The vendor-library product gets its scratch memory the first time a product may need it."""
    global _library_tried
    if not _library_tried:
        _library_tried = True
        native.init_library_gemm(torch.device(device))


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
    L = _lib.load()
    _lib.check(L.oi_gemm_stream(out.data_ptr(), 1 if out.dtype == torch.bfloat16 else 0, out.stride(0), x.data_ptr(),
                                x.stride(0), w.data_ptr(), w.stride(0), M, N, K, L.oi_stream_slices(N, K), int(act),
                                _lib.current_stream()), "gemm_stream")
    return True


def gate_up_silu_mul(x: torch.Tensor, w_gate_up: torch.Tensor, act: str = "silu") -> Optional[torch.Tensor]:
    """act(x Wg^T) * (x Wu^T) for up to 32 rows of x in ONE weight-streaming kernel, or None when it
    does not take the operands. ``w_gate_up`` [2 I, K]: blocks of 64 gate rows followed by the 64 up
    rows of the same indices."""
    M = x.shape[0]
    if policy.batch_invariant():
        return None
    if (_lib.load().oi_option(native.OPT_DECODE_GEMM) != 0 or not 0 < M <= DECODE_MAX_ROWS or x.dtype != torch.bfloat16
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


def _skinny(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, silu_mul: int, act: int = 1) -> bool:
    """The mma.sync weight-streaming kernel with four K slices, when it takes the shape (a slice's activations
    must fit in shared memory beside the 48 KB of weight rings)."""
    M, N, K = x.shape[0], w.shape[0], w.shape[1]
    if M > SKINNY_MAX_ROWS or not _operands_ok(out, x, w):
        return False
    valid = [c for c in (4, 2, 8, 1) if K % (32 * c) == 0 and 49152 + 32 * (K // c + 64) + 4096 <= 200 * 1024]
    if not valid:
        return False
    L = _lib.load()
    _lib.check(L.oi_gemm_skinny(out.data_ptr(), 1 if out.dtype == torch.bfloat16 else 0, out.stride(0), x.data_ptr(),
                                x.stride(0), w.data_ptr(), w.stride(0), M, N, K, int(silu_mul), int(act), valid[0],
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
    if x.shape[1] != w.shape[1] or x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1 or out.shape != (M, N):
        raise ops.KernelError(f"linear: operands not accepted: x={tuple(x.shape)} w={tuple(w.shape)} out={tuple(out.shape)}")
    codes = native.DTYPE_CODE
    if x.dtype not in codes or w.dtype not in codes or out.dtype not in codes:
        raise ops.KernelError(f"linear: dtypes {x.dtype}, {w.dtype} -> {out.dtype} are not supported (float32 or bfloat16)")
    if _bf16_gemm is not None and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and not policy.batch_invariant():
        if _bf16_gemm(out, x, w):
            return out
    if M > DECODE_MAX_ROWS:
        ensure_library(x.device)
    L = _lib.load()
    _lib.check(L.oi_linear(out.data_ptr(), codes[out.dtype], out.stride(0), x.data_ptr(), codes[x.dtype], x.stride(0),
                           w.data_ptr(), codes[w.dtype], w.stride(0), M, N, x.shape[1], _lib.current_stream()), "linear")
    return out
