"""y = x W^T for the projections: picks the product kernel by operand types.

* bfloat16 x bfloat16: the tensor-core path. The reference's engine calls the vendor
  library for every projection (pegainfer-kernels/csrc/shared/linear.cu:312-362,
  ``cublasGemmEx`` with float32 accumulation); the same library call stands here until
  a hand-written tcgen05 kernel takes the shape (see ``set_bf16_gemm``).
* anything with a float32 operand: the hand-written float32-accumulate kernel on the
  ordinary pipes (no reduced-precision matrix mode), summed in ascending k.
"""
from __future__ import annotations

from ctypes import c_int, c_longlong, c_void_p
from typing import Callable, Optional

import torch

from . import lib as _lib
from . import ops


# programmatic dependent launch of the decode products (see gemm_skinny.cu)
import os as _os  # noqa: E402
USE_PDL = _os.environ.get('OI_PDL', '1') == '1'
_FORCE_C = int(_os.environ.get('OI_SKINNY_C', '0'))

SKINNY_MAX_ROWS = 16
# Measured on B200 (cold weights, M = 8, K = 4096): the skinny kernel beats the library where a
# product is short enough for fixed costs to matter (N 4096..6144: 12-15 us vs 14-16 us) and loses on
# long ones (N 24576: 43 vs 38 us; N 151936: 221 vs 208 us), so those stay with the library.
SKINNY_MAX_WEIGHT_ROWS = 8192
# Forming silu(gate) * up while the product kernel stages its activations repeats the exponentials
# once per 64-row tile of the weight (64 times at N = 4096): measured 44.7 us for the fused down
# projection against 25 + 3.2 us for the two kernels. The fused path stays available and tested.
FUSE_SILU_MUL = False
_SM_COUNT = None

# hook for a hand-written bf16 kernel: fn(out, x, w) -> bool (True when it took the shape)
_bf16_gemm: Optional[Callable[[torch.Tensor, torch.Tensor, torch.Tensor], bool]] = None


def set_bf16_gemm(fn: Optional[Callable[[torch.Tensor, torch.Tensor, torch.Tensor], bool]]) -> None:
    global _bf16_gemm
    _bf16_gemm = fn


def skinny_cluster_size(N: int, K: int, sm_count: int) -> int:
    """How many K slices (CTAs per cluster) the skinny kernel uses, 0 if it does not take the
    shape: the fewest slices that fill the GPU twice over, each slice's activations within 64 KB
    of shared memory where possible."""
    row_tiles = -(-N // 64)
    valid = [c for c in (1, 2, 4, 8) if K % (32 * c) == 0 and 49152 + 32 * (K // c + 64) + 4096 <= 200 * 1024]
    if not valid:
        return 0
    # measured on B200 at M = 8: four slices are best for the short products (N 4096..6144)
    for c in (4, 2, 8, 1):
        if c in valid:
            return c
    return valid[-1]


def _skinny(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, silu_mul: int) -> bool:
    """The hand-written weight-streaming kernel, when it takes the shape."""
    global _SM_COUNT
    M, N = x.shape[0], w.shape[0]
    K = w.shape[1]
    if M > SKINNY_MAX_ROWS or N > SKINNY_MAX_WEIGHT_ROWS or out.dtype not in (torch.bfloat16, torch.float32):
        return False
    if x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        return False
    if x.stride(0) % 8 or w.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16:
        return False
    if _SM_COUNT is None:
        _SM_COUNT = torch.cuda.get_device_properties(x.device).multi_processor_count
    c = skinny_cluster_size(N, K, _SM_COUNT)
    if c == 0:
        return False
    if _FORCE_C and K % (32 * _FORCE_C) == 0 and 49152 + 32 * (K // _FORCE_C + 64) + 4096 <= 200 * 1024:
        c = _FORCE_C
    L = _lib.load()
    _lib.check(L.oi_gemm_skinny(out.data_ptr(), 1 if out.dtype == torch.bfloat16 else 0, out.stride(0), x.data_ptr(),
                                x.stride(0), w.data_ptr(), w.stride(0), M, N, K, int(silu_mul), c,
                                1 if USE_PDL else 0, torch.cuda.current_stream().cuda_stream), "gemm_skinny")
    return True


def linear_silu_mul(gate_up: torch.Tensor, w: torch.Tensor, block: Optional[int] = None) -> torch.Tensor:
    """(silu(gate) * up) W^T for a fused [M, 2K] gate|up buffer (blocks of ``block`` gates then
    their ups; default all gates, then all ups) and w [N, K]."""
    M, K = gate_up.shape[0], w.shape[1]
    block = K if block is None else block
    if FUSE_SILU_MUL and gate_up.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 0 < M <= SKINNY_MAX_ROWS:
        out = torch.empty((M, w.shape[0]), dtype=gate_up.dtype, device=gate_up.device)
        if _skinny(out, gate_up, w, block):
            return out
    act = torch.empty((M, K), dtype=gate_up.dtype, device=gate_up.device)
    ops.silu_mul(act, gate_up, block)
    return linear(act, w)


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
        if _bf16_gemm is not None and _bf16_gemm(out, x, w):
            return out
        if M <= SKINNY_MAX_ROWS and _skinny(out, x, w, 0):
            return out
        if out_dtype == torch.bfloat16:
            torch.mm(x, w.t(), out=out)
        else:
            out.copy_(torch.mm(x, w.t(), out_dtype=out_dtype))
        return out
    return ops.gemm_generic(out, x, w)
