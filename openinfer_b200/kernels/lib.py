"""Loads the CUDA library and declares its C entry points.

There is no fallback: if the library cannot be built or loaded, or an entry point
reports an error, a ``KernelError`` is raised.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_char_p, c_float, c_int, c_longlong, c_void_p
from typing import Optional

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


class KernelError(RuntimeError):
    pass


P, I, L, F = c_void_p, c_int, c_longlong, c_float

# name -> argument types (all return int)
_SIGNATURES = {
    "oi_embedding": [P, I, P, I, P, I, I, I, P],
    "oi_gather_tokens": [P, P, P, I, I, P],
    "oi_copy_words": [P, P, I, I, I, I, P, I, P],
    "oi_rmsnorm": [P, P, P, I, P, I, P, I, I, F, F, P],
    "oi_add_inplace": [P, P, I, L, P],
    "oi_scale_cap": [P, I, L, F, F, P],
    "oi_silu_mul": [P, P, I, I, I, I, I, P],
    "oi_qk_norm_rope_kv": [P, I, I, I, I, I, I, P, P, I, F, F, P, P, I, I, P, P, P, P, L, I, I, I, P],
    "oi_attention_generic": [P, I, P, I, I, P, P, L, I, P, I, P, P, I, I, I, I, F, I, P],
    "oi_gemm_generic": [P, I, P, I, P, I, I, I, I, L, L, L, P],
    "oi_argmax": [P, P, I, I, L, P, P, P],
    "oi_token_logprobs": [P, L, I, P, P, P, I, I, P, P, P, P],
    "oi_sample": [P, P, L, P, I, I, P, P, P, P, P, P],
    "oi_sample_use_clusters": [I],
    "oi_gemm_skinny": [P, I, L, P, L, P, L, I, I, I, I, I, I, P],
    "oi_gemm_tcgen05": [P, I, L, P, L, P, L, I, I, I, I, I, P],
    "oi_gemm_tcgen05_pair": [P, I, L, P, L, P, L, I, I, I, I, P],
    "oi_gemm_tcgen05_status": [ctypes.POINTER(c_int)],
    "oi_gemm_stream": [P, I, L, P, L, P, L, I, I, I, I, I, P],
    "oi_set_pdl": [I],
    "oi_gemm_stream_status": [ctypes.POINTER(c_int)],
    "oi_attention_mma": [P, I, P, I, P, P, L, I, P, I, P, P, P, I, P, I, I, I, I, I, F, I, P, P, I, I, P],
    "oi_attention_decode": [P, I, P, I, P, P, L, I, P, I, P, P, P, I, P, I, I, I, I, F, I, P, P, I, I, P],
    "oi_attention_decode_rope": [P, I, P, I, P, P, L, I, P, I, P, P, P, I, P, I, I, I, I, F, I, P, P, I, I,
                                 P, P, I, F, F, P, P, I, I, P, P, I, P],
    "oi_attention_tcgen05": [P, L, I, P, I, P, P, L, I, I, P, I, P, P, P, I, I, I, I, F, I, P, I, P, P, I, P],
    "oi_attention_merge_slices": [P, I, P, P, P, I, I, I, I, P],
    "oi_attention_tcgen05_status": [ctypes.POINTER(c_int)],
    "oi_argmax_noalloc": [P, P, I, I, L, P],
}


def load(verbose: bool = True) -> ctypes.CDLL:
    """The loaded library (built on first use)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        from ..csrc.build import BuildError, ensure_built

        try:
            path = ensure_built(verbose=verbose)
        except BuildError as e:
            raise KernelError(f"the CUDA kernels could not be built: {e}") from e
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"the CUDA kernel library {path} could not be loaded: {e}") from e
        lib.oi_last_error.restype = c_char_p
        lib.oi_last_error.argtypes = []
        lib.oi_abi_version.restype = c_int
        for name, args in _SIGNATURES.items():
            fn = getattr(lib, name, None)
            if fn is None:
                raise KernelError(f"{path} lacks entry point {name}")
            fn.argtypes = args
            fn.restype = c_int
        _declare_optional(lib)
        from . import native
        native.declare(lib)
        native.configure_from_environment(lib)
        _lib = lib
        return lib


# entry points of code outside this package (an extension's own kernels linked into the library)
_OPTIONAL = {}


def declare(name: str, argtypes) -> None:
    """Register the signature of a further entry point. Every entry point of this package is listed
    in ``_SIGNATURES`` above, so that none can be called with undeclared (32-bit) arguments."""
    _OPTIONAL[name] = argtypes
    if _lib is not None:
        _declare_optional(_lib)


def _declare_optional(lib) -> None:
    for name, args in _OPTIONAL.items():
        fn = getattr(lib, name, None)
        if fn is not None:
            fn.argtypes = args
            fn.restype = c_int


# kernels of recorded graphs that replays launched (the library counts the kernels it launches itself)
replayed = 0


def launch_count() -> int:
    """Kernels of this library launched so far: by its entry points, and by replays of recorded graphs."""
    return int(load().oi_launches()) + replayed


try:    # the raw handle of the current stream without building a Stream object (about ten times faster)
    from torch._C import _cuda_getCurrentRawStream as _raw_stream
    from torch._C import _cuda_getDevice as _raw_device
except Exception:   # pragma: no cover - a torch without the private entry points
    _raw_stream = _raw_device = None


def current_stream() -> int:
    """The CUDA stream handle that torch's current stream of the current device stands for."""
    if _raw_stream is not None:
        return _raw_stream(_raw_device())
    import torch
    return torch.cuda.current_stream().cuda_stream


def check(code: int, what: str) -> None:
    if code != 0:
        msg = load().oi_last_error().decode(errors="replace")
        raise KernelError(f"{what} failed (code {code}): {msg}")
