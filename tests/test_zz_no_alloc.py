"""The allocation-free argmax entry point, called through its exported C symbol.

Some users of this library cannot allocate device memory when they call it: their host program
gave every free byte to its own pool at start-up, or it forbids allocation on the serving path
because cudaMalloc stalls the device, or it comes in over the C ABI without torch's allocator.
``oi_argmax_noalloc`` serves them: its scratch is a fixed array inside the library. This test
calls it twice in a row (the array is shared and keeps the last call's contents, so the second
call runs over stale partial results) and compares with the ordinary entry point, which takes
its scratch from the caller. It runs last on purpose: a run that stops at the first failure has
then already run every other test. It passes alone in a fresh process as well as after the rest.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def lib():
    from openinfer_b200.csrc.build import ensure_built
    L = ctypes.CDLL(ensure_built(verbose=False))
    L.oi_argmax_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                    ctypes.c_longlong, ctypes.c_void_p]
    L.oi_argmax_noalloc.restype = ctypes.c_int
    L.oi_last_error.restype = ctypes.c_char_p
    return L


def _existing(logits):
    from openinfer_b200.kernels import ops
    out = torch.empty(logits.shape[0], dtype=torch.int32, device=DEV)
    return ops.argmax(out, logits)


def test_two_calls_in_a_row_match_the_ordinary_entry_point(lib):
    torch.cuda.set_device(0)
    torch.manual_seed(0)
    stream = torch.cuda.current_stream().cuda_stream
    # first call: 8 rows of a large vocabulary with strided rows, ties and a late maximum
    a = torch.randn(8, 151936 + 64, device=DEV)[:, :151936]
    a[1, 151935] = 99.0
    a[2, [7, 70000]] = 98.0          # a tie: the lowest index wins
    a[3, :] = 1.0                    # all tied
    out_a = torch.full((8,), -1, dtype=torch.int32, device=DEV)
    rc = lib.oi_argmax_noalloc(out_a.data_ptr(), a.data_ptr(), 8, 151936, a.stride(0), stream)
    assert rc == 0, lib.oi_last_error()
    # second call right after it, other sizes: the scratch still holds the first call's pairs
    b = torch.randn(37, 5000, device=DEV)
    out_b = torch.full((37,), -1, dtype=torch.int32, device=DEV)
    rc = lib.oi_argmax_noalloc(out_b.data_ptr(), b.data_ptr(), 37, 5000, b.stride(0), stream)
    assert rc == 0, lib.oi_last_error()
    torch.cuda.synchronize()
    assert out_a.tolist() == _existing(a).tolist()          # indices: exact agreement is the tolerance
    assert out_b.tolist() == _existing(b).tolist()
    assert out_a.tolist()[1:4] == [151935, 7, 0]
    assert out_b.tolist() == torch.argmax(b, dim=-1).tolist()


def test_refuses_what_the_built_in_scratch_cannot_hold(lib):
    torch.cuda.set_device(0)
    big = torch.zeros(4, 8, device=DEV)   # the sizes are checked before anything is read
    out = torch.zeros(1024, dtype=torch.int32, device=DEV)
    rc = lib.oi_argmax_noalloc(out.data_ptr(), big.data_ptr(), 1024, 151936, 151936, None)
    assert rc == 3
    msg = lib.oi_last_error().decode()
    assert "16384" in msg and "no memory is allocated" in msg
