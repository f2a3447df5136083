"""Numeric policy: whether a request's results may depend, at rounding level, on what else is in the batch.

By default the kernels are chosen for speed by the shape of the whole step: the streaming product up to
32 rows and the library beyond, more or fewer key slices per decode row depending on how many rows there
are, tiles of 64 or 128 query rows, the rotation inside or in front of the attention kernel. Every choice
computes the same thing in float32 but may round differently, so a request's logits agree between batches
only "beyond rounding".

With ``set_batch_invariant(True)`` (the reference's ``--batch-invariant``, pegainfer-qwen3/src/lib.rs:419-443:
request-local prompt portions, pinned product algorithm, request-local key slices) every choice depends on
the request alone: all bfloat16 products go through ONE kernel (gemm_tcgen05: a row's dot products are formed
in the same order whatever else is in the step), decode rows always get 16 key slices, prompt tiles are
never cut and always hold 128 query rows, the rotation kernel always runs on its own. Together with
request-local portions in the scheduler a request's logits are then the same BIT FOR BIT whatever it is batched
with. It costs speed, mostly in decode (the product kernel is built for prompt-sized steps). The prefix cache
must be off, as in the reference (pegainfer-qwen3/src/lib.rs:549-554): a hit moves a prompt's portions off the
request's own grid, and a position's bits depend on the portion it is computed in (a portion of one token goes
to the decode kernel, for one); ``LLM`` and the command line refuse the combination. Two engines give the same
bits when they cut prompts alike (the same ``max_prefill_tokens``).
"""
from __future__ import annotations

_BATCH_INVARIANT = False
INVARIANT_DECODE_SPLITS = 16


def set_batch_invariant(on: bool) -> None:
    """Process-wide; the native dispatch of the products is told as well."""
    global _BATCH_INVARIANT
    _BATCH_INVARIANT = bool(on)
    from . import lib, native
    lib.check(lib.load().oi_configure(native.OPT_BATCH_INVARIANT, 1 if _BATCH_INVARIANT else 0), "configure")


def batch_invariant() -> bool:
    return _BATCH_INVARIANT
