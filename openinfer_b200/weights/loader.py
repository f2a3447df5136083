"""Weights from safetensors, by tensor name.

A model folder holds ``model.safetensors`` or an index ``model.safetensors.index.json``
with a ``weight_map`` to shards (pegainfer-core/src/weight_loader.rs:32-64). Every
expected tensor is checked (present, shape) before anything is uploaded, as the
reference validates its whole plan first (weight_loader.rs:411-439), and ONE error lists
everything that is wrong: missing tensors, unexpected tensors, wrong shapes, unusable
dtypes.

Tensors the model did not ask for are not an error by themselves: the reference looks
tensors up by name and never reads the rest (pegainfer-core/src/weight_loader.rs:251-269;
``lm_head.weight`` of a tied model is skipped, pegainfer-qwen3/src/weights/load.rs:85-91),
and real checkpoints carry such tensors (a tied model that still stores its head, rotary
``inv_freq`` buffers of older exports). They are reported back (``ignored``), named in the
error when something else is wrong (a misnamed tensor shows up as one missing and one
unexpected), and refused on their own only with ``strict=True``.

Storage rules: floating tensors are kept in the model dtype, except that a tensor
stored in 32-bit stays 32-bit in a bfloat16 model; in a float32 model everything is
widened (exactly) to float32; integer tensors are kept as int32.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, List, Optional, Tuple

import torch
from safetensors import safe_open

from ..parts.spec import ParamInfo

_FLOAT = {"F64", "F32", "F16", "BF16"}
_INT = {"I64", "I32", "I16", "I8", "U8", "BOOL", "U16", "U32", "U64"}


class WeightError(ValueError):
    """The checkpoint does not fit the model. The message lists every problem."""


def _read_header(path: str) -> Dict[str, dict]:
    with open(path, "rb") as fh:
        raw = fh.read(8)
        if len(raw) != 8:
            raise WeightError(f"{path}: not a safetensors file (too short)")
        (n,) = struct.unpack("<Q", raw)
        if n <= 0 or n > 1 << 30:
            raise WeightError(f"{path}: not a safetensors file (header length {n})")
        try:
            header = json.loads(fh.read(n))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise WeightError(f"{path}: not a safetensors file (bad header: {e})") from None
    header.pop("__metadata__", None)
    return header


def checkpoint_index(folder: str) -> Dict[str, Tuple[str, Tuple[int, ...], str]]:
    """tensor name -> (file path, shape, safetensors dtype string) for every tensor in the folder."""
    single = os.path.join(folder, "model.safetensors")
    index = os.path.join(folder, "model.safetensors.index.json")
    files: List[str] = []
    if os.path.isfile(single):
        files = [single]
    elif os.path.isfile(index):
        with open(index) as fh:
            weight_map = json.load(fh).get("weight_map", {})
        files = sorted({os.path.join(folder, f) for f in weight_map.values()})
        for f in files:
            if not os.path.isfile(f):
                raise WeightError(f"{index} names shard {os.path.basename(f)}, which does not exist")
    else:
        raise WeightError(f"{folder}: neither model.safetensors nor model.safetensors.index.json found")
    out: Dict[str, Tuple[str, Tuple[int, ...], str]] = {}
    for f in files:
        for name, meta in _read_header(f).items():
            out[name] = (f, tuple(int(d) for d in meta["shape"]), str(meta["dtype"]))
    return out


def _target_dtype(stored: str, integer: bool, model_dtype: torch.dtype):
    if integer:
        return torch.int32 if stored in _INT else None
    if stored not in _FLOAT:
        return None
    if model_dtype == torch.float32:
        return torch.float32
    return torch.float32 if stored in ("F32", "F64") else torch.bfloat16


def load_tensors(folder: str, expected: Dict[str, ParamInfo], model_dtype: torch.dtype,
                 device, strict: bool = False, ignored: Optional[List[str]] = None) -> Dict[str, torch.Tensor]:
    """Load every expected tensor onto ``device``. Raises one ``WeightError`` that lists all
    missing tensors, unexpected tensors, wrong shapes and unusable dtypes. Unexpected tensors
    alone raise only when ``strict``; otherwise their names are appended to ``ignored``."""
    index = checkpoint_index(folder)
    missing = sorted(n for n in expected if n not in index)
    unexpected = sorted(n for n in index if n not in expected)
    wrong_shape, wrong_dtype = [], []
    for name, info in expected.items():
        if name not in index:
            continue
        _, shape, stored = index[name]
        if tuple(shape) != tuple(info.shape):
            wrong_shape.append(f"{name}: has shape {list(shape)}, the config expects {list(info.shape)}")
        if _target_dtype(stored, info.integer, model_dtype) is None:
            kind = "an integer" if info.integer else "a floating"
            wrong_dtype.append(f"{name}: stored as {stored}, expected {kind} type")
    if missing or wrong_shape or wrong_dtype or (strict and unexpected):
        lines = [f"{folder}: the checkpoint does not fit the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shapes ({len(wrong_shape)}):")
            lines += [f"    {w}" for w in wrong_shape]
        if wrong_dtype:
            lines.append(f"  wrong dtypes ({len(wrong_dtype)}):")
            lines += [f"    {w}" for w in wrong_dtype]
        raise WeightError("\n".join(lines))
    if ignored is not None:
        ignored.extend(unexpected)

    by_file: Dict[str, List[str]] = {}
    for name in expected:
        by_file.setdefault(index[name][0], []).append(name)
    out: Dict[str, torch.Tensor] = {}
    for path, names in by_file.items():
        with safe_open(path, framework="pt", device="cpu") as f:
            for name in names:
                t = f.get_tensor(name)
                target = _target_dtype(index[name][2], expected[name].integer, model_dtype)
                out[name] = t.to(device=device, dtype=target)
    return out
