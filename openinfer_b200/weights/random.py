"""Random weights from a configuration and a seed.

Each tensor is drawn from its own generator, seeded from (seed, tensor name), so a
tensor's values do not depend on which other tensors exist. Matrices are N(0, std),
norm weights 1 + N(0, std), drawn in float32 and rounded once to the stored dtype.
The reference has no random-weights mode (its tests need real checkpoints); this is
what makes tiny and full-size models available without any download.
"""
from __future__ import annotations

import os
import zlib
from typing import Dict

import torch
from safetensors.torch import save_file

from ..config.base import ModelConfig, resolve_architecture
from ..parts.spec import ParamInfo


def _tensor_seed(seed: int, name: str) -> int:
    return (int(seed) * 0x9E3779B1 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFFFFFF


def random_tensors(expected: Dict[str, ParamInfo], seed: int, dtype: torch.dtype = torch.bfloat16,
                   device="cpu") -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    device = torch.device(device)
    for name in sorted(expected):
        info = expected[name]
        gen = torch.Generator(device=device)
        gen.manual_seed(_tensor_seed(seed, name))
        if info.integer:
            out[name] = torch.randint(0, 2, info.shape, generator=gen, device=device, dtype=torch.int32)
            continue
        kind, std = info.init
        t = torch.randn(info.shape, generator=gen, device=device, dtype=torch.float32) * std
        if kind == "one_plus_normal":
            t = t + 1.0
        elif kind != "normal":
            raise ValueError(f"{name}: unknown init {kind!r}")
        out[name] = t.to(dtype)
    return out


def expected_tensors(config: ModelConfig) -> Dict[str, ParamInfo]:
    """Names and shapes of the tensors the architecture of ``config`` loads."""
    from ..parts.model import Model

    entry = resolve_architecture(config.to_dict())
    return Model(entry.build_spec(config), torch.bfloat16).expected_tensors()


def write_random_model(config: ModelConfig, folder: str, seed: int,
                       dtype: torch.dtype = torch.bfloat16) -> str:
    """Write ``folder/config.json`` and ``folder/model.safetensors`` with random weights."""
    os.makedirs(folder, exist_ok=True)
    config.save(folder)
    tensors = random_tensors(expected_tensors(config), seed, dtype=dtype, device="cpu")
    save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(folder, "model.safetensors"))
    return folder
