"""Typed configuration: the base class every architecture's config derives from,
and the registry from an architecture's name to its config class and model builder.

A config class lists the config.json keys it reads as dataclass fields. A key
without a default is required; unknown keys are ignored (as the reference's
serde struct does, pegainfer-qwen3/src/config.rs:27-44). No size or constant
that config.json gives is repeated anywhere else in the package.
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, Callable, ClassVar, Dict, List, Optional, Type


class ConfigError(ValueError):
    """A config.json that cannot be used: missing key, wrong type, bad value."""


_MISSING = dataclasses.MISSING


@dataclasses.dataclass(frozen=True)
class ModelConfig:
    """Base of all architecture configs.

    Subclasses are frozen dataclasses whose fields are config.json keys, and
    set ``architecture`` (the name in config.json's ``architectures`` list) and
    ``model_type``.
    """

    architecture: ClassVar[str] = ""
    model_type: ClassVar[str] = ""

    # ---- construction -------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "ModelConfig":
        kwargs: Dict[str, Any] = {}
        missing: List[str] = []
        for f in dataclasses.fields(cls):
            if f.name in raw and raw[f.name] is not None:
                kwargs[f.name] = cls._coerce(f, raw[f.name])
            elif f.default is _MISSING and f.default_factory is _MISSING:  # type: ignore[misc]
                missing.append(f.name)
        if missing:
            raise ConfigError(
                f"{cls.__name__}: config.json lacks required key(s): {', '.join(missing)}"
            )
        cfg = cls(**kwargs)
        cfg.validate()
        return cfg

    @staticmethod
    def _coerce(f: dataclasses.Field, value: Any) -> Any:
        t = f.type if isinstance(f.type, str) else getattr(f.type, "__name__", str(f.type))
        if t.startswith("Optional["):
            t = t[len("Optional["):-1]
        if t.startswith("Tuple[") and isinstance(value, (list, tuple)):
            return tuple(value)
        try:
            if t == "int":
                if isinstance(value, bool) or not isinstance(value, (int, float)) or value != int(value):
                    raise TypeError
                return int(value)
            if t == "float":
                if isinstance(value, bool) or not isinstance(value, (int, float)):
                    raise TypeError
                return float(value)
            if t == "bool":
                if not isinstance(value, bool):
                    raise TypeError
                return value
        except (TypeError, ValueError):
            raise ConfigError(f"config key {f.name!r}: expected {t}, got {value!r}") from None
        return value

    def validate(self) -> None:  # overridden
        pass

    def to_dict(self) -> Dict[str, Any]:
        """The config.json content that reads back as this config."""
        d = dataclasses.asdict(self)
        d["architectures"] = [self.architecture]
        d["model_type"] = self.model_type
        return d

    def save(self, folder: str) -> None:
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w") as fh:
            json.dump(self.to_dict(), fh, indent=2)


# ---------------------------------------------------------------------------
# Registry: architecture name -> (config class, model-spec builder)
# ---------------------------------------------------------------------------
@dataclasses.dataclass(frozen=True)
class ArchitectureEntry:
    name: str
    config_cls: Type[ModelConfig]
    # build_spec(config) -> parts.spec.ModelSpec (the layers, their order, tensor names)
    build_spec: Callable[[ModelConfig], Any]


_ARCHITECTURES: Dict[str, ArchitectureEntry] = {}


def register_architecture(
    name: str, config_cls: Type[ModelConfig], build_spec: Callable[[ModelConfig], Any]
) -> None:
    """Add (or replace) an architecture. ``name`` is what config.json lists under
    ``architectures``; the reference keys its model lines the same way
    (pegainfer-qwen3/src/config.rs:512-527, pegainfer-frontend/src/model_line.rs:364-396)."""
    _ARCHITECTURES[name] = ArchitectureEntry(name, config_cls, build_spec)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures() -> List[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def _ensure_builtin() -> None:
    # the built-in architectures register themselves on import
    from .. import models  # noqa: F401


def resolve_architecture(raw: Dict[str, Any]) -> ArchitectureEntry:
    """Pick the one registered architecture that a config.json dict names."""
    _ensure_builtin()
    archs = raw.get("architectures") or []
    if isinstance(archs, str):
        archs = [archs]
    hits = [a for a in archs if a in _ARCHITECTURES]
    if not hits:
        raise ConfigError(
            f"no registered architecture among {list(archs)!r} "
            f"(model_type={raw.get('model_type')!r}); known: {sorted(_ARCHITECTURES)}"
        )
    if len(set(hits)) > 1:
        raise ConfigError(f"config names several registered architectures: {hits}")
    entry = _ARCHITECTURES[hits[0]]
    want_type = entry.config_cls.model_type
    if want_type and raw.get("model_type", want_type) != want_type:
        raise ConfigError(
            f"architecture {entry.name} expects model_type={want_type!r}, "
            f"config.json says {raw.get('model_type')!r}"
        )
    return entry


def read_config_json(folder: str) -> Dict[str, Any]:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no such file")
    with open(path) as fh:
        try:
            raw = json.load(fh)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON: {e}") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return raw


def load_config(folder: str) -> ModelConfig:
    """Read ``folder/config.json`` into the typed config of the architecture it names."""
    raw = read_config_json(folder)
    entry = resolve_architecture(raw)
    cfg = entry.config_cls.from_dict(raw)
    stops = _stop_token_ids(folder, raw)
    if stops is not None and hasattr(cfg, "with_stop_token_ids"):
        cfg = cfg.with_stop_token_ids(stops)
    return cfg


def _stop_token_ids(folder: str, raw: Dict[str, Any]) -> Optional[List[int]]:
    """generation_config.json's eos_token_id (int or list) wins over config.json's
    (pegainfer-qwen3/src/config.rs:251-265)."""
    path = os.path.join(folder, "generation_config.json")
    eos = None
    if os.path.isfile(path):
        with open(path) as fh:
            eos = json.load(fh).get("eos_token_id")
    if eos is None:
        eos = raw.get("eos_token_id")
    if eos is None:
        return None
    ids = [eos] if isinstance(eos, int) else list(eos)
    out: List[int] = []
    for t in ids:
        if int(t) not in out:
            out.append(int(t))
    return out
