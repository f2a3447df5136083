"""Registries from a spec's ``kind`` to the class that implements it.

A part is added by registering a class under a new kind; the spec of that kind is
whatever dataclass the class expects (it must have a ``kind`` attribute). Nothing
else in the package has to change: blocks build their mixer, feed-forward and norms
through these tables, and the model builds its blocks through them.
"""
from __future__ import annotations

from typing import Any, Callable, Dict

MIXERS: Dict[str, Callable[[Any], Any]] = {}
FEED_FORWARDS: Dict[str, Callable[[Any], Any]] = {}
NORMS: Dict[str, Callable[[Any], Any]] = {}
POSITION_ENCODINGS: Dict[str, Callable[[Any], Any]] = {}
BLOCKS: Dict[str, Callable[[Any], Any]] = {}


def _register(table: Dict[str, Any], what: str):
    def decorator_or_call(kind: str, cls=None):
        def do(c):
            table[kind] = c
            return c
        return do if cls is None else do(cls)
    decorator_or_call.__doc__ = f"Register a {what} class under ``kind`` (usable as a decorator)."
    return decorator_or_call


register_mixer = _register(MIXERS, "mixer")
register_feed_forward = _register(FEED_FORWARDS, "feed-forward")
register_norm = _register(NORMS, "norm")
register_position_encoding = _register(POSITION_ENCODINGS, "position encoding")
register_block = _register(BLOCKS, "block")


def _build(table: Dict[str, Any], what: str, spec: Any):
    kind = getattr(spec, "kind", None)
    if kind not in table:
        raise KeyError(f"no {what} registered under kind {kind!r}; known: {sorted(table)}")
    return table[kind](spec)


def build_mixer(spec):
    return _build(MIXERS, "mixer", spec)


def build_feed_forward(spec):
    return _build(FEED_FORWARDS, "feed-forward", spec)


def build_norm(spec):
    return _build(NORMS, "norm", spec)


def build_position_encoding(spec):
    return _build(POSITION_ENCODINGS, "position encoding", spec)


def build_block(spec):
    return _build(BLOCKS, "block", spec)
