"""One registry from an architecture's name to its model, and one from a part's kind to its class.

The reference picks its engine by a manifest string (``kindi/server.py:87-97``) after recognising the file's
architecture (``kindi/nanbeige_cli.py:11-15``: ``general.architecture == "llama"``); here config.json's
``architectures[0]`` (or ``model_type``) picks an ``Architecture``: a function from the typed configuration to a
``ModelSpec``. Parts (mixers, feed-forwards, norms, position encodings, block arrangements) are looked up by kind
when the model is built, so a new part is one ``register_part`` call and needs no change to this package.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Tuple


@dataclass(frozen=True)
class Architecture:
    name: str
    build_spec: Callable        # (ModelConfig) -> ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}
_PARTS: Dict[Tuple[str, str], type] = {}
PART_CATEGORIES = ("block", "mixer", "feed_forward", "norm", "position")


def register_architecture(name: str, build_spec: Callable, *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise KeyError("architecture %r is already registered" % name)
    _ARCHITECTURES[name] = Architecture(name, build_spec)


def architecture(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise KeyError("unknown architecture %r; known: %s" % (name, ", ".join(sorted(_ARCHITECTURES)))) from None


def architectures() -> Tuple[str, ...]:
    _ensure_builtin()
    return tuple(sorted(_ARCHITECTURES))


def register_part(category: str, kind: str, cls: type, *, replace: bool = False) -> None:
    if category not in PART_CATEGORIES:
        raise KeyError("unknown part category %r; categories: %s" % (category, ", ".join(PART_CATEGORIES)))
    if (category, kind) in _PARTS and not replace:
        raise KeyError("%s part %r is already registered" % (category, kind))
    _PARTS[(category, kind)] = cls


def part_class(category: str, kind: str) -> type:
    _ensure_builtin()
    try:
        return _PARTS[(category, kind)]
    except KeyError:
        known = sorted(k for c, k in _PARTS if c == category)
        raise KeyError("unknown %s part %r; known: %s" % (category, kind, ", ".join(known))) from None


_builtin_done = False


def _ensure_builtin() -> None:
    """import the built-in parts and architectures once (they register themselves)"""
    global _builtin_done
    if _builtin_done:
        return
    _builtin_done = True
    from .. import parts as _parts          # noqa: F401
    from .. import models as _models        # noqa: F401
