"""One registry from an architecture's name to its model, and one from a part's kind to its class.

The reference picks its engine by a manifest string (``kindi/server.py:87-97``) after recognising the file's
architecture (``kindi/nanbeige_cli.py:11-15``: ``general.architecture == "llama"``), and each engine class reads its
own configuration. Here config.json's ``architectures[0]`` (or ``model_type``) picks an ``Architecture``: a reader of
that architecture's own config.json keys (``read_config``: raw JSON object -> its typed configuration) and a function
from that configuration to a ``ModelSpec`` (``build_spec``). Nothing is parsed before the name is looked up, so an
architecture with other keys (no heads, another activation) is a registry entry, not a change to this package.
Parts (embeddings, mixers, feed-forwards, norms, position encodings, block arrangements, heads) are looked up by
kind when the model is built, so a new part is one ``register_part`` call.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Optional, Tuple

from .model_config import architecture_name, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    build_spec: Callable        # (the architecture's configuration) -> ModelSpec
    read_config: Callable       # (raw JSON object of config.json) -> the architecture's configuration


_ARCHITECTURES: Dict[str, Architecture] = {}
_PARTS: Dict[Tuple[str, str], type] = {}
PART_CATEGORIES = ("embedding", "block", "mixer", "feed_forward", "norm", "position", "head")


def register_architecture(name: str, build_spec: Callable, read_config: Optional[Callable] = None, *,
                          replace: bool = False) -> None:
    """``read_config`` turns the raw JSON object of a folder's config.json into whatever ``build_spec`` takes
    (default: the raw object itself)"""
    if name in _ARCHITECTURES and not replace:
        raise KeyError("architecture %r is already registered" % name)
    _ARCHITECTURES[name] = Architecture(name, build_spec, read_config or (lambda raw: raw))


def architecture(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise KeyError("unknown architecture %r; known: %s" % (name, ", ".join(sorted(_ARCHITECTURES)))) from None


def architectures() -> Tuple[str, ...]:
    _ensure_builtin()
    return tuple(sorted(_ARCHITECTURES))


def model_from_config(raw: Mapping[str, Any]):
    """(the architecture's typed configuration, its ModelSpec) for the JSON object of a config.json: the name is
    looked up first, then the entry reads the keys it knows"""
    arch = architecture(architecture_name(raw))
    cfg = arch.read_config(raw)
    spec = arch.build_spec(cfg)
    spec.validate()
    return cfg, spec


def model_from_dir(model_dir: str):
    return model_from_config(read_config_json(model_dir))


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
