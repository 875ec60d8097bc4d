"""Reading a model folder's ``config.json``: the file, the architecture's name, and a typed reader of keys.

Nothing here knows an architecture. The folder's ``architectures[0]`` (or ``model_type``) picks an entry of the
registry, and that entry reads its own keys through a ``ConfigReader``: every key is asked for by name with its
type, so a missing or ill-typed key is an error that names it, and when the architecture has read what it knows,
``finish()`` refuses the keys nobody asked for. The reference's rule is the same for its own configuration file:
an unknown key ends the program (``kindi/config.py:86-88``), because a key that is silently ignored is a model
that silently computes something else. Keys that carry no arithmetic (``HARMLESS_KEYS``: the writer's version,
training-time options, tokenizer hints) are let through.

No size or constant of a model stands anywhere in the package: every part receives its numbers from the
architecture's typed configuration.
"""
from __future__ import annotations

import json
import os
from typing import Any, Iterable, Mapping, Sequence, Tuple


class ConfigError(ValueError):
    """A config.json that cannot be used; the message names the key."""


# keys a config.json commonly carries that change nothing a forward pass computes
HARMLESS_KEYS = frozenset({
    "_name_or_path", "transformers_version", "use_cache", "pad_token_id", "initializer_range", "pretraining_tp",
    "attention_dropout", "hidden_dropout", "resid_pdrop", "embd_pdrop", "auto_map", "tokenizer_class",
    "output_attentions", "output_hidden_states", "return_dict", "torchscript", "is_decoder", "is_encoder_decoder",
    "add_cross_attention", "tie_encoder_decoder", "id2label", "label2id", "problem_type", "finetuning_task",
    "chunk_size_feed_forward", "use_bfloat16", "sep_token_id", "decoder_start_token_id",
    "torch_dtype", "dtype",             # how the folder's tensors are stored: the files say that themselves
})

_MISSING = object()


def read_config_json(model_dir: str) -> dict:
    """the JSON object of ``model_dir/config.json``"""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError("no config.json in %s" % model_dir)
    with open(path) as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError("config.json in %s is not valid JSON: %s" % (model_dir, e))
    if not isinstance(d, dict):
        raise ConfigError("config.json in %s must hold a JSON object" % model_dir)
    return d


def architecture_name(raw: Mapping[str, Any]) -> str:
    """``architectures[0]``, else ``model_type``: the key of the architecture registry"""
    archs = raw.get("architectures")
    if isinstance(archs, (list, tuple)) and archs and isinstance(archs[0], str):
        return archs[0]
    mt = raw.get("model_type")
    if isinstance(mt, str):
        return mt
    raise ConfigError("config.json: neither 'architectures' nor 'model_type' names the architecture")


class ConfigReader:
    """Typed access to the keys of one JSON object that remembers which keys were asked for."""

    def __init__(self, raw: Mapping[str, Any], what: str = "config.json"):
        if not isinstance(raw, Mapping):
            raise ConfigError("%s must be a JSON object, found %r" % (what, raw))
        self.raw = raw
        self.what = what
        self._used = set()

    # ------------------------------------------------------------------ typed getters
    def _value(self, key: str, default):
        self._used.add(key)
        if key not in self.raw or self.raw[key] is None:
            if default is _MISSING:
                raise ConfigError("%s: required key %r is missing" % (self.what, key))
            return _MISSING
        return self.raw[key]

    def integer(self, key: str, default=_MISSING):
        v = self._value(key, default)
        if v is _MISSING:
            return default
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError("%s: key %r must be an integer, found %r" % (self.what, key, v))
        return v

    def number(self, key: str, default=_MISSING):
        v = self._value(key, default)
        if v is _MISSING:
            return default
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError("%s: key %r must be a number, found %r" % (self.what, key, v))
        return float(v)

    def boolean(self, key: str, default=_MISSING):
        v = self._value(key, default)
        if v is _MISSING:
            return default
        if not isinstance(v, bool):
            raise ConfigError("%s: key %r must be true or false, found %r" % (self.what, key, v))
        return v

    def string(self, key: str, default=_MISSING):
        v = self._value(key, default)
        if v is _MISSING:
            return default
        if not isinstance(v, str):
            raise ConfigError("%s: key %r must be a string, found %r" % (self.what, key, v))
        return v

    def id_list(self, key: str) -> Tuple[int, ...]:
        """a token id or a list of token ids (absent: none)"""
        v = self._value(key, None)
        if v is _MISSING:
            return ()
        if isinstance(v, int) and not isinstance(v, bool):
            return (v,)
        if isinstance(v, (list, tuple)) and all(isinstance(i, int) and not isinstance(i, bool) for i in v):
            return tuple(v)
        raise ConfigError("%s: key %r must be a token id or a list of token ids, found %r" % (self.what, key, v))

    def any(self, key: str, default=None):
        """the value as it stands (lists, nested objects); the caller checks it"""
        v = self._value(key, default)
        return default if v is _MISSING else v

    # ------------------------------------------------------------------ keys that are not read
    def ignore(self, *keys: str) -> None:
        """keys this architecture knows and has no use for"""
        self._used.update(keys)

    def neutral(self, key: str, neutral_values: Sequence[Any], meaning: str) -> None:
        """a key that changes the arithmetic of models that carry it: accepted only while its value says
        that it is off"""
        self._used.add(key)
        if key in self.raw and self.raw[key] is not None and self.raw[key] not in tuple(neutral_values):
            raise ConfigError("%s: %s = %r is not supported: %s" % (self.what, key, self.raw[key], meaning))

    def finish(self, harmless: Iterable[str] = HARMLESS_KEYS) -> None:
        """every key must have been asked for, or be harmless: anything else is a model this code does not compute"""
        unknown = sorted(k for k in self.raw if k not in self._used and k not in set(harmless))
        if unknown:
            raise ConfigError("%s: unknown key%s %s: nothing in this architecture reads %s, so the model would be "
                              "computed without %s; remove the key if it is meaningless, or use an architecture that "
                              "implements it" % (self.what, "s" if len(unknown) > 1 else "",
                                                 ", ".join(repr(k) for k in unknown),
                                                 "them" if len(unknown) > 1 else "it",
                                                 "them" if len(unknown) > 1 else "it"))
