"""Typed model configuration read from a model folder's ``config.json``.

The keys are the ones a Llama-style ``config.json`` carries; they are the same ones the reference reads where it
reads such a file (``kindi/dspine.py:220-227``: hidden_size, num_attention_heads, num_key_value_heads, head_dim,
num_hidden_layers, intermediate_size, rms_norm_eps, rope_theta or rope_parameters.rope_theta), plus what its GGUF
path takes from the file's metadata (``kindi/nanbeige.py:249-259``: block count, widths, head counts, norm epsilon,
rope base with default 10000.0, vocabulary size).

No size or constant of a model stands anywhere else in the package: every part receives its numbers from here.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that cannot be used; the message names the key."""


_MISSING = object()


def _get(d: Mapping[str, Any], key: str, typ, default=_MISSING):
    if key not in d or d[key] is None:
        if default is _MISSING:
            raise ConfigError("config.json: required key %r is missing" % key)
        return default
    v = d[key]
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError("config.json: key %r must be an integer, found %r" % (key, v))
        return v
    if typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError("config.json: key %r must be a number, found %r" % (key, v))
        return float(v)
    if typ is bool:
        if not isinstance(v, bool):
            raise ConfigError("config.json: key %r must be true or false, found %r" % (key, v))
        return v
    if typ is str:
        if not isinstance(v, str):
            raise ConfigError("config.json: key %r must be a string, found %r" % (key, v))
        return v
    return v


def _id_list(v, key) -> Tuple[int, ...]:
    if v is None:
        return ()
    if isinstance(v, int) and not isinstance(v, bool):
        return (v,)
    if isinstance(v, (list, tuple)) and all(isinstance(i, int) and not isinstance(i, bool) for i in v):
        return tuple(v)
    raise ConfigError("config.json: key %r must be a token id or a list of token ids, found %r" % (key, v))


@dataclass(frozen=True)
class ModelConfig:
    """The Llama-arch dense decoder's hyper-parameters (Nanbeige is this architecture).

    ``head_dim`` defaults to hidden_size // num_attention_heads as in ``kindi/nanbeige.py:257``; ``rope_theta``
    defaults to 10000.0 as in ``kindi/nanbeige.py:256``; ``rms_norm_eps`` has no default, as in
    ``kindi/nanbeige.py:255``.
    """

    architecture: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool = False
    max_position_embeddings: Optional[int] = None
    sliding_window: Optional[int] = None
    layer_types: Optional[Tuple[str, ...]] = None     # "full_attention" | "sliding_attention" per layer
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False, hash=False)

    @property
    def gqa_ratio(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def layer_window(self, layer: int) -> Optional[int]:
        """the attention window of a layer (None: all keys)"""
        if self.sliding_window is None:
            return None
        if self.layer_types is None:
            return self.sliding_window
        return self.sliding_window if self.layer_types[layer] == "sliding_attention" else None

    # ------------------------------------------------------------------ reading
    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "ModelConfig":
        arch = None
        archs = d.get("architectures")
        if isinstance(archs, (list, tuple)) and archs:
            arch = archs[0]
        if arch is None:
            arch = d.get("model_type")
        if not isinstance(arch, str):
            raise ConfigError("config.json: neither 'architectures' nor 'model_type' names the architecture")
        hidden = _get(d, "hidden_size", int)
        heads = _get(d, "num_attention_heads", int)
        if heads <= 0:
            raise ConfigError("config.json: num_attention_heads must be positive, found %d" % heads)
        kv = _get(d, "num_key_value_heads", int, heads)
        head_dim = _get(d, "head_dim", int, None)
        if head_dim is None:
            if hidden % heads:
                raise ConfigError("config.json: hidden_size %d is not a multiple of num_attention_heads %d and "
                                  "head_dim is not given" % (hidden, heads))
            head_dim = hidden // heads
        theta = _get(d, "rope_theta", float, None)
        if theta is None:
            rp = d.get("rope_parameters")
            if isinstance(rp, Mapping) and rp.get("rope_theta") is not None:
                theta = _get(rp, "rope_theta", float)
            else:
                theta = 10000.0
        scaling = d.get("rope_scaling")
        if scaling is None and isinstance(d.get("rope_parameters"), Mapping):
            rt = d["rope_parameters"].get("rope_type", "default")
            scaling = None if rt in ("default", None) else d["rope_parameters"]
        if scaling is not None and not (isinstance(scaling, Mapping)
                                        and scaling.get("rope_type", scaling.get("type")) in ("default", None)):
            raise ConfigError("config.json: rope_scaling %r is not supported by this architecture's position "
                              "encoding (plain rotary only)" % (scaling,))
        for k in ("attention_bias", "mlp_bias"):
            if _get(d, k, bool, False):
                raise ConfigError("config.json: %s = true is not supported (the architecture has no biases)" % k)
        act = _get(d, "hidden_act", str, "silu")
        if act != "silu":
            raise ConfigError("config.json: hidden_act %r is not supported (the feed-forward is SwiGLU: 'silu')" % act)
        window = _get(d, "sliding_window", int, None)
        if window is not None and window <= 0:
            raise ConfigError("config.json: sliding_window must be positive, found %d" % window)
        n_layers = _get(d, "num_hidden_layers", int)
        lt = d.get("layer_types")
        if lt is not None:
            if (not isinstance(lt, (list, tuple)) or len(lt) != n_layers
                    or any(t not in ("full_attention", "sliding_attention") for t in lt)):
                raise ConfigError("config.json: layer_types must list 'full_attention' or 'sliding_attention' for "
                                  "each of the %d layers, found %r" % (n_layers, lt))
            if "sliding_attention" in lt and window is None:
                raise ConfigError("config.json: layer_types names sliding_attention but sliding_window is missing")
            lt = tuple(lt)
        known = {"architectures", "model_type", "vocab_size", "hidden_size", "intermediate_size",
                 "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim", "rms_norm_eps",
                 "rope_theta", "rope_parameters", "rope_scaling", "tie_word_embeddings",
                 "max_position_embeddings", "sliding_window", "layer_types", "bos_token_id", "eos_token_id",
                 "torch_dtype", "dtype", "attention_bias", "mlp_bias", "hidden_act"}
        cfg = ModelConfig(
            architecture=arch,
            vocab_size=_get(d, "vocab_size", int),
            hidden_size=hidden,
            intermediate_size=_get(d, "intermediate_size", int),
            num_hidden_layers=n_layers,
            num_attention_heads=heads,
            num_key_value_heads=kv,
            head_dim=head_dim,
            rms_norm_eps=_get(d, "rms_norm_eps", float),
            rope_theta=theta,
            tie_word_embeddings=_get(d, "tie_word_embeddings", bool, False),
            max_position_embeddings=_get(d, "max_position_embeddings", int, None),
            sliding_window=window,
            layer_types=lt,
            bos_token_id=_get(d, "bos_token_id", int, None),
            eos_token_ids=_id_list(d.get("eos_token_id"), "eos_token_id"),
            torch_dtype=_get(d, "torch_dtype", str, None) or _get(d, "dtype", str, "bfloat16"),
            extra={k: v for k, v in d.items() if k not in known},
        )
        cfg.validate()
        return cfg

    @staticmethod
    def from_dir(model_dir: str) -> "ModelConfig":
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
        return ModelConfig.from_dict(d)

    # ------------------------------------------------------------------ checks
    def validate(self) -> None:
        for k in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "head_dim"):
            if getattr(self, k) <= 0:
                raise ConfigError("config.json: %s must be positive, found %d" % (k, getattr(self, k)))
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError("config.json: num_attention_heads %d is not a multiple of num_key_value_heads %d"
                              % (self.num_attention_heads, self.num_key_value_heads))
        if self.head_dim % 2:
            raise ConfigError("config.json: head_dim %d must be even (rotary pairs)" % self.head_dim)
        if not (self.rms_norm_eps > 0.0):
            raise ConfigError("config.json: rms_norm_eps must be positive, found %r" % self.rms_norm_eps)
        if not (self.rope_theta > 0.0):
            raise ConfigError("config.json: rope_theta must be positive, found %r" % self.rope_theta)

    def to_dict(self) -> dict:
        """the config.json that reads back as this configuration"""
        d = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "mlp_bias": False,
            "torch_dtype": self.torch_dtype,
        }
        if self.max_position_embeddings is not None:
            d["max_position_embeddings"] = self.max_position_embeddings
        if self.sliding_window is not None:
            d["sliding_window"] = self.sliding_window
        if self.layer_types is not None:
            d["layer_types"] = list(self.layer_types)
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        d.update(self.extra)
        return d
