"""Run-time options, with the reference's names, meanings and defaults.

``kindi/config.py:12-48`` keeps these as a flat table of typed keys: ``ctx``, ``max_tokens`` 1024, ``temperature``
0.7, ``top_p`` 0.8, ``top_k`` 20, ``min_p`` 0, ``repeat_penalty`` 1.0, ``repeat_last_n`` 64; an unknown key is an
error (``config.py:86-88``). The same keys are used here, as explicit arguments only: no file or environment lookup
selects code paths.
"""
from __future__ import annotations

from dataclasses import dataclass, fields, replace
from typing import Optional, Tuple


@dataclass(frozen=True)
class SamplingParams:
    """How the next token is picked (``kindi/sampling.py:91-114``).

    temperature <= 0 is greedy (``sampling.py:38-39``). Otherwise: top-k (0: all), then top-p and min-p on the
    probabilities at temperature 1 (``order="llama"``; ``order="hf"`` applies the temperature before top-p, the
    reference's KINDI_SAMPLER_ORDER=hf, ``sampling.py:19,103``), then the temperature. The repeat penalty divides
    a recent token's logit when positive and multiplies it when negative (``sampling.py:117-123``) over the last
    ``repeat_last_n`` tokens (-1: the whole sequence).
    """

    temperature: float = 0.7
    top_p: float = 0.8
    top_k: int = 20
    min_p: float = 0.0
    repeat_penalty: float = 1.0
    repeat_last_n: int = 64
    max_tokens: int = 1024
    seed: Optional[int] = None
    stop_token_ids: Tuple[int, ...] = ()
    order: str = "llama"

    def __post_init__(self):
        if self.order not in ("llama", "hf"):
            raise ValueError("order must be 'llama' or 'hf', not %r" % (self.order,))
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1, found %r" % (self.max_tokens,))
        if self.top_k < 0:
            raise ValueError("top_k must be 0 (off) or positive, found %r" % (self.top_k,))
        if not (0.0 <= self.min_p <= 1.0):
            raise ValueError("min_p must lie in [0, 1], found %r" % (self.min_p,))
        if self.repeat_penalty <= 0.0:
            raise ValueError("repeat_penalty must be positive, found %r" % (self.repeat_penalty,))

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @staticmethod
    def from_options(**kw) -> "SamplingParams":
        names = {f.name for f in fields(SamplingParams)}
        bad = sorted(set(kw) - names)
        if bad:
            raise KeyError("unknown sampling option(s): %s; known: %s" % (", ".join(bad), ", ".join(sorted(names))))
        kw = {k: v for k, v in kw.items() if v is not None}
        if "stop_token_ids" in kw:
            kw["stop_token_ids"] = tuple(int(t) for t in kw["stop_token_ids"])
        return SamplingParams(**kw)

    def with_(self, **kw) -> "SamplingParams":
        return replace(self, **kw)


GREEDY = SamplingParams(temperature=0.0)


@dataclass(frozen=True)
class EngineConfig:
    """``ctx``: the most tokens all live sequences hold together (it sizes the cache; the reference's ``ctx`` is
    the same bound for its one sequence, ``kindi/nanbeige.py:245``). ``dtype``: "bfloat16" (serving kernels) or
    "float32" (every operation in true 32-bit). ``max_batch``: the most sequences that run together."""

    ctx: int = 24576
    dtype: str = "bfloat16"
    max_batch: int = 64
    device: str = "cuda:0"
    cuda_graphs: bool = True

    def __post_init__(self):
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError("dtype must be 'bfloat16' or 'float32', not %r" % (self.dtype,))
        if self.ctx < 1:
            raise ValueError("ctx must be positive, found %r" % (self.ctx,))
        if self.max_batch < 1:
            raise ValueError("max_batch must be positive, found %r" % (self.max_batch,))
