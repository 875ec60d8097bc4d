"""The pre-norm residual block: ``x += mixer(norm1(x)); x += feed_forward(norm2(x))``.

The adds are deferred: each norm first adds the branch that the part before it produced, so a block receives the
previous block's pending branch and returns its own (the reference's arrangement, ``kindi/nanbeige.py:688-718``:
``nbq_add_rms_q8`` adds ``br`` into ``x`` before it normalises). Which mixer, feed-forward and norms a block has is
given by its spec; the names of the sub-prefixes of its tensors are parameters too.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

from ..config.registry import part_class, register_part
from ..config.spec import PartSpec
from .base import Block, Branch, StepContext, WeightView

_DEFAULT_NAMES = {"norm1": "input_layernorm.", "mixer": "self_attn.", "norm2": "post_attention_layernorm.",
                  "feed_forward": "mlp."}
_CATEGORY = {"norm1": "norm", "mixer": "mixer", "norm2": "norm", "feed_forward": "feed_forward"}


class PreNormBlock(Block):
    @classmethod
    def _names(cls, spec: PartSpec):
        n = dict(_DEFAULT_NAMES)
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def tensor_shapes(cls, spec: PartSpec, width: int) -> Dict[str, Tuple[int, ...]]:
        out = {}
        for role, sub in cls._names(spec).items():
            ps: PartSpec = spec[role]
            for suffix, shape in part_class(_CATEGORY[role], ps.kind).tensor_shapes(ps, width).items():
                out[sub + suffix] = shape
        return out

    @classmethod
    def tensor_init(cls, spec: PartSpec, width: int) -> Dict[str, str]:
        out = {}
        for role, sub in cls._names(spec).items():
            ps: PartSpec = spec[role]
            for suffix, kind in part_class(_CATEGORY[role], ps.kind).tensor_init(ps, width).items():
                out[sub + suffix] = kind
        return out

    @classmethod
    def cache_need(cls, spec: PartSpec, width: int):
        ps: PartSpec = spec["mixer"]
        return part_class("mixer", ps.kind).cache_need(ps, width)

    def __init__(self, spec, width, weights: WeightView, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        names = self._names(spec)

        def make(role):
            ps: PartSpec = spec[role]
            return part_class(_CATEGORY[role], ps.kind)(ps, width, weights.sub(names[role]), dtype=dtype,
                                                        device=device)
        self.norm1, self.mixer, self.norm2, self.feed_forward = (make(r) for r in
                                                                 ("norm1", "mixer", "norm2", "feed_forward"))
        self.graph_safe = all(p.graph_safe for p in (self.norm1, self.mixer, self.norm2, self.feed_forward))

    def forward(self, ctx: StepContext, x, pending: Optional[Branch]) -> Optional[Branch]:
        y = self.norm1.add_norm(ctx, x, pending)
        pending = self.mixer.forward(ctx, y)
        y = self.norm2.add_norm(ctx, x, pending)
        return self.feed_forward.forward(ctx, y)

    def bytes_read(self) -> int:
        return sum(p.bytes_read() for p in (self.norm1, self.mixer, self.norm2, self.feed_forward))


register_part("block", "prenorm", PreNormBlock)
