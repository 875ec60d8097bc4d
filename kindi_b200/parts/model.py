"""A decoder built from a ``ModelSpec``: its embedding part, the layers' blocks run in schedule order, the final norm
and its head part.

The head runs only on the rows whose logits are wanted (the reference runs its head on the last prompt row only,
``kindi/nanbeige.py:1011-1019``, and on every row of a check pass, ``:1126-1129``); logits are 32-bit.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Tuple

import torch

from ..config.registry import part_class
from ..config.spec import ModelSpec
from .base import Branch, StepContext, WeightView


def _model_parts(spec: ModelSpec):
    """(category, part spec, tensor-name prefix) of every part that hangs directly on the model"""
    yield "embedding", spec.embedding, ""
    for layer in spec.layers:
        yield "block", layer.block, layer.prefix
    yield "norm", spec.final_norm, spec.final_norm_prefix
    yield "head", spec.head, ""


def expected_tensors(spec: ModelSpec) -> Dict[str, Tuple[int, ...]]:
    """every tensor the model reads, by name, with its shape (a tensor two parts name, a tied head's, once)"""
    out: Dict[str, Tuple[int, ...]] = {}
    for category, ps, prefix in _model_parts(spec):
        for suffix, shape in part_class(category, ps.kind).tensor_shapes(ps, spec.width).items():
            name, shape = prefix + suffix, tuple(int(n) for n in shape)
            if out.setdefault(name, shape) != shape:
                raise ValueError("tensor %s is asked for with shapes %s and %s" % (name, out[name], shape))
    return out


def tensor_inits(spec: ModelSpec) -> Dict[str, str]:
    """the tensors that the random-weights mode does not draw around zero: name -> "gain" | "zero", as the parts
    that own them say"""
    out: Dict[str, str] = {}
    for category, ps, prefix in _model_parts(spec):
        for suffix, kind in part_class(category, ps.kind).tensor_init(ps, spec.width).items():
            out[prefix + suffix] = kind
    return out


def cache_needs(spec: ModelSpec) -> List:
    """the cache need of each cache entry (index = ScheduleEntry.cache)"""
    needs: List = [None] * spec.n_cache_entries
    for e in spec.schedule:
        if e.reads_cache_of is None:
            layer = spec.layers[e.layer]
            needs[e.cache] = part_class("block", layer.block.kind).cache_need(layer.block, spec.width)
    return needs


class DecoderModel:
    def __init__(self, spec: ModelSpec, tensors: Mapping[str, torch.Tensor], *, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)

        def make(category, ps, prefix):
            return part_class(category, ps.kind)(ps, spec.width, WeightView(tensors, prefix), dtype=dtype,
                                                 device=device)
        self.embedding = make("embedding", spec.embedding, "")
        self.blocks = [make("block", l.block, l.prefix) for l in spec.layers]
        self.final_norm = make("norm", spec.final_norm, spec.final_norm_prefix)
        self.head = make("head", spec.head, "")
        self.graph_safe = all(p.graph_safe for p in [self.embedding, self.final_norm, self.head] + self.blocks)

    def forward(self, ctx: StepContext, rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """run the step's tokens through every scheduled layer (keys, values and state are stored on the way);
        returns 32-bit logits ``[len(rows), vocab]`` of the listed rows, or None when no row is wanted"""
        x = self.embedding.forward(ctx)
        pending: Optional[Branch] = None
        for entry in self.spec.schedule:
            ctx.entry = entry
            pending = self.blocks[entry.layer].forward(ctx, x, pending)
        ctx.entry = None
        if rows is None or rows.numel() == 0:
            return None
        y = self.final_norm.add_norm(ctx, x, pending, rows=rows)
        return self.head.forward(ctx, y)

    def bytes_read(self, n_rows: int) -> int:
        """weight bytes one step reads: every scheduled layer once, the head once, n_rows embedding rows"""
        per_layer = [b.bytes_read() for b in self.blocks]
        total = sum(per_layer[e.layer] for e in self.spec.schedule)
        return total + self.final_norm.bytes_read() + self.head.bytes_read() + self.embedding.bytes_read(n_rows)
