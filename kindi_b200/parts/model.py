"""A decoder built from a ``ModelSpec``: embedding, the layers' blocks run in schedule order, final norm, head.

The head runs only on the rows whose logits are wanted (the reference runs its head on the last prompt row only,
``kindi/nanbeige.py:1011-1019``, and on every row of a check pass, ``:1126-1129``); logits are 32-bit.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Tuple

import torch

from ..config.registry import part_class
from ..config.spec import ModelSpec
from ..kernels import lib as K
from ..kernels import linear as L
from .base import Branch, StepContext, WeightView


def expected_tensors(spec: ModelSpec) -> Dict[str, Tuple[int, ...]]:
    """every tensor the model reads, by name, with its shape"""
    out: Dict[str, Tuple[int, ...]] = {spec.embedding_name: (spec.vocab_size, spec.width)}
    for layer in spec.layers:
        cls = part_class("block", layer.block.kind)
        for suffix, shape in cls.tensor_shapes(layer.block, spec.width).items():
            out[layer.prefix + suffix] = tuple(shape)
    ncls = part_class("norm", spec.final_norm.kind)
    for suffix, shape in ncls.tensor_shapes(spec.final_norm, spec.width).items():
        out[spec.final_norm_prefix + suffix] = tuple(shape)
    if spec.head_name is not None:
        out[spec.head_name] = (spec.vocab_size, spec.width)
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
        self.embedding = tensors[spec.embedding_name]
        self.blocks = [part_class("block", l.block.kind)(l.block, spec.width, WeightView(tensors, l.prefix),
                                                         dtype=dtype, device=device) for l in spec.layers]
        self.final_norm = part_class("norm", spec.final_norm.kind)(
            spec.final_norm, spec.width, WeightView(tensors, spec.final_norm_prefix), dtype=dtype, device=device)
        self.head = self.embedding if spec.head_name is None else tensors[spec.head_name]
        self.graph_safe = all(b.graph_safe for b in self.blocks) and self.final_norm.graph_safe

    def forward(self, ctx: StepContext, rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """run the step's tokens through every scheduled layer (keys, values and state are stored on the way);
        returns 32-bit logits ``[len(rows), vocab]`` of the listed rows, or None when no row is wanted"""
        x = torch.empty((ctx.T, self.spec.width), dtype=torch.float32, device=self.device)
        K.embed(self.embedding, ctx.tok, x, ctx.status)
        pending: Optional[Branch] = None
        for entry in self.spec.schedule:
            ctx.entry = entry
            pending = self.blocks[entry.layer].forward(ctx, x, pending)
        ctx.entry = None
        if rows is None or rows.numel() == 0:
            return None
        y = self.final_norm.add_norm(ctx, x, pending, rows=rows)
        return L.linear(ctx, y, self.head, torch.float32)

    def bytes_read(self, n_rows: int) -> int:
        """weight bytes one step reads: every scheduled layer once, the head once, n_rows embedding rows"""
        per_layer = [b.bytes_read() for b in self.blocks]
        total = sum(per_layer[e.layer] for e in self.spec.schedule)
        total += self.final_norm.bytes_read() + self.head.numel() * self.head.element_size()
        total += n_rows * self.spec.width * self.embedding.element_size()
        return total
