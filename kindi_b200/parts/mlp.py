"""SwiGLU feed-forward: ``h = silu(Wg y) * (Wu y)``, branch ``= Wd h``; no biases.

Gate and up run as one product over the concatenated weights (the reference's fused gate/up launch,
``kindi/nanbeige.py:710-716``), ``silu(g) * u = g / (1 + exp(-g)) * u`` in 32-bit (``kindi/nbq.cu:461-467``), then
the down product (``kindi/nanbeige.py:718``). The intermediate size is a parameter of the part.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..config.registry import register_part
from ..config.spec import PartSpec
from ..kernels import linear as L
from .base import Branch, FeedForward, StepContext, WeightView


class SwiGLU(FeedForward):
    @classmethod
    def tensor_shapes(cls, spec: PartSpec, width: int) -> Dict[str, Tuple[int, ...]]:
        f = int(spec["intermediate"])
        return {"gate_proj.weight": (f, width), "up_proj.weight": (f, width), "down_proj.weight": (width, f)}

    def __init__(self, spec, width, weights: WeightView, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        self.f = int(spec["intermediate"])
        g, u = weights("gate_proj.weight"), weights("up_proj.weight")
        if g.dtype != u.dtype:
            raise ValueError("gate and up weights of %s are stored in different dtypes" % weights.prefix)
        # gate and up rows are put together in the order the products' SwiGLU epilogues want (the kernels' choice)
        self.wgu, self.group = L.join_gate_up(g, u)
        self.wd = weights("down_proj.weight")

    def forward(self, ctx: StepContext, y: torch.Tensor) -> Branch:
        h = L.gate_up_swiglu(ctx, y, self.wgu, self.group, self.f, self.dtype)
        return Branch(L.planes(ctx, h, self.wd))

    def bytes_read(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.wgu, self.wd))


register_part("feed_forward", "swiglu", SwiGLU)
