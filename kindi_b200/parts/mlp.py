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
from ..kernels import lib as K
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
        # gate and up rows in groups of 16: 16 gate rows, then the 16 up rows of the same outputs. A tile of the
        # product then holds both halves of its outputs (32 neighbouring accumulator columns of a prompt-sized product,
        # the two half-warps of 32 accumulator lanes of a decode-sized one), so SwiGLU is finished in the product's
        # epilogue; the stand-alone SwiGLU kernel reads the same grouping. (Sizes that are no multiple of 16: all
        # gates, then all ups.)
        self.group = 16 if self.f % 16 == 0 else self.f
        n = self.f // self.group
        self.wgu = torch.stack([g.view(n, self.group, width), u.view(n, self.group, width)], dim=1) \
            .reshape(2 * self.f, width).contiguous()
        self.wd = weights("down_proj.weight")

    def forward(self, ctx: StepContext, y: torch.Tensor) -> Branch:
        from ..kernels import fast
        h = torch.empty((y.shape[0], self.f), dtype=self.dtype, device=y.device)
        fused = ctx.fast and self.group == 16 and (fast.gemm_swiglu_decode(y, self.wgu, h, ctx.status)
                                                   or fast.gemm_swiglu_rows(y, self.wgu, h, ctx.status))
        if not fused:
            gu = L.rows_or_planes(ctx, y, self.wgu, self.dtype)
            K.swiglu(gu, h, self.group)
        return Branch(L.planes(ctx, h, self.wd))

    def bytes_read(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.wgu, self.wd))


register_part("feed_forward", "swiglu", SwiGLU)
