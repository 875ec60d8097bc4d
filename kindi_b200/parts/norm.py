"""RMS norm with the residual add fused in front of it.

``v = x + pending branch`` (written back to the 32-bit residual), ``y = (rsqrt(mean(v^2) + eps) * v) * w`` with the
sum of squares, the scale and both products in 32-bit - the reference's ``nbq_add_rms_q8`` (``kindi/nbq.cu:412-432``)
and, for the final norm on the rows whose logits are wanted, ``nbq_add_rms`` (``kindi/nbq.cu:435-453``). The weight
multiplies as stored (no ``1 + w``). ``eps`` is a parameter of the part.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..config.registry import register_part
from ..config.spec import PartSpec
from ..kernels import lib as K
from .base import Branch, Norm, StepContext, WeightView


class RMSNorm(Norm):
    @classmethod
    def tensor_shapes(cls, spec: PartSpec, width: int) -> Dict[str, Tuple[int, ...]]:
        return {"weight": (width,)}

    @classmethod
    def tensor_init(cls, spec: PartSpec, width: int) -> Dict[str, str]:
        return {"weight": "gain"}

    def __init__(self, spec, width, weights: WeightView, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        self.eps = float(spec["eps"])
        self.weight = weights("weight")

    def add_norm(self, ctx: StepContext, x, pending: Optional[Branch], rows=None):
        n_out = x.shape[0] if rows is None else rows.numel()
        y = torch.empty((n_out, self.width), dtype=self.dtype, device=x.device)
        K.add_rmsnorm(x, None if pending is None else pending.parts, self.weight, self.eps, y, rows,
                      write_back=rows is None and pending is not None, status=ctx.status)
        return y

    def bytes_read(self) -> int:
        return self.weight.numel() * self.weight.element_size()


register_part("norm", "rmsnorm", RMSNorm)
