"""The back end of a model: normalised hidden rows to 32-bit logits.

``logits = W y`` over the rows whose logits are wanted, no bias (``kindi/nanbeige.py:720-724``: the reference runs its
head on the last prompt row only, ``:1011-1019``). With ``tied_to`` the matrix is another tensor of the model, the
embedding table (``kindi/tp.py:850-851``: "head = token_embd when output.weight is absent"). ``scale`` multiplies the
logits and ``softcap`` bounds them by ``softcap * tanh(logits / softcap)``, for architectures that carry such
constants; the Nanbeige decoder has neither. Names and constants are parameters of the part.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..config.registry import register_part
from ..config.spec import PartSpec
from ..kernels import lib as K
from ..kernels import linear as L
from .base import Head, StepContext, WeightView


class LinearHead(Head):
    @classmethod
    def tensor_shapes(cls, spec: PartSpec, width: int) -> Dict[str, Tuple[int, ...]]:
        return {spec.get("tied_to") or spec["name"]: (int(spec["vocab"]), width)}

    def __init__(self, spec, width, weights: WeightView, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        self.weight = weights(spec.get("tied_to") or spec["name"])
        self.scale = float(spec.get("scale") or 1.0)
        self.softcap = float(spec.get("softcap") or 0.0)

    def forward(self, ctx: StepContext, y: torch.Tensor) -> torch.Tensor:
        logits = L.linear(ctx, y, self.weight, torch.float32)
        if self.scale != 1.0 or self.softcap > 0.0:
            K.logit_post(logits, self.scale, self.softcap)
        return logits

    def bytes_read(self) -> int:
        return self.weight.numel() * self.weight.element_size()


register_part("head", "linear", LinearHead)
