"""The front end of a model: token ids to rows of the 32-bit residual stream.

``x[t] = table[tok[t]]``, the row as stored, without the scaling by the square root of the width that some
architectures apply (``kindi/nbq.cu:472-487``; ``kindi/nanbeige.py:577,681``); an architecture that does scale gives
``scale``. The tensor's full name, the vocabulary size and the scale are parameters of the part. An architecture
whose front end is something else (a learned position table added in, several tables) registers its own part of the
category "embedding" with the same ``forward``.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..config.registry import register_part
from ..config.spec import PartSpec
from ..kernels import lib as K
from .base import Embedding, StepContext, WeightView


class TokenEmbedding(Embedding):
    @classmethod
    def tensor_shapes(cls, spec: PartSpec, width: int) -> Dict[str, Tuple[int, ...]]:
        return {spec["name"]: (int(spec["vocab"]), width)}

    def __init__(self, spec, width, weights: WeightView, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        self.table = weights(spec["name"])
        self.scale = float(spec.get("scale") or 1.0)

    def forward(self, ctx: StepContext) -> torch.Tensor:
        x = torch.empty((ctx.T, self.width), dtype=torch.float32, device=self.table.device)
        K.embed(self.table, ctx.tok, x, ctx.status, self.scale)
        return x

    def bytes_read(self, n_rows: int = 0) -> int:
        return n_rows * self.width * self.table.element_size()


register_part("embedding", "table", TokenEmbedding)
