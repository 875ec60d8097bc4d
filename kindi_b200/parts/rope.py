"""Position encodings. The attention mixer hands its projections to its position encoding, which rotates queries
and keys and stores keys and values (one fused kernel); an encoding that is a rotation also offers its table
(``inv_freq[i]`` for each rotated pair and the number of rotated dimensions) to kernels that rotate on the fly.

Rotary (rotate-half pairing, for tensors in the safetensors layout): pair ``(i, i + rot/2)``, angle
``float(pos) * inv_freq[i]`` with ``inv_freq[i] = base ** (-2 i / rot)`` rounded to 32-bit; the reference's form
for such tensors is ``kindi/dspine.cu:151-174`` (angle in 32-bit, ``a c - b s`` / ``b c + a s``), its GGUF path
rotates adjacent pairs of permuted rows, which is the same function (``kindi/nbq.cu:497-520``); the base defaults
to 10000.0 (``kindi/nanbeige.py:256``). ``NoPosition`` rotates nothing.
"""
from __future__ import annotations

import torch

from ..config.registry import register_part
from ..kernels import lib as K
from .base import PositionEncoding


class RotationEncoding(PositionEncoding):
    """a rotation of the pairs (i, i + rotary_dim / 2) by pos * inv_freq[i]; subclasses set ``inv_freq`` (float32
    ``[max(1, rotary_dim / 2)]`` on the device) and ``rotary_dim`` (even, at most the head size; 0 rotates nothing)"""

    # a hashable name of the frequency table when parts of other layers may have the very same one (then a step
    # computes its rows' cosines and sines once and every such part uses them); None: this part's table is its own
    angles_key = None

    def rotation(self):
        return self.inv_freq, self.rotary_dim

    def encode_and_store(self, ctx, qkv, q_out, n_heads, n_kv_store, head_dim, pool, table, n_pages) -> None:
        angles = None
        if self.angles_key is not None and ctx.T >= K.rope_table_min_rows() and self.rotary_dim >= 16:
            angles = ctx.scratch.get(self.angles_key)
            if angles is None:
                angles = ctx.scratch[self.angles_key] = K.rope_table(ctx.pos, self.inv_freq, self.rotary_dim)
        K.rope_store(qkv, q_out, self.inv_freq, self.rotary_dim, ctx.pos, ctx.seq, ctx.slot, n_heads, n_kv_store,
                     head_dim, pool if n_kv_store else None, table, n_pages, ctx.status, angles)


class Rotary(RotationEncoding):
    def __init__(self, spec, width, weights, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        self.base = float(spec["base"])
        self.rotary_dim = int(spec["rotary_dim"])
        if self.rotary_dim % 2 or self.rotary_dim <= 0:
            raise ValueError("rotary_dim must be even and positive, found %d" % self.rotary_dim)
        i = torch.arange(0, self.rotary_dim // 2, dtype=torch.float64)
        self.inv_freq = (self.base ** (-2.0 * i / self.rotary_dim)).to(torch.float32).to(device)
        self.angles_key = ("rotary", self.base, self.rotary_dim)


class NoPosition(RotationEncoding):
    def __init__(self, spec, width, weights, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        self.rotary_dim = 0
        self.inv_freq = torch.zeros(1, dtype=torch.float32, device=device)


register_part("position", "rotary", Rotary)
register_part("position", "none", NoPosition)
