"""Causal self-attention with grouped queries over the paged cache.

``q, k, v = W y`` without biases (one product over the concatenated weights, as the reference launches its three
together, ``kindi/nanbeige.py:936-937``); the position encoding rotates q and k; k and v are stored at the row's
position of its sequence's cache; query head h reads key/value head ``h // (n_heads / n_kv_heads)``
(``kindi/nbq.cu:525-633``); scores are ``(q * scale) . k`` with ``scale = 1 / sqrt(head_dim)``
(``kindi/nanbeige.py:684``) unless the spec gives another; softmax and the weighted sum are 32-bit; the output
projection's result is the branch (``kindi/nanbeige.py:707-709``). ``window`` limits a row to the last ``window``
positions. All sizes are parameters of the part.
"""
from __future__ import annotations

import math
from typing import Dict, Tuple

import torch

from ..config.registry import part_class, register_part
from ..config.spec import PartSpec
from ..kernels import attention as A
from ..kernels import linear as L
from .base import Branch, KVNeed, Mixer, StepContext, WeightView


class CausalSelfAttention(Mixer):
    @classmethod
    def _sizes(cls, spec: PartSpec):
        return int(spec["n_heads"]), int(spec["n_kv_heads"]), int(spec["head_dim"])

    @classmethod
    def tensor_shapes(cls, spec: PartSpec, width: int) -> Dict[str, Tuple[int, ...]]:
        nh, nkv, hd = cls._sizes(spec)
        return {"q_proj.weight": (nh * hd, width), "k_proj.weight": (nkv * hd, width),
                "v_proj.weight": (nkv * hd, width), "o_proj.weight": (width, nh * hd)}

    @classmethod
    def cache_need(cls, spec: PartSpec, width: int):
        nh, nkv, hd = cls._sizes(spec)
        return KVNeed(nkv, hd, spec.get("window"))

    def __init__(self, spec, width, weights: WeightView, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        self.nh, self.nkv, self.hd = self._sizes(spec)
        if self.nh % self.nkv:
            raise ValueError("n_heads %d is not a multiple of n_kv_heads %d" % (self.nh, self.nkv))
        if self.hd % 2 or self.hd > 256:
            raise ValueError("head_dim must be even and at most 256, found %d" % self.hd)
        self.window = int(spec.get("window") or 0)
        self.scale = float(spec.get("scale") or 1.0 / math.sqrt(self.hd))
        pspec: PartSpec = spec["position"]
        self.position = part_class("position", pspec.kind)(pspec, width, weights, dtype=dtype, device=device)
        rot = self.position.rotation()
        if rot is not None and rot[1] > self.hd:
            raise ValueError("rotary_dim %d exceeds head_dim %d" % (rot[1], self.hd))
        ws = [weights("q_proj.weight"), weights("k_proj.weight"), weights("v_proj.weight")]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError("q, k and v weights of %s are stored in different dtypes" % weights.prefix)
        self.wqkv = torch.cat(ws, dim=0).contiguous()
        self.wo = weights("o_proj.weight")

    def forward(self, ctx: StepContext, y: torch.Tensor) -> Branch:
        nh, nkv, hd = self.nh, self.nkv, self.hd
        entry = ctx.entry
        reads_other = entry is not None and entry.reads_cache_of is not None
        n_q = nh * hd
        if reads_other:
            qkv = L.rows_or_planes(ctx, y, self.wqkv[:n_q], self.dtype)
            pool, table, n_pages = ctx.cache.kv_view(entry.reads_cache_of)
            store_kv = 0
        else:
            qkv = L.rows_or_planes(ctx, y, self.wqkv, self.dtype)
            pool, table, n_pages = ctx.cache.kv_view(entry.cache)
            store_kv = nkv
        att = torch.empty((ctx.T, n_q), dtype=self.dtype, device=y.device)
        if not reads_other and A.attention_from_planes(ctx, qkv, att, nh, nkv, hd, self.scale, self.window,
                                                       self.position.rotation(), pool, table, n_pages):
            # a small decode step of the serving kernels: the attention kernel summed the planes, rotated and stored
            return Branch(L.planes(ctx, att, self.wo))
        # the position encoding sums 32-bit planes, encodes and writes the queries out as rows (rows are encoded in
        # place) and stores keys and values; then attention over the cache
        q = qkv if qkv.dim() == 2 else torch.empty((ctx.T, n_q), dtype=self.dtype, device=y.device)
        self.position.encode_and_store(ctx, qkv, q, nh, store_kv, hd, pool, table, n_pages)
        A.attention(ctx, q, att, nh, nkv, hd, self.scale, self.window, pool, table, n_pages)
        return Branch(L.planes(ctx, att, self.wo))

    def bytes_read(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.wqkv, self.wo))


register_part("mixer", "attention", CausalSelfAttention)
