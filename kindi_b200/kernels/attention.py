"""Attention over the cache: the choice of kernel by dtype and by the step's shape."""
from __future__ import annotations

from . import lib as K


def attention(ctx, q, out, nh, nkv, hd, scale, window, pool, table, n_pages) -> None:
    if ctx.fast:
        from . import fast
        if fast.attention_bf16(ctx, q, out, nh, nkv, hd, scale, window, pool, table, n_pages):
            return
    K.attn_generic(q, out, ctx.pos, ctx.seq, ctx.slot, nh, nkv, hd, scale, window, pool, table, n_pages, ctx.status)
