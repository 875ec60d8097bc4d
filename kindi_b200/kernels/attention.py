"""Attention over the cache: the choice of kernel by dtype and by the step's shape."""
from __future__ import annotations

from . import lib as K


def attention(ctx, q, out, nh, nkv, hd, scale, window, pool, table, n_pages) -> None:
    """``out`` = attention of the (already position-encoded) query rows ``q`` over their sequences' cached keys and
    values, which include this step's"""
    if ctx.fast:
        from . import fast
        if fast.attention_bf16(ctx, q, out, nh, nkv, hd, scale, window, pool, table, n_pages):
            return
    K.attn_generic(q, out, ctx.pos, ctx.seq, ctx.slot, nh, nkv, hd, scale, window, pool, table, n_pages, ctx.status)


def attention_from_planes(ctx, qkv, out, nh, nkv, hd, scale, window, rotation, pool, table, n_pages) -> bool:
    """a decode step of the serving kernels whose QKV product came as 32-bit planes: one kernel sums them, rotates
    queries and the newest key by ``rotation`` (``(inv_freq, rotary_dim)`` of the position encoding, None when it is
    no rotation), stores the newest key and value and attends. False: not taken (the caller encodes, stores and
    attends in separate steps)"""
    if not (ctx.fast and ctx.decode and qkv.dim() == 3 and rotation is not None):
        return False
    from . import fast
    inv_freq, rotary_dim = rotation
    return fast.attention_decode_rope(ctx, qkv, out, nh, nkv, hd, scale, window, inv_freq, rotary_dim, pool, True,
                                      table, n_pages)
