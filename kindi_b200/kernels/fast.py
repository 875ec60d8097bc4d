"""The bfloat16 serving kernels (tensor-core matrix products, tiled attention) and the rules for when each may
run. Every function returns False / None when its kernel does not take the given operands, and the caller uses the
general kernel instead; nothing here falls back to library code."""
from __future__ import annotations

from typing import Optional

import torch

from . import lib as K

N_SM = 148                 # B200: 2 dies x 74 SMs
SMALL_M = 128              # up to here the weights go through the 128-row side of the MMA ("swap" form)


def _tc_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    """what the TMA maps need: bf16, unit inner stride, 16-byte aligned bases and row strides"""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2 and w.dim() == 2
            and a.stride(1) == 1 and w.stride(1) == 1 and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def _swap_bn(m: int) -> int:
    return 16 if m <= 16 else 32 if m <= 32 else 64 if m <= 64 else 128


def wants_planes(a: torch.Tensor, w: torch.Tensor) -> bool:
    return a.shape[0] <= SMALL_M and _tc_ok(a, w)


def _splits_for(m: int, n: int, k: int, bn: int) -> int:
    """how many ways to split K for the persistent CTAs (one per SM). Estimated time of a launch, in microseconds:
    rounds of units times the K blocks of a unit (16 KB of weights each, at one SM's share of the memory bandwidth),
    plus what the 32-bit planes cost to write and to read again by the consumer (they grow with the batch)"""
    tiles = -(-n // 128) * -(-m // bn)
    total_kb = -(-k // 64)
    us_per_kb = 16384.0 / (6.6e6 / N_SM)
    best, best_cost = 1, None
    for s in range(1, min(16, total_kb) + 1):
        kbps = -(-total_kb // s)
        if -(-total_kb // kbps) != s or (s > 1 and kbps < 2):
            continue
        rounds = -(-tiles * s // N_SM)
        cost = rounds * (kbps + 0.5) * us_per_kb + s * m * n * 4 / 6.6e6
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def _prefill_bn(m: int, n: int) -> int:
    """the width of the weight side of a prefill tile: the one whose tiles fill whole rounds of the persistent CTAs
    best (a round costs about its width; a partly filled last round costs a whole one)"""
    if n <= 64:
        return 64
    best, best_cost = 128, None
    for bn in (256, 224, 192, 160, 128):
        units = -(-m // 128) * -(-n // bn)
        cost = -(-units // N_SM) * (bn + 32)
        if best_cost is None or cost < best_cost:
            best, best_cost = bn, cost
    return best


def gemm_rows(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> bool:
    if not _tc_ok(a, w) or not out.is_contiguous():
        return False
    m, n = a.shape[0], w.shape[0]
    if m <= SMALL_M:
        K.gemm_tc(a, w, out, swap=True, bn=_swap_bn(m), splits=1, status=status)
    else:
        K.gemm_tc(a, w, out, swap=False, bn=_prefill_bn(m, n), splits=1, status=status)
    return True


def gemm_planes(a: torch.Tensor, w: torch.Tensor, status: torch.Tensor) -> Optional[torch.Tensor]:
    if not _tc_ok(a, w):
        return None
    m, k = a.shape
    n = w.shape[0]
    if m <= SMALL_M:
        bn = _swap_bn(m)
        want = _splits_for(m, n, k, bn)
        s = K.gemm_tc_splits(k, want)
        out = torch.empty((s, m, n), dtype=torch.float32, device=a.device)
        K.gemm_tc(a, w, out, swap=True, bn=bn, splits=want, status=status)
        return out
    out = torch.empty((1, m, n), dtype=torch.float32, device=a.device)
    K.gemm_tc(a, w, out[0], swap=False, bn=_prefill_bn(m, n), splits=1, status=status)
    return out


def gemm_swiglu_rows(a: torch.Tensor, w_grouped: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> bool:
    """out (bf16 [M, F]) = silu(g) * u for a prompt-sized step, finished inside the product's epilogue; w_grouped
    [2F, K] holds 64 gate rows then the 64 up rows of the same outputs, group after group. False: not taken"""
    m, n = a.shape[0], w_grouped.shape[0]
    if m <= SMALL_M or not _tc_ok(a, w_grouped) or n % 128 or not out.is_contiguous() or (n // 2) % 8:
        return False
    bn = _prefill_bn(m, n)
    K.gemm_tc(a, w_grouped, out, swap=False, bn=bn if bn in (128, 256) else 256, splits=1, status=status, swiglu=True)
    return True


def attention_bf16(ctx, q, out, nh, nkv, hd, scale, window, pool, table, n_pages) -> bool:
    """the tensor-core attention kernel, where it takes the shape: head size 64 or 128, bf16, aligned rows"""
    if hd not in (64, 128) or q.dtype != torch.bfloat16 or q.stride(0) % 8 or q.data_ptr() % 16:
        return False
    g = nh // nkv
    if ctx.decode and g <= 16:
        # position splits: two CTAs fit an SM, so as many splits as fill one wave of 2 x 148 CTAs over all
        # (sequence, key/value head) pairs, never more (a second, partly filled wave would cost a whole one)
        splits = max(1, min(64, 2 * N_SM // (ctx.B * nkv)))
        K.attn_mma(q, out, ctx.slot, ctx.q_start, ctx.kv_len, ctx.B, nh, nkv, hd, scale, window, pool, table,
                   n_pages, decode=True, grid_x=splits, status=ctx.status)
        return True
    if ctx.graph:
        return False
    if hd == 128 and g <= 128 and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0:
        # prompt-sized steps: the tcgen05 kernel (S and O in tensor memory)
        K.attn_tc(q, out, ctx.slot, ctx.q_start, ctx.kv_len, ctx.B, nh, nkv, hd, scale, window, pool, table, n_pages,
                  grid_x=-(-ctx.max_q // (128 // g)), status=ctx.status)
        return True
    K.attn_mma(q, out, ctx.slot, ctx.q_start, ctx.kv_len, ctx.B, nh, nkv, hd, scale, window, pool, table, n_pages,
               decode=False, grid_x=-(-ctx.max_q * g // 64), status=ctx.status)
    return True


def gate_up_swiglu(y, ffn):
    """the fused gate/up product with the SwiGLU epilogue, or None when it does not take this shape"""
    return None
