"""The bfloat16 serving kernels (tensor-core matrix products, tiled attention) and the rules for when each may
run. Every function returns False / None when its kernel does not take the given operands, and the caller uses the
general kernel instead; nothing here falls back to library code."""
from __future__ import annotations

import functools
from typing import Optional

import torch

from . import lib as K
from .device import DEVICE as DEV

N_SM = DEV.n_sm            # the device's own count (148 on a B200)
# A TMA tensor whose whole extent (rows x row stride) is below 128 KB is read more slowly when it is the 128-row side of
# a product: gate/up of 2560 x 20992 in the prompt form takes 28.5 us with 25 activation rows (125 KB) and 22.8 us
# with 26 (130 KB), and 22.7 us with 8 rows that lie 32 KB apart. (Found by a sweep over the row count; the decode
# forms, where the activations are the narrow side, show no such step.)
TMA_SMALL_EXTENT = 128 * 1024
SMALL_M = 128              # up to here the weights go through the 128-row side of the MMA ("swap" form)
# prompt-form products of fewer rows may split K into planes (_prefill_split): the down product of 1024 rows takes
# 51.7 us in six planes and 59.9 us in one; from 1280 rows on the plan finds nothing better than one plane
SPLIT_K_BELOW_M = 1280


def _tc_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    """what the TMA maps need: bf16, unit inner stride, 16-byte aligned bases and row strides"""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2 and w.dim() == 2
            and a.stride(1) == 1 and w.stride(1) == 1 and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def _swap_bn(m: int) -> int:
    return 16 if m <= 16 else 32 if m <= 32 else 64 if m <= 64 else 128


def wants_planes(a: torch.Tensor, w: torch.Tensor) -> bool:
    return a.shape[0] <= SMALL_M and _tc_ok(a, w)


@functools.lru_cache(maxsize=4096)
def _splits_for(m: int, n: int, k: int, bn: int) -> int:
    """how many ways to split K for the persistent CTAs (one per SM). Estimated time of a launch, in microseconds:
    rounds of units times the K blocks of a unit (16 KB of weights each, at one SM's share of the memory bandwidth),
    plus what the 32-bit planes cost to write and to read again by the consumer (they grow with the batch)"""
    tiles = -(-n // 128) * -(-m // bn)
    total_kb = -(-k // 64)
    us_per_kb = 16384.0 / (DEV.hbm_bytes_per_us / N_SM)
    best, best_cost = 1, None
    for s in range(1, min(16, total_kb) + 1):
        kbps = -(-total_kb // s)
        if -(-total_kb // kbps) != s or (s > 1 and kbps < 2):
            continue
        rounds = -(-tiles * s // N_SM)
        cost = rounds * (kbps + 0.5) * us_per_kb + s * m * n * 4 / DEV.hbm_bytes_per_us
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


@functools.lru_cache(maxsize=4096)
def _prefill_tile(m: int, n: int, k: int, swiglu: bool = False):
    """(kind, columns of a tile, variant) for a prompt-sized product: what has the least estimated time.

    kind "tc" (variant = row tiles per unit, 1 or 2): one CTA per unit. A K block of a unit costs what is slower, its
    MMAs (0.276 us for 128 x 256 x 64) or bringing its operand tiles from the L2 (about 1.15 ns per operand row); two
    row tiles over one weight tile halve the weight traffic per FLOP but leave the epilogue exposed; units fill the
    persistent CTAs in rounds and a partly filled round costs a whole one.

    kind "pair" (variant = True: the K blocks of all tiles dealt out evenly, False: tile by tile): two CTAs per
    256-row tile, each with half of the weight tile. Measured 0.36-0.39 us per K block of 256 x 256 x 64 (the rate of
    the library's product under the power limit); dealing out K blocks costs about 10 us for the tiles that two pairs
    finish together."""
    if n <= 64:
        return "tc", 64, 1
    kb = -(-k // 64)
    best, best_cost = ("tc", 128, 1), None
    for mt in ((1, 2) if m > 128 else (1,)):       # (129 to 255 rows: a second row tile that is partly empty costs less
                                                     # than a second unit; gate/up 32.0 -> 27.8 us)
        for bn in (256, 240, 224, 208, 192, 176, 160, 144, 128):
            if swiglu and bn % 32:
                continue
            units = -(-m // (128 * mt)) * -(-n // bn)
            t_kb = max(DEV.mma_us_per_kblock_128x256 * mt * bn / 256.0, DEV.l2_us_per_operand_row * (128 * mt + bn))
            epilogue = (0.02 if mt == 2 else 0.004) * bn * mt
            cost = -(-units // N_SM) * (kb * t_kb + epilogue)
            if best_cost is None or cost < best_cost:
                best, best_cost = ("tc", bn, mt), cost
    if m >= 512:
        pairs = N_SM // 2
        for bn in (256, 192, 128):
            units = -(-m // 256) * -(-n // bn)
            t_kb = max(DEV.pair_us_per_kblock_256x256 * bn / 256.0, DEV.pair_us_per_kblock_floor)
            cost = -(-units // pairs) * (kb * t_kb + 1.5)
            if cost < best_cost:
                best, best_cost = ("pair", bn, False), cost
            # (dealt out, the pairs that share an operand tile read it some K blocks apart in time: both operands have
            # to stay in the L2 meanwhile, or the product waits for DRAM: 5120 x 13824 weights, 288 us against 226)
            if not swiglu and units >= pairs and (m + n) * k * 2 <= DEV.l2_resident_bytes:
                cost = units * kb / pairs * t_kb + 10.0
                if cost < best_cost:
                    best, best_cost = ("pair", bn, True), cost
    return best


@functools.lru_cache(maxsize=4096)
def _prefill_split(m: int, n: int, k: int):
    """(columns of a tile, ways to split K) for a product of a few hundred rows whose consumer takes 32-bit planes (the
    output and down products of a short prompt or a wide decode step), or None when one plane from _prefill_tile is as
    good. With so few rows there are fewer 128-row tiles than SMs, and a tile's K loop is long (164 blocks for a
    feed-forward of 10496): splitting K fills the SMs, at the price of writing and re-reading a plane per split."""
    kb = -(-k // 64)
    best, best_cost = None, None
    for bn in (256, 192, 128):
        units = -(-m // 128) * -(-n // bn)
        t_kb = max(DEV.mma_us_per_kblock_128x256 * bn / 256.0, DEV.l2_us_per_operand_row * (128 + bn))
        for sp in (1, 2, 3, 4, 6, 8):
            kbps = -(-kb // sp)
            if sp > 1 and (kbps < 8 or units * sp > 2 * N_SM):
                continue
            z = -(-kb // kbps)
            cost = -(-units * z // N_SM) * (kbps * t_kb + 0.004 * bn + 2.0) + z * m * n * 8 / DEV.hbm_bytes_per_us
            if best_cost is None or cost < best_cost - 1e-9:
                best, best_cost = (bn, sp), cost
    return best if best is not None and best[1] > 1 else None


_PAIR_SCRATCH = {}         # device -> (partial tiles, flags): scratch of tiles that two pairs of SMs finish together


def _prefill_product(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, status: torch.Tensor, swiglu: bool) -> None:
    m, k = a.shape
    n = w.shape[0]
    kind, bn, variant = _prefill_tile(m, n, k, swiglu)
    if kind == "tc":
        K.gemm_tc(a, w, out, swap=False, bn=bn, splits=1, status=status, swiglu=swiglu, mt=variant)
        return
    part = flags = None
    if variant:
        tiles = -(-m // 256) * -(-n // bn)
        have = _PAIR_SCRATCH.get(a.device)
        if have is None or have[0].numel() < tiles * 256 * bn or have[1].numel() < 8 * tiles:
            have = (torch.empty(tiles * 256 * bn, dtype=torch.float32, device=a.device),
                    torch.zeros(8 * tiles, dtype=torch.int32, device=a.device))
            _PAIR_SCRATCH[a.device] = have
        part, flags = have
    K.gemm_pair(a, w, out, bn=bn, status=status, swiglu=swiglu, part=part, flags=flags)


def gemm_rows(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> bool:
    if not _tc_ok(a, w) or not out.is_contiguous():
        return False
    m, n = a.shape[0], w.shape[0]
    if m <= SMALL_M:
        K.gemm_tc(a, w, out, swap=True, bn=_swap_bn(m), splits=1, status=status)
    else:
        _prefill_product(a, w, out, status, False)
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
    if m < SPLIT_K_BELOW_M:
        plan = _prefill_split(m, n, k)
        if plan is not None:
            bn, want = plan
            out = torch.empty((K.gemm_tc_splits(k, want), m, n), dtype=torch.float32, device=a.device)
            K.gemm_tc(a, w, out, swap=False, bn=bn, splits=want, status=status)
            return out
    out = torch.empty((1, m, n), dtype=torch.float32, device=a.device)
    _prefill_product(a, w, out[0], status, False)
    return out


def gemm_swiglu_rows(a: torch.Tensor, w_grouped: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> bool:
    """out (bf16 [M, F]) = silu(g) * u for a prompt-sized step, finished inside the product's epilogue; w_grouped
    [2F, K] holds 16 gate rows then the 16 up rows of the same outputs, group after group. False: not taken"""
    m, n = a.shape[0], w_grouped.shape[0]
    if _swiglu_in_decode_form(a) or not _tc_ok(a, w_grouped) or n % 32 or not out.is_contiguous() or (n // 2) % 8:
        return False
    _prefill_product(a, w_grouped, out, status, True)
    return True


def _swiglu_in_decode_form(a: torch.Tensor) -> bool:
    """which of the two gate/up products that finish SwiGLU themselves takes a step of up to 128 rows: the decode form
    up to 16 rows (21.6 against 22.7 us at 8 rows), and as long as the activations are a small tensor for the TMA (17
    to 25 rows of 2560: 23.6-24.8 against 27.5-28.5 us); else the prompt form (26 to 32 rows: 22.8 against 25.1-25.7)"""
    m = a.shape[0]
    return m <= 16 or (m <= SMALL_M and m * a.stride(0) * a.element_size() < TMA_SMALL_EXTENT)


_SK_SCRATCH = {}           # (device, tiles, bn) -> (partial tiles, flags): scratch of the decode gate/up product


def reset_scratch() -> None:
    """lower every flag of the products' scratch (decode gate/up, tiles shared by two pairs of SMs): after a step whose kernels reported an error (a wait
    that ran out can leave a flag raised, which the next step would take for a partial tile that is there)"""
    for _, flags in list(_SK_SCRATCH.values()) + list(_PAIR_SCRATCH.values()):
        flags.zero_()


def gemm_swiglu_decode(a: torch.Tensor, w_grouped: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> bool:
    """out (bf16 [M, F]) = silu(g) * u for a decode-sized step, finished inside the product (no split-K planes, no
    SwiGLU kernel); w_grouped [2F, K] as for gemm_swiglu_rows. False: not taken"""
    m, n = a.shape[0], w_grouped.shape[0]
    if not _swiglu_in_decode_form(a) or not _tc_ok(a, w_grouped) or n % 32 or out.stride(1) != 1 \
            or out.dtype != torch.bfloat16:
        return False
    bn = _swap_bn(m)
    tiles = -(-n // 128)
    key = (a.device, tiles, bn)
    if key not in _SK_SCRATCH:
        _SK_SCRATCH[key] = (torch.empty(tiles * bn * 128, dtype=torch.float32, device=a.device),
                            torch.zeros(tiles, dtype=torch.int32, device=a.device))
    part, flags = _SK_SCRATCH[key]
    K.gemm_swiglu_decode(a, w_grouped, out, bn, part, flags, status)
    return True


def attention_bf16(ctx, q, out, nh, nkv, hd, scale, window, pool, table, n_pages) -> bool:
    """the tensor-core attention kernel, where it takes the shape: head size 64 or 128, bf16, aligned rows"""
    if hd not in (64, 128) or q.dtype != torch.bfloat16 or q.stride(0) % 8 or q.data_ptr() % 16:
        return False
    g = nh // nkv
    if ctx.decode and g <= 16:
        splits = decode_splits(ctx, nkv)
        K.attn_mma(q, out, ctx.slot, ctx.q_start, ctx.kv_len, ctx.B, nh, nkv, hd, scale, window, pool, table,
                   n_pages, decode=True, grid_x=splits, status=ctx.status)
        return True
    # (in a recording ctx.max_q is the most rows a sequence can bring: the grid then has tiles to spare, which leave)
    if g <= 128 and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0:
        # prompt-sized steps: the tcgen05 kernel (S and O in tensor memory)
        K.attn_tc(q, out, ctx.slot, ctx.q_start, ctx.kv_len, ctx.B, nh, nkv, hd, scale, window, pool, table, n_pages,
                  grid_x=-(-ctx.max_q // (128 // g)), status=ctx.status)
        return True
    K.attn_mma(q, out, ctx.slot, ctx.q_start, ctx.kv_len, ctx.B, nh, nkv, hd, scale, window, pool, table, n_pages,
               decode=False, grid_x=-(-ctx.max_q * g // 64), status=ctx.status)
    return True


def decode_splits(ctx, nkv: int) -> int:
    """position splits of a decode step: two CTAs fit an SM, so as many splits as fill one wave of 2 x SMs CTAs over
    all (sequence, key/value head) pairs, never more (a second, partly filled wave would cost a whole one). When that
    leaves two splits the pairs alone nearly fill the SMs, and one split without the merge kernel is as fast at long
    contexts and faster at short ones (32 sequences x 4 heads, 8 layers: 0.732 against 0.779 ms at context 512)"""
    s = 2 * N_SM // (ctx.B * nkv)
    return 1 if s <= 2 else min(64, s)


def attention_decode_rope(ctx, qkv, out, nh, nkv, hd, scale, window, inv_freq, rotary_dim, pool, store, table,
                          n_pages) -> bool:
    """a decode step's attention straight from the QKV planes (rotation and the store of the newest key and value
    inside the attention kernel), where the kernel takes the shape; False: not taken"""
    if ctx.B >= 32:
        return False        # many rows: one pass of the row-wise rotate-and-store kernel costs less than every CTA's own sums
    if not (ctx.decode and qkv.dim() == 3 and qkv.dtype == torch.float32 and hd in (64, 128) and rotary_dim == hd
            and nh // nkv <= 16 and out.dtype == torch.bfloat16 and pool.dtype == torch.bfloat16):
        return False
    if qkv.stride(2) != 1 or qkv.stride(1) != qkv.shape[2] or qkv.shape[2] % 2 or qkv.stride(0) % 2 \
            or qkv.data_ptr() % 8 or out.stride(0) % 2:
        return False
    splits = decode_splits(ctx, nkv)
    if splits == 1:
        # one CTA per (sequence, key/value head): nothing runs beside a CTA's sums and rotation, and the step is
        # slower than with the rotate-and-store kernel in front (25 / 28 / 31 sequences x 4 heads at context 8192:
        # 4.54 / 4.59 / 4.67 ms against 4.33 / 4.44 / 4.58)
        return False
    K.attn_decode_rope(qkv, inv_freq, out, ctx.slot, ctx.q_start, ctx.kv_len, ctx.B, nh, nkv, hd, scale, window, pool,
                       store, table, n_pages, grid_x=splits, status=ctx.status)
    return True
