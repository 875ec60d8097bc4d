"""The bfloat16 serving kernels (tensor-core matrix products, tiled attention) and the rules for when each may
run. Every function returns False / None when its kernel does not take the given shape, and the caller uses the
general kernel instead; nothing here falls back to library code."""
from __future__ import annotations

from typing import Optional

import torch


def gemm_bf16(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    return False


def gemm_bf16_branch(a: torch.Tensor, w: torch.Tensor) -> Optional[torch.Tensor]:
    return None


def attention_bf16(ctx, q, out, nh, nkv, hd, scale, window, pool, table, n_pages) -> bool:
    return False


def gate_up_swiglu(y, ffn):
    """the fused gate/up product with the SwiGLU epilogue, or None when it does not take this shape"""
    return None
