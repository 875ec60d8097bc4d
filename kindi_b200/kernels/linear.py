"""Matrix products ``out = a @ w^T`` (weights stored ``[out, in]``, as the reference's row-major ``[out][in]``
matrices, ``kindi/nbq.cu:266-296``): the choice of kernel by dtype and shape.

float32 operands always run the fixed-order 32-bit kernel (no tensor cores: the true 32-bit path). bfloat16
operands run the tcgen05 kernel where its alignment rules hold, else the general kernel. Nothing here calls a
library product.
"""
from __future__ import annotations

import torch

from . import fast
from . import lib as K


def linear(ctx, a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """a [M, K] @ w [N, K]^T -> [M, N] in out_dtype"""
    out = torch.empty((a.shape[0], w.shape[0]), dtype=out_dtype, device=a.device)
    if not (ctx.fast and fast.gemm_rows(a, w, out, ctx.status)):
        K.gemm_simt(a, w, out)
    return out


def planes(ctx, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """a @ w^T as 32-bit partial sums [S, M, N]: their sum over S, taken in order, is the product. The consumers
    (the next norm for a branch, the rotary/store and SwiGLU kernels) add the planes themselves, so a product that
    is split over K for the sake of parallelism needs no pass of its own to be reduced"""
    if ctx.fast:
        p = fast.gemm_planes(a, w, ctx.status)
        if p is not None:
            return p
    out = torch.empty((1, a.shape[0], w.shape[0]), dtype=torch.float32, device=a.device)
    K.gemm_simt(a, w, out[0])
    return out


def rows_or_planes(ctx, a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """the product for a consumer that takes either form: 32-bit planes when the step is small (so that K can be
    split), else rows in out_dtype"""
    if ctx.fast and fast.wants_planes(a, w):
        p = fast.gemm_planes(a, w, ctx.status)
        if p is not None:
            return p
    return linear(ctx, a, w, out_dtype)


# ----------------------------------------------------------------------------------------------- gate / up / SwiGLU
GATE_UP_GROUP = 16      # rows of a gate group: a 32-column piece of a prompt-sized product's accumulator, the two
                        # half-warps of an epilogue warp of a decode-sized one


def join_gate_up(gate: torch.Tensor, up: torch.Tensor):
    """(the joined ``[2F, K]`` matrix, its group size). Gate and up rows alternate in groups of ``GATE_UP_GROUP``: 16
    gate rows, then the 16 up rows of the same outputs, so that a tile of the product holds both halves of its outputs
    and SwiGLU is finished in the product's epilogue; the stand-alone SwiGLU kernel reads the same grouping. A size
    that is no multiple of the group: all gates, then all ups (group = F)."""
    f, width = gate.shape
    group = GATE_UP_GROUP if f % GATE_UP_GROUP == 0 else f
    n = f // group
    joined = torch.stack([gate.view(n, group, width), up.view(n, group, width)], dim=1).reshape(2 * f, width)
    return joined.contiguous(), group


def gate_up_swiglu(ctx, y: torch.Tensor, wgu: torch.Tensor, group: int, f: int, out_dtype: torch.dtype) -> torch.Tensor:
    """``silu(g) * u`` (``[M, F]`` in out_dtype) with ``[g | u] = y @ wgu^T``, ``wgu`` as ``join_gate_up`` made it:
    inside the product where a tensor-core kernel takes the shape, else the product followed by the SwiGLU kernel"""
    h = torch.empty((y.shape[0], f), dtype=out_dtype, device=y.device)
    if ctx.fast and group == GATE_UP_GROUP and (fast.gemm_swiglu_decode(y, wgu, h, ctx.status)
                                                or fast.gemm_swiglu_rows(y, wgu, h, ctx.status)):
        return h
    gu = rows_or_planes(ctx, y, wgu, out_dtype)
    K.swiglu(gu, h, group)
    return h
