"""Matrix products ``out = a @ w^T`` (weights stored ``[out, in]``, as the reference's row-major ``[out][in]``
matrices, ``kindi/nbq.cu:266-296``): the choice of kernel by dtype and shape.

float32 operands always run the fixed-order 32-bit kernel (no tensor cores: the true 32-bit path). bfloat16
operands run the tcgen05 kernels where their shape rules hold, else the general kernel.
"""
from __future__ import annotations

import torch

from . import lib as K


def linear(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """a [M, K] @ w [N, K]^T -> [M, N] in out_dtype"""
    out = torch.empty((a.shape[0], w.shape[0]), dtype=out_dtype, device=a.device)
    linear_into(a, w, out)
    return out


def linear_into(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    if a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        from . import fast
        if fast.gemm_bf16(a, w, out):
            return
    K.gemm_simt(a, w, out)


def branch(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """a branch output: 32-bit partial sums [S, M, N] whose sum over S (in order) is a @ w^T"""
    if a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        from . import fast
        parts = fast.gemm_bf16_branch(a, w)
        if parts is not None:
            return parts
    out = torch.empty((1, a.shape[0], w.shape[0]), dtype=torch.float32, device=a.device)
    K.gemm_simt(a, w, out[0])
    return out
