"""Each kernel alone against a plain PyTorch float32 reference of the same operation, at sizes other than the
engine's: odd widths, tile edges, head sizes in steps of 16, any number of heads and groups."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from kindi_b200.kernels import lib
    lib.load()
    return lib


def _status():
    return torch.zeros(1, dtype=torch.int32, device="cuda")


def _rel(a, b):
    return float((a.double() - b.double()).abs().max() / (b.double().abs().max() + 1e-30))


@pytest.mark.parametrize("M,N,K_", [(1, 7, 5), (3, 64, 64), (65, 130, 33), (128, 96, 200), (9, 331, 72)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_simt(K, M, N, K_, dtype):
    g = torch.Generator(device="cuda").manual_seed(M * 1000 + N)
    a = torch.randn(M, K_, device="cuda", generator=g).to(dtype)
    w = torch.randn(N, K_, device="cuda", generator=g).to(dtype)
    out = torch.empty(M, N, device="cuda", dtype=torch.float32)
    K.gemm_simt(a, w, out)
    ref = a.double() @ w.double().T
    assert _rel(out, ref) < 1e-6


# (M, N, K, swap, bn, splits): tile edges in every dimension, K tails that are no multiple of 64, both forms
TC_CASES = [
    (128, 256, 64, False, 256, 1), (128, 128, 128, False, 128, 1), (200, 300, 136, False, 128, 1),
    (2048, 512, 2560, False, 256, 1), (130, 72, 72, False, 64, 1), (257, 1000, 520, False, 256, 1),
    (1, 128, 64, True, 16, 1), (8, 384, 2560, True, 16, 1), (8, 384, 2560, True, 16, 5), (17, 200, 264, True, 32, 3),
    (64, 331 * 8, 1096, True, 64, 4), (100, 256, 4096, True, 128, 8), (5, 130, 72, True, 16, 2),
]


@pytest.mark.parametrize("M,N,K_,swap,bn,splits", TC_CASES)
def test_gemm_tc(K, M, N, K_, swap, bn, splits):
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K_)
    a = torch.randn(M, K_, device="cuda", generator=g).to(torch.bfloat16)
    w = torch.randn(N, K_, device="cuda", generator=g).to(torch.bfloat16)
    ref = a.double() @ w.double().T
    st = _status()
    S = K.gemm_tc_splits(K_, splits)
    if splits > 1:
        out = torch.full((S, M, N), float("nan"), device="cuda", dtype=torch.float32)
        K.gemm_tc(a, w, out, swap=swap, bn=bn, splits=splits, status=st)
        got = out.sum(dim=0)
    else:
        got = torch.full((M, N), float("nan"), device="cuda", dtype=torch.float32)
        K.gemm_tc(a, w, got, swap=swap, bn=bn, splits=1, status=st)
    assert int(st.item()) == 0
    assert _rel(got, ref) < 1e-5            # exact bf16 products, 32-bit accumulation
    if splits == 1:
        o16 = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        K.gemm_tc(a, w, o16, swap=swap, bn=bn, splits=1, status=st)
        assert int(st.item()) == 0
        assert _rel(o16.float(), ref) < 5e-3
