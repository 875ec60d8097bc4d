"""The plain implementation against stored outputs of the reference's own kernels (``tests/golden/reference_kernels.npz``,
made on a B200 by ``tests/golden/make_reference_kernel_golden.py``): RMS norm with and without the added branch,
rotation of queries, decode attention over 300 and 151 cached positions, prompt attention from position 0 and from
position 100, and the argmax with an exact tie."""
import numpy as np

import reference_kernels as R


def test_plain_functions_equal_the_references_kernels():
    ref = dict(np.load(R.GOLDEN))
    errs = R.compare(ref, R.run_plain())
    assert set(errs) == set(R.TOLERANCE)


def test_the_comparison_can_fail():
    """the stored outputs are not trivially matched: another pairing of the rotated dimensions, an unscaled score or a
    dropped key are all far outside the tolerances"""
    import math
    import torch
    import plain_model as P
    ref = dict(np.load(R.GOLDEN))
    d = {k: torch.from_numpy(v).double() for k, v in R.inputs().items()}
    cos, sin = P.rope_tables(torch.arange(R.N_POS), R.HD, R.BASE, torch.float64)
    q_wrong = P.rope_rotate_half(d["q"].view(R.N_POS, R.NH, R.HD), cos, sin)      # rotate-half on adjacent-pair rows
    got = q_wrong[list(R.ROPE_ROWS)].reshape(len(R.ROPE_ROWS), -1).numpy()
    assert np.abs(got - ref["q_rotated"]).max() / np.abs(ref["q_rotated"]).max() > 0.1
    q = P.rope_rotate_half(R.to_half(d["q"].view(R.N_POS, R.NH, R.HD)), cos, sin)
    k = P.rope_rotate_half(R.to_half(d["k"].view(R.N_POS, R.NKV, R.HD)), cos, sin)
    v = d["v"].view(R.N_POS, R.NKV, R.HD)
    unscaled = P.attention(q, k, v, 1.0).reshape(R.N_POS, -1)[list(R.DECODE_ROWS)].numpy()
    assert np.abs(unscaled - ref["decode"]).max() / np.abs(ref["decode"]).max() > 0.1
    short = P.attention(q[1:], k[1:], v[1:], 1.0 / math.sqrt(R.HD)).reshape(R.N_POS - 1, -1)[[298, 149]].numpy()
    assert np.abs(short - ref["decode"]).max() / np.abs(ref["decode"]).max() > 10 * R.TOLERANCE["decode"]
