"""The reference's own kernels, compiled as they stand for sm_100a and run here, against the plain implementation and
against the stored outputs. Skipped where the three source files of ahtx/kindi are not at hand (they are no part of
this repository: ``baseline/_ref/kindi/`` or KINDI_REFERENCE names them)."""
import numpy as np
import pytest

import reference_kernels as R

pytestmark = pytest.mark.gpu


def test_reference_kernels_equal_plain_and_the_stored_outputs(tmp_path):
    if R.reference_dir() is None:
        pytest.skip("kindi/nbq.cu, nbq_fa.cu and nbq_grids.h are not at hand (baseline/_ref/kindi or KINDI_REFERENCE)")
    ref = R.run_reference(R.build(str(tmp_path)))
    R.compare(ref, R.run_plain())
    stored = dict(np.load(R.GOLDEN))
    for name in R.TOLERANCE:
        assert np.allclose(ref[name], stored[name], rtol=0, atol=1e-5 * np.abs(stored[name]).max()), name
