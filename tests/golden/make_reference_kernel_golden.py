#!/usr/bin/env python3
"""Makes tests/golden/reference_kernels.npz: outputs of ahtx/kindi's own CUDA kernels on small seeded inputs.

The kernels that take and give 32-bit tensors (add + RMS norm, rotation with the key/value store, decode attention with
its merge, prompt attention, argmax; ``kindi/nbq.cu``, ``kindi/nbq_fa.cu``) are compiled as they stand for sm_100a
through ``tests/golden/reference_kernels_harness.cu`` and run on a GPU; what they return is stored.
``tests/test_reference_golden_cpu.py`` checks the plain implementation against this file on any machine, and
``tests/test_reference_kernels_gpu.py`` runs the kernels again where a GPU and the sources are at hand.

Run on a machine with a B200 from the repository root, with kindi/nbq.cu, nbq_fa.cu and nbq_grids.h under
baseline/_ref/kindi/ (or KINDI_REFERENCE=<checkout of ahtx/kindi>):
    python tests/golden/make_reference_kernel_golden.py
"""
import os
import sys
import tempfile

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import reference_kernels as R          # noqa: E402


def main():
    with tempfile.TemporaryDirectory() as tmp:
        ref = R.run_reference(R.build(tmp))
    errs = R.compare(ref, R.run_plain())
    np.savez_compressed(R.GOLDEN, **ref)
    print("wrote %s (%d bytes); reference against plain: %s" % (
        R.GOLDEN, os.path.getsize(R.GOLDEN), ", ".join("%s %.2g" % kv for kv in sorted(errs.items()))))


if __name__ == "__main__":
    main()
