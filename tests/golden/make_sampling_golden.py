#!/usr/bin/env python3
"""Makes tests/golden/sampling_golden.json: the reference's own sampling distribution on small random logits.

The only model-side code of ahtx/kindi that imports on a CPU without CuPy is ``kindi/sampling.py`` (NumPy only): its
``distribution(cand, z, temperature, top_p, kk, min_p)`` is run here on seeded logits, and the token ids and
probabilities it returns are stored. ``tests/test_plain_cpu.py`` checks the plain implementation's
``sampling_distribution`` against this file, so the plain sampler is anchored on the reference's behaviour and not
only on its formulas. The model itself (``kindi/nanbeige.py``) needs CuPy, a GPU and a quantised GGUF file, and
cannot be run here: the plain model rests on the formulas.

Run from the repository root with the reference checkout on PYTHONPATH:
    PYTHONPATH=<path to ahtx/kindi> python tests/golden/make_sampling_golden.py
"""
import json
import os

import numpy as np

from kindi import sampling as ref


def main():
    rng = np.random.RandomState(7)
    cases = []
    for n, temperature, top_p, top_k, min_p in [
            (50, 0.7, 0.8, 20, 0.0), (50, 1.0, 1.0, 0, 0.0), (300, 0.3, 0.9, 0, 0.0), (300, 1.5, 0.5, 40, 0.05),
            (64, 0.8, 0.95, 5, 0.0), (1000, 0.7, 0.8, 20, 0.1), (17, 2.0, 0.3, 0, 0.0), (128, 0.5, 1.0, 1, 0.0)]:
        z = (rng.randn(n) * 3.0).astype(np.float32).astype(np.float64)
        ids, p = ref.distribution(np.arange(n, dtype=np.int64), z, temperature, top_p, top_k, min_p)
        cases.append({"logits": [float(v) for v in z], "temperature": temperature, "top_p": top_p, "top_k": top_k,
                      "min_p": min_p, "ids": [int(i) for i in ids], "p": [float(v) for v in p]})
    z = np.array([1.0, -2.0, 0.5, 3.0, -0.25, 0.0])
    pen = ref.penalize(np.arange(6, dtype=np.int64), z, 1.3, [3, 1, 3])
    out = {"source": "kindi/sampling.py distribution() and penalize(), SAMPLER_ORDER=%s" % ref.SAMPLER_ORDER,
           "cases": cases, "penalize": {"logits": list(z), "rp": 1.3, "recent": [3, 1, 3], "out": [float(v) for v in pen]}}
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "sampling_golden.json")
    with open(path, "w") as f:
        json.dump(out, f)
    print("wrote", path, len(cases), "cases")


if __name__ == "__main__":
    main()
