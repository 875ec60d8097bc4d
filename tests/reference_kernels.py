"""The reference's own 32-bit-in, 32-bit-out kernels beside the plain implementation.

ahtx/kindi's model cannot run here as a whole (CuPy, a quantised GGUF file), but five of its kernels take and give
plain 32-bit tensors and need no quantised weight: the fused add + RMS norm (``kindi/nbq.cu:435-453``), the rotation
with the key/value store (``:497-520``), the decode attention over position splits with its merge (``:525-649``), the
prompt attention (``kindi/nbq_fa.cu:31-161``) and the two-stage argmax (``kindi/nbq.cu:670-694``), for 5 query heads per
key/value head of size 128 (the benchmark's shape). ``tests/golden/reference_kernels_harness.cu`` includes those files
as they stand and launches them with the reference's grids; this module makes the inputs (seeded), runs the harness
(on a GPU), and computes the same outputs with ``tests/plain_model.py``.

The reference rotates adjacent pairs ``(2i, 2i+1)`` of rows stored in its file format's order; the plain model rotates
``(i, i + 64)`` of rows in the safetensors order. The two are the same function under the fixed permutation
``half[i] = adjacent[2i], half[i + 64] = adjacent[2i + 1]`` of a head's dimensions (applied to queries and keys alike,
so scores do not change), which ``to_half`` / ``to_adjacent`` apply here.
"""
from __future__ import annotations

import ctypes
import math
import os
import subprocess
from typing import Dict, Optional

import numpy as np
import torch

import plain_model as P

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
HARNESS = os.path.join(HERE, "golden", "reference_kernels_harness.cu")
GOLDEN = os.path.join(HERE, "golden", "reference_kernels.npz")

NKV, G, HD = 2, 5, 128
NH = NKV * G
CTX, N_POS, NSPLIT = 512, 300, 16          # NSPLIT as kindi/nanbeige.py:17
BASE, EPS, WIDTH, VOCAB = 70000000.0, 1e-5, 2560, 166144
DECODE_ROWS = (299, 150)                   # positions of the two decode queries
PREFILL = {"a": (0, 70, (0, 1, 13, 63, 64, 69)), "b": (100, 40, (0, 20, 39))}     # pos0, tokens, rows kept
ROPE_ROWS = (0, 150, 299)


def reference_dir() -> Optional[str]:
    """where kindi/nbq.cu lies: the copy that travels with the repository's baseline folder, else a checkout named by
    KINDI_REFERENCE"""
    for d in (os.path.join(ROOT, "baseline", "_ref", "kindi"), os.path.join(os.environ.get("KINDI_REFERENCE", ""), "kindi")):
        if all(os.path.isfile(os.path.join(d, f)) for f in ("nbq.cu", "nbq_fa.cu", "nbq_grids.h")):
            return d
    return None


def build(out_dir: str) -> ctypes.CDLL:
    ref = reference_dir()
    if ref is None:
        raise FileNotFoundError("kindi/nbq.cu, nbq_fa.cu and nbq_grids.h are not at hand")
    lib = os.path.join(out_dir, "libkindi_reference_kernels.so")
    cmd = ["nvcc", "-shared", "-Xcompiler", "-fPIC", "-std=c++14", "-use_fast_math", "-w", "-gencode",
           "arch=compute_100a,code=sm_100a", "-I", ref, HARNESS, "-o", lib]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed on the reference's kernels:\n" + r.stderr[-3000:])
    return ctypes.CDLL(lib)


def inputs() -> Dict[str, np.ndarray]:
    rng = np.random.RandomState(20251)
    f = lambda *s: rng.standard_normal(s).astype(np.float32)
    d = {"x": f(WIDTH), "add": f(WIDTH) * 0.3, "w": (1.0 + 0.1 * f(WIDTH)),
         "q": f(N_POS, NH * HD), "k": f(N_POS, NKV * HD), "v": f(N_POS, NKV * HD), "logits": f(VOCAB) * 2.0}
    d["logits"][777] = d["logits"][99999] = d["logits"].max() + 1.0           # an exact tie of the two best
    return d


def to_half(x: torch.Tensor) -> torch.Tensor:
    """a head's dimensions from the adjacent-pair order to the rotate-half order (last axis = HD)"""
    return torch.cat([x[..., 0::2], x[..., 1::2]], dim=-1)


def to_adjacent(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.stack([x[..., :h], x[..., h:]], dim=-1).reshape(x.shape)


# --------------------------------------------------------------------------------------------- the reference (GPU)
def run_reference(lib: ctypes.CDLL) -> Dict[str, np.ndarray]:
    dev = "cuda"
    d = {k: torch.from_numpy(v).to(dev) for k, v in inputs().items()}
    p = lambda t: ctypes.c_void_p(t.data_ptr())

    def ok(rc, what):
        if rc != 0:
            raise RuntimeError("%s: CUDA error %d" % (what, rc))
    out: Dict[str, np.ndarray] = {}
    y = torch.empty(WIDTH, device=dev)
    ok(lib.ref_add_rms(p(d["x"]), p(d["add"]), p(d["w"]), WIDTH, ctypes.c_float(EPS), p(y)), "add_rms")
    out["rms_add"] = y.cpu().numpy().copy()
    ok(lib.ref_add_rms(p(d["x"]), None, p(d["w"]), WIDTH, ctypes.c_float(EPS), p(y)), "add_rms")
    out["rms"] = y.cpu().numpy().copy()
    # every position's query is rotated in place and its key and value go to the fp16 cache (zero-filled, as the
    # reference allocates it: kindi/nanbeige.py:587-594)
    kc = torch.zeros(NKV * CTX * HD, dtype=torch.float16, device=dev)
    vc = torch.zeros(NKV * CTX * HD, dtype=torch.float16, device=dev)
    q = d["q"].clone()
    theta_scale = float(np.float32(BASE ** (-2.0 / HD)))                      # kindi/nanbeige.py:683
    pos = torch.arange(N_POS, dtype=torch.int32, device=dev)
    for t in range(N_POS):
        ok(lib.ref_rope_store(p(q[t]), p(d["k"][t]), p(d["v"][t]), p(pos[t:]), NH, NKV, ctypes.c_float(theta_scale),
                              p(kc), p(vc), CTX), "rope_store")
    out["q_rotated"] = q[list(ROPE_ROWS)].cpu().numpy().copy()
    scale = 1.0 / math.sqrt(HD)
    rows = len(DECODE_ROWS)
    qd = q[list(DECODE_ROWS)].contiguous()
    pd = torch.tensor(DECODE_ROWS, dtype=torch.int32, device=dev)
    part_o = torch.zeros(rows * NH * NSPLIT * HD, device=dev)
    part_ms = torch.zeros(rows * NH * NSPLIT * 2, device=dev)
    o = torch.empty(rows, NH * HD, device=dev)
    ok(lib.ref_attn_decode_g5(p(qd), p(kc), p(vc), p(pd), CTX, ctypes.c_float(scale), p(part_o), p(part_ms), NH * HD,
                              NKV, NSPLIT, rows, p(o)), "attn_decode")
    out["decode"] = o.cpu().numpy().copy()
    for name, (pos0, nt, keep) in PREFILL.items():
        qp = q[pos0:pos0 + nt].contiguous()
        o = torch.empty(nt, NH * HD, device=dev)
        ok(lib.ref_fa_prefill_g5(p(qp), NH * HD, nt, pos0, p(kc), p(vc), CTX, ctypes.c_float(scale), p(o), NKV),
           "fa_prefill")
        out["prefill_" + name] = o[list(keep)].cpu().numpy().copy()
    pv = torch.empty(256, device=dev)
    pi = torch.empty(256, dtype=torch.int32, device=dev)
    best = torch.zeros(1, dtype=torch.int32, device=dev)
    ok(lib.ref_argmax(p(d["logits"]), VOCAB, p(pv), p(pi), p(best)), "argmax")
    out["argmax"] = best.cpu().numpy().copy()
    return out


# --------------------------------------------------------------------------------------------- the plain implementation
def run_plain() -> Dict[str, np.ndarray]:
    d = {k: torch.from_numpy(v).double() for k, v in inputs().items()}
    out: Dict[str, np.ndarray] = {}
    out["rms_add"] = P.rms_norm(d["x"] + d["add"], d["w"], EPS).numpy()
    out["rms"] = P.rms_norm(d["x"], d["w"], EPS).numpy()
    cos, sin = P.rope_tables(torch.arange(N_POS), HD, BASE, torch.float64)
    q = P.rope_rotate_half(to_half(d["q"].view(N_POS, NH, HD)), cos, sin)
    k = P.rope_rotate_half(to_half(d["k"].view(N_POS, NKV, HD)), cos, sin)
    v = d["v"].view(N_POS, NKV, HD)
    out["q_rotated"] = to_adjacent(q)[list(ROPE_ROWS)].reshape(len(ROPE_ROWS), NH * HD).numpy()
    # the reference keeps keys and values in fp16; the plain attention is given the same rounded tensors
    k16, v16 = k.to(torch.float16).double(), v.to(torch.float16).double()
    att = P.attention(q, k16, v16, 1.0 / math.sqrt(HD)).reshape(N_POS, NH * HD)
    out["decode"] = att[list(DECODE_ROWS)].numpy()
    for name, (pos0, nt, keep) in PREFILL.items():
        out["prefill_" + name] = att[[pos0 + r for r in keep]].numpy()
    out["argmax"] = np.array([P.greedy(d["logits"].numpy())], dtype=np.int32)
    return out


# what the comparison allows: max |a - b| / max |b|. Norm: one rounding of rsqrt and two products. Rotation: fast-math
# sine and cosine of angles up to 299 radians. Attention: the reference's exponentials are fast-math; the prompt
# kernel also rounds the scaled queries and the probabilities to fp16 (kindi/nbq_fa.cu:1-6).
# (Measured on a B200: 8e-8, 1.4e-5, 1.9e-5 and 2.7e-4.)
TOLERANCE = {"rms_add": 1e-6, "rms": 1e-6, "q_rotated": 1e-4, "decode": 2e-4, "prefill_a": 1.5e-3, "prefill_b": 1.5e-3}


def compare(ref: Dict[str, np.ndarray], plain: Dict[str, np.ndarray]) -> Dict[str, float]:
    errs = {}
    for name, tol in TOLERANCE.items():
        a, b = np.asarray(ref[name], dtype=np.float64), np.asarray(plain[name], dtype=np.float64)
        assert a.shape == b.shape, (name, a.shape, b.shape)
        errs[name] = float(np.abs(a - b).max() / np.abs(b).max())
        assert errs[name] <= tol, "%s: the reference's kernel and the plain function differ by %.3g (allowed %.3g)" % (
            name, errs[name], tol)
    assert int(ref["argmax"][0]) == int(plain["argmax"][0]) == 777, (ref["argmax"], plain["argmax"])
    return errs
