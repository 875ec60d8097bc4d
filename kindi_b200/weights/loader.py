"""Loading a model folder's tensors by name, checked against what the model expects.

The model states what it needs (``name -> shape``); the folder's files say what they hold. Everything that does
not fit - missing names, names nobody asked for, wrong shapes, unusable dtypes - is collected and raised as one
``WeightError`` that lists all of it, before anything is copied to the device. (The reference reads tensors by name
from its file's table, ``kindi/nanbeige.py:399-402,577-599``, and fails on the first problem.)

Storage types: a tensor stored in bfloat16 stays bfloat16; a tensor stored in 32-bit stays 32-bit; float16 and
float64 become 32-bit; integer tables become int32. With ``dtype="float32"`` every floating tensor becomes 32-bit
(an exact widening), so that the whole model runs in true 32-bit.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from .safetensors_io import SafetensorsFile, SafetensorsError, folder_files


class WeightError(ValueError):
    """The folder's tensors do not fit the model. ``missing``, ``unexpected`` and ``wrong_shape`` hold the names."""

    def __init__(self, msg, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=()):
        super().__init__(msg)
        self.missing = tuple(missing)
        self.unexpected = tuple(unexpected)
        self.wrong_shape = tuple(wrong_shape)
        self.wrong_dtype = tuple(wrong_dtype)


def _some(names: Sequence[str], limit: int = 12) -> str:
    names = list(names)
    s = ", ".join(names[:limit])
    return s + (", ... (%d more)" % (len(names) - limit) if len(names) > limit else "")


def target_dtype(stored: torch.dtype, run_dtype: str) -> torch.dtype:
    if stored in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8):
        return torch.int32
    if run_dtype == "float32":
        return torch.float32
    if stored == torch.bfloat16:
        return torch.bfloat16
    return torch.float32


def load_tensors(model_dir: str, expected: Mapping[str, Tuple[int, ...]], *, run_dtype: str = "bfloat16",
                 device: str = "cpu", optional: Sequence[str] = ()) -> Dict[str, torch.Tensor]:
    """read the tensors named in ``expected`` (name -> shape) from the folder's safetensors files.

    ``optional`` names may be absent (a tied head). Raises one ``WeightError`` naming every problem."""
    try:
        paths = folder_files(model_dir)
    except (OSError, KeyError, ValueError) as e:
        raise WeightError("cannot list the safetensors files of %s: %s" % (model_dir, e))
    if not paths:
        raise WeightError("no *.safetensors file in %s" % model_dir)
    files: List[SafetensorsFile] = []
    where: Dict[str, SafetensorsFile] = {}
    dup: List[str] = []
    try:
        for p in paths:
            f = SafetensorsFile(p)
            files.append(f)
            for name in f.entries:
                if name in where:
                    dup.append(name)
                where[name] = f
    except (OSError, SafetensorsError) as e:
        raise WeightError(str(e))
    opt = set(optional)
    missing = sorted(n for n in expected if n not in where and n not in opt)
    unexpected = sorted(n for n in where if n not in expected)
    wrong_shape, wrong_dtype = [], []
    for n, shape in expected.items():
        if n in where:
            dt, found = where[n].entries[n]
            if tuple(found) != tuple(shape):
                wrong_shape.append((n, tuple(shape), tuple(found)))
            if dt == "BOOL":
                wrong_dtype.append((n, dt))
    if missing or unexpected or wrong_shape or wrong_dtype or dup:
        lines = ["the tensors in %s do not fit the model:" % model_dir]
        if missing:
            lines.append("  missing (%d): %s" % (len(missing), _some(missing)))
        if unexpected:
            lines.append("  unexpected (%d): %s" % (len(unexpected), _some(unexpected)))
        if wrong_shape:
            lines.append("  wrong shape (%d): %s" % (len(wrong_shape), _some(
                ["%s expected %s found %s" % (n, list(a), list(b)) for n, a, b in wrong_shape])))
        if wrong_dtype:
            lines.append("  unusable dtype (%d): %s" % (len(wrong_dtype), _some(
                ["%s is %s" % (n, d) for n, d in wrong_dtype])))
        if dup:
            lines.append("  stored in more than one file (%d): %s" % (len(dup), _some(sorted(dup))))
        raise WeightError("\n".join(lines), missing, unexpected, [w[0] for w in wrong_shape],
                          [w[0] for w in wrong_dtype])
    out: Dict[str, torch.Tensor] = {}
    for n in expected:
        if n not in where:
            continue
        t = where[n].tensor(n)
        td = target_dtype(t.dtype, run_dtype)
        out[n] = t.to(device=device, dtype=td, copy=True).contiguous()
    for f in files:
        f.close()
    return out
