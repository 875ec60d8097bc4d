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

import fnmatch
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
                 device: str = "cpu", may_ignore: Sequence[str] = (), copies: Optional[Mapping[str, str]] = None,
                 log=None) -> Dict[str, torch.Tensor]:
    """read the tensors named in ``expected`` (name -> shape) from the folder's safetensors files.

    ``may_ignore``: ``fnmatch`` patterns of names the folder may hold that the model does not read. ``copies``:
    ``{name: other}``: the folder may hold ``name`` only as a bit-for-bit copy of ``other`` (a tied head stored
    beside the embedding table); a copy that differs is reported. Raises one ``WeightError`` naming every problem.
    ``log`` is told about matrices that stay in 32-bit in a bfloat16 run."""
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
    copies = dict(copies or {})
    missing = sorted(n for n in expected if n not in where)
    unexpected = sorted(n for n in where if n not in expected and n not in copies
                        and not any(fnmatch.fnmatchcase(n, pat) for pat in may_ignore))
    wrong_shape, wrong_dtype, differs = [], [], []
    for n, other in copies.items():
        if n in where and other in where and n not in expected:
            a, b = where[n].tensor(n), where[other].tensor(other)
            if a.shape != b.shape or a.dtype != b.dtype or not torch.equal(a, b):
                differs.append((n, other))
    for n, shape in expected.items():
        if n in where:
            dt, found = where[n].entries[n]
            if tuple(found) != tuple(shape):
                wrong_shape.append((n, tuple(shape), tuple(found)))
            if dt == "BOOL":
                wrong_dtype.append((n, dt))
    if missing or unexpected or wrong_shape or wrong_dtype or dup or differs:
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
        if differs:
            lines.append("  stored beside the tensor it should equal, and different (%d): %s" % (len(differs), _some(
                ["%s != %s" % (n, o) for n, o in differs])))
        if dup:
            lines.append("  stored in more than one file (%d): %s" % (len(dup), _some(sorted(dup))))
        raise WeightError("\n".join(lines), missing, unexpected + [n for n, _ in differs],
                          [w[0] for w in wrong_shape], [w[0] for w in wrong_dtype])
    out: Dict[str, torch.Tensor] = {}
    wide: List[str] = []
    for n in expected:
        t = where[n].tensor(n)
        td = target_dtype(t.dtype, run_dtype)
        if run_dtype == "bfloat16" and td == torch.float32 and t.dim() >= 2:
            wide.append(n)
        out[n] = t.to(device=device, dtype=td, copy=True).contiguous()
    if wide and log is not None:
        # a tensor stored in 32-bit stays 32-bit; its products then cannot use the bfloat16 tensor-core kernels
        log("%d matrices of %s are stored in 32-bit and stay so (%s): their products run the general kernel with "
            "32-bit weights, many times slower than the bfloat16 tensor-core kernels; store the folder in bfloat16 "
            "for serving speed" % (len(wide), model_dir, _some(wide, 3)))
    for f in files:
        f.close()
    return out
