"""Seeded random weights: as tensors, or written out as a model folder (config.json + model.safetensors).

Every tensor is drawn from N(0, std) unless the part that owns it says otherwise: gains (a norm's weight) are
``1 + N(0, std)`` (a gain near 0.02 would be valid arithmetic but shrinks every logit towards zero, which hides
faults), biases are zero. Each tensor has a generator
of its own, seeded from the run's seed and the tensor's name, so the values do not depend on the order in which
tensors are made or on which tensors exist. The reference has no such mode (it always reads a real model file).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Mapping, Optional, Tuple

import torch

from ..config.registry import model_from_config
from .safetensors_io import write_file


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(("%d:%s" % (seed, name)).encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(name: str, shape: Tuple[int, ...], seed: int, std: float, dtype: torch.dtype,
                  device="cpu", init: str = "normal") -> torch.Tensor:
    """``init``: "normal" is N(0, std), "gain" is 1 + N(0, std), "zero" is all zeros"""
    if init == "zero":
        return torch.zeros(shape, dtype=dtype, device=device)
    if init not in ("normal", "gain"):
        raise ValueError("tensor %s: unknown init kind %r (normal, gain, zero)" % (name, init))
    g = torch.Generator(device=device)
    g.manual_seed(_seed_for(seed, name))
    t = torch.randn(shape, generator=g, dtype=torch.float32, device=device) * std
    if init == "gain":
        t = t + 1.0
    return t.to(dtype)


def random_tensors(expected: Mapping[str, Tuple[int, ...]], seed: int, *, std: float = 0.02,
                   dtype: torch.dtype = torch.bfloat16, device="cpu",
                   inits: Optional[Mapping[str, str]] = None) -> Dict[str, torch.Tensor]:
    """``inits``: name -> "gain" | "zero" for the tensors that are not drawn around zero (``parts.model.tensor_inits``
    collects what the parts say)"""
    inits = inits or {}
    return {n: random_tensor(n, tuple(s), seed, std, dtype, device, inits.get(n, "normal"))
            for n, s in expected.items()}


def write_random_model(out_dir: str, config, seed: int, *, std: float = 0.02, dtype: str = "bfloat16") -> str:
    """write ``config.json`` and ``model.safetensors`` for the configuration with weights drawn from the seed.
    ``config``: the JSON object of a config.json (any registered architecture's), or a typed configuration that
    offers ``to_dict()``"""
    from ..parts.model import expected_tensors, tensor_inits
    raw = dict(config if isinstance(config, Mapping) else config.to_dict())
    raw["torch_dtype"] = dtype
    tdt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    _, spec = model_from_config(raw)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(raw, f, indent=2)
    tensors = random_tensors(expected_tensors(spec), seed, std=std, dtype=tdt, inits=tensor_inits(spec))
    write_file(os.path.join(out_dir, "model.safetensors"), tensors,
               metadata={"format": "pt", "seed": str(seed), "std": repr(std)})
    return out_dir
