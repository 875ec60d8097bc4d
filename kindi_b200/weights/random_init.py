"""Seeded random weights: as tensors, or written out as a model folder (config.json + model.safetensors).

Every matrix and the embedding table are drawn from N(0, std); norm gains are ``1 + N(0, std)`` (a gain near 0.02
would be valid arithmetic but shrinks every logit towards zero, which hides faults). Each tensor has a generator
of its own, seeded from the run's seed and the tensor's name, so the values do not depend on the order in which
tensors are made or on which tensors exist. The reference has no such mode (it always reads a real model file).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Mapping, Tuple, Union

import torch

from ..config.model_config import ModelConfig
from ..config.registry import architecture
from .safetensors_io import write_file


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(("%d:%s" % (seed, name)).encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(name: str, shape: Tuple[int, ...], seed: int, std: float, dtype: torch.dtype,
                  device="cpu") -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_seed_for(seed, name))
    t = torch.randn(shape, generator=g, dtype=torch.float32, device=device) * std
    if len(shape) == 1:
        t = t + 1.0
    return t.to(dtype)


def random_tensors(expected: Mapping[str, Tuple[int, ...]], seed: int, *, std: float = 0.02,
                   dtype: torch.dtype = torch.bfloat16, device="cpu") -> Dict[str, torch.Tensor]:
    return {n: random_tensor(n, tuple(s), seed, std, dtype, device) for n, s in expected.items()}


def write_random_model(out_dir: str, config: Union[ModelConfig, Mapping], seed: int, *, std: float = 0.02,
                       dtype: str = "bfloat16") -> str:
    """write ``config.json`` and ``model.safetensors`` for the configuration with weights drawn from the seed"""
    from ..parts.model import expected_tensors
    cfg = config if isinstance(config, ModelConfig) else ModelConfig.from_dict(config)
    tdt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    spec = architecture(cfg.architecture).build_spec(cfg)
    os.makedirs(out_dir, exist_ok=True)
    d = cfg.to_dict()
    d["torch_dtype"] = dtype
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(d, f, indent=2)
    tensors = random_tensors(expected_tensors(spec), seed, std=std, dtype=tdt)
    write_file(os.path.join(out_dir, "model.safetensors"), tensors,
               metadata={"format": "pt", "seed": str(seed), "std": repr(std)})
    return out_dir
