"""The sampler: one kernel call per step picks every row's next token on the device.

Options are the reference's (``kindi/sampling.py:91-114``; defaults ``kindi/config.py:41-47``). Each sequence draws
from a random stream of its own, seeded from the request's seed and the sequence's index in the request
(``kindi/nanbeige_gen.py:229-230`` seeds one NumPy generator per request; without a seed it uses the clock), so a
sequence's tokens do not depend on which other sequences share its batch.
"""
from __future__ import annotations

import time
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..config.runtime import SamplingParams
from ..kernels import lib as K


class SequenceRandom:
    """the uniform numbers of one sequence"""

    def __init__(self, seed: int, index: int):
        self._g = np.random.Generator(np.random.Philox(np.random.SeedSequence([int(seed) & 0xFFFFFFFF, int(index)])))

    def next(self) -> float:
        return float(self._g.random())


def request_seed(params: SamplingParams) -> int:
    return params.seed if params.seed is not None else int(time.time() * 1000) % 2 ** 31


def recent_tokens(history: Sequence[int], last_n: int) -> List[int]:
    """the distinct tokens among the last ``last_n`` of the history (-1: all of it; 0: none)"""
    if last_n == 0:
        return []
    h = history if last_n < 0 else history[-last_n:]
    return sorted(set(int(t) for t in h))


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)

    def pick(self, logits: torch.Tensor, params: SamplingParams, uniforms: Optional[Sequence[float]] = None,
             histories: Optional[Sequence[Sequence[int]]] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """logits: float32 [R, V] on the device (changed in place by the repeat penalty). Returns int32 [R] on the
        device (``out`` when given). ``uniforms``: one number in [0, 1) per row (needed unless greedy).
        ``histories``: each row's tokens so far, for the repeat penalty."""
        R, V = logits.shape
        assert logits.dtype == torch.float32 and logits.stride(1) == 1
        if out is None:
            out = torch.empty(R, dtype=torch.int32, device=logits.device)
        assert out.dtype == torch.int32 and out.numel() == R and out.is_contiguous()
        lib = K.load()
        st = torch.cuda.current_stream().cuda_stream
        if params.repeat_penalty != 1.0 and histories is not None:
            rec = [recent_tokens(h, params.repeat_last_n) for h in histories]
            n = max((len(r) for r in rec), default=0)
            if n:
                arr = np.full((R, n), -1, dtype=np.int32)
                for i, r in enumerate(rec):
                    arr[i, :len(r)] = r
                dev = torch.from_numpy(arr).pin_memory().to(logits.device, non_blocking=True)
                K._check(lib.kb_penalize(logits.data_ptr(), logits.stride(0), R, V, dev.data_ptr(), n,
                                         float(params.repeat_penalty), st), "penalize")
        if params.greedy:
            u = None
        else:
            if uniforms is None or len(uniforms) != R:
                raise ValueError("temperature sampling needs one uniform number per row")
            # (from pinned memory, without a wait: the host goes on to issue the next step meanwhile)
            u = torch.tensor(list(uniforms), dtype=torch.float32).pin_memory().to(logits.device, non_blocking=True)
        K._check(lib.kb_sample(logits.data_ptr(), logits.stride(0), R, V, float(params.temperature),
                               int(params.top_k), float(params.top_p), float(params.min_p),
                               1 if params.order == "hf" else 0, None if u is None else u.data_ptr(),
                               out.data_ptr(), st), "sample")
        return out
