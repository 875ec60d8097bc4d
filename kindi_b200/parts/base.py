"""Interfaces of the parts a layer is made of, and the per-step context they all receive.

Every part works on the packed tokens of one step: ``T`` rows, the new tokens of all sequences of the batch one
after another. ``StepContext`` says, for each row, which sequence and which position it is, and for each sequence
its cache slot, the range of its rows and its length after the step. Parts take their sizes and constants from
their ``PartSpec`` and their tensors from a ``WeightView``; none of them knows which model it is in.

The residual stream is 32-bit throughout. A part that produces a branch output returns a ``Branch``: one or more
32-bit partial results whose sum is added to the residual by the next norm (the reference defers the add in the
same way: its fused add + RMS norm at the start of the next sub-layer, ``kindi/nanbeige.py:688-689,709``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple

import torch

from ..config.spec import PartSpec


# ----------------------------------------------------------------------------- what a part asks of the cache
@dataclass(frozen=True)
class KVNeed:
    """keys and values of ``n_kv_heads`` x ``head_dim`` per position; ``window`` None keeps every position, else
    only the last ``window`` positions are ever read (older pages are given back)."""

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """a fixed-size 32-bit state per sequence, zero when a sequence starts"""

    shape: Tuple[int, ...]


# ----------------------------------------------------------------------------- the step's metadata
@dataclass
class StepContext:
    """The packed batch of one step.

    Device tensors (int32): ``tok[T]``, ``pos[T]`` (absolute position of each row), ``seq[T]`` (index of the row's
    sequence in the batch), ``slot[B]``, ``q_start[B+1]`` (row range of each sequence), ``kv_len[B]`` (length of
    each sequence once this step's tokens are stored). Host copies carry the same numbers for parts written in
    plain PyTorch. ``decode`` is true when every sequence brings exactly one token."""

    T: int
    B: int
    tok: torch.Tensor
    pos: torch.Tensor
    seq: torch.Tensor
    slot: torch.Tensor
    q_start: torch.Tensor
    kv_len: torch.Tensor
    h_slot: Tuple[int, ...]
    h_q_start: Tuple[int, ...]
    h_kv_len: Tuple[int, ...]
    decode: bool
    max_q: int
    max_kv: int
    dtype: torch.dtype
    device: torch.device
    status: Any = None                 # device int32[1]: kernels set bits here instead of trapping
    cache: Any = None                  # the engine's cache (kindi_b200.cache.SequenceCache)
    entry: Any = None                  # the schedule entry being run
    fast: bool = True                  # bfloat16 serving kernels (False: the true 32-bit path)
    graph: bool = False                # the launches are being recorded for replay: host-side numbers (h_*,
                                       # max_kv) are not available and nothing may depend on them
    scratch: Dict[Any, Any] = field(default_factory=dict)     # what parts keep for the rest of this step (a table that
                                                              # is the same in every layer is made once)


@dataclass
class Branch:
    """a branch output not yet added to the residual: ``parts`` is 32-bit ``[S, T, width]``; the sum over S, taken
    in order, is the branch"""

    parts: torch.Tensor


# ----------------------------------------------------------------------------- tensors by name
class WeightView:
    """the tensors of one prefix (``model.layers.3.``): parts ask for them by their own suffixes"""

    def __init__(self, tensors: Mapping[str, torch.Tensor], prefix: str = ""):
        self._t = tensors
        self.prefix = prefix

    def __call__(self, suffix: str) -> torch.Tensor:
        return self._t[self.prefix + suffix]

    def sub(self, more: str) -> "WeightView":
        return WeightView(self._t, self.prefix + more)


# ----------------------------------------------------------------------------- the parts
class Part:
    """Base of every part. ``tensor_shapes`` (a classmethod: the loader needs it before anything is built) gives the
    suffixes and shapes of the tensors the part reads; the constructor receives the spec, the model width, the
    run's dtype/device and a ``WeightView``."""

    category = ""
    # False for a part whose forward reads the step's host-side numbers (h_slot, h_q_start, h_kv_len, max_kv) or
    # launches work that cannot be recorded: the engine then runs every step launch by launch
    graph_safe = True

    @classmethod
    def tensor_shapes(cls, spec: PartSpec, width: int) -> Dict[str, Tuple[int, ...]]:
        return {}

    @classmethod
    def tensor_init(cls, spec: PartSpec, width: int) -> Dict[str, str]:
        """how the random-weights mode draws the part's tensors that are not plain matrices: ``{suffix: "gain"}``
        (around one: a norm's weight) or ``{suffix: "zero"}`` (a bias); every other tensor is drawn around zero"""
        return {}

    def __init__(self, spec: PartSpec, width: int, weights: WeightView, *, dtype: torch.dtype, device):
        self.spec = spec
        self.width = width
        self.dtype = dtype
        self.device = device

    def bytes_read(self) -> int:
        """bytes of weights one step reads (for the roofline account)"""
        return 0


class Norm(Part):
    category = "norm"

    def add_norm(self, ctx: StepContext, x: torch.Tensor, pending: Optional[Branch],
                 rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x`` (32-bit ``[T, width]``) += pending branch (written back unless ``rows`` is given); returns the
        normalised rows in the run dtype: all ``T`` rows, or the rows listed in ``rows`` (int32)"""
        raise NotImplementedError


class Embedding(Part):
    """token ids to the 32-bit residual stream. Its tensors are named in full by its spec (no prefix)."""

    category = "embedding"

    def forward(self, ctx: StepContext) -> torch.Tensor:
        """32-bit ``[T, width]`` rows of the step's tokens (``ctx.tok``)"""
        raise NotImplementedError

    def bytes_read(self, n_rows: int = 0) -> int:
        return 0


class Head(Part):
    """normalised hidden rows to 32-bit logits. Its tensors are named in full by its spec (no prefix)."""

    category = "head"

    def forward(self, ctx: StepContext, y: torch.Tensor) -> torch.Tensor:
        """``y`` (run dtype ``[R, width]``) -> float32 ``[R, vocab]``"""
        raise NotImplementedError


class PositionEncoding(Part):
    """How a mixer's queries and keys learn their positions. The attention mixer hands its projections to
    ``encode_and_store``: the encoding writes the encoded queries, and encodes and stores the keys (and stores the
    values) at each row's position of its sequence's cache. An encoding that is a rotation of pairs also answers
    ``rotation()`` so that kernels which rotate on the fly can take its table; any other encoding returns None there
    and only ``encode_and_store`` is used."""

    category = "position"

    def rotation(self):
        """``(inv_freq float32 [rotary_dim / 2] on the device, rotary_dim)`` when the encoding is a rotation of the
        pairs ``(i, i + rotary_dim / 2)`` by ``pos * inv_freq[i]``, else None"""
        return None

    def encode_and_store(self, ctx: StepContext, qkv: torch.Tensor, q_out: torch.Tensor, n_heads: int,
                         n_kv_store: int, head_dim: int, pool, table, n_pages: int) -> None:
        """``qkv``: rows ``[T, (n_heads + 2 n_kv) head_dim]`` in the run dtype, or 32-bit planes ``[S, T, ...]`` whose
        sum they are. Writes the encoded query heads to ``q_out`` (``[T, >= n_heads head_dim]``; may be ``qkv``
        itself) and, when ``n_kv_store`` > 0, the encoded keys and the values of ``n_kv_store`` heads into ``pool``
        at each row's position (``ctx.pos``) of its sequence's pages (``table``)"""
        raise NotImplementedError


class Mixer(Part):
    category = "mixer"

    @classmethod
    def cache_need(cls, spec: PartSpec, width: int):
        """``KVNeed``, ``StateNeed`` or None"""
        return None

    def forward(self, ctx: StepContext, y: torch.Tensor) -> Branch:
        raise NotImplementedError


class FeedForward(Part):
    category = "feed_forward"

    def forward(self, ctx: StepContext, y: torch.Tensor) -> Branch:
        raise NotImplementedError


class Block(Part):
    """the arrangement of mixer, feed-forward and norms in a layer"""

    category = "block"

    @classmethod
    def cache_need(cls, spec: PartSpec, width: int):
        return None

    def forward(self, ctx: StepContext, x: torch.Tensor, pending: Optional[Branch]) -> Optional[Branch]:
        """run the layer on residual ``x`` with the previous layer's pending branch; returns the new pending
        branch"""
        raise NotImplementedError
