"""The description of a model as data: which parts make each layer, and in which order layers run.

A model is a list of layers; a layer is a block arrangement over a mixer, a feed-forward and norms; each part is
named by its kind (a key of the parts registry) and carries its own sizes and constants as parameters. The run
order is a list too (``schedule``): an entry names the layer whose weights run and the cache entry it uses, so a
layer may run twice (two schedule entries, each with a cache entry of its own) or read the keys and values that
another entry wrote (``reads_cache_of``). Nothing here knows which architecture it describes; an architecture is a
function from its config.json to a ``ModelSpec`` (see ``kindi_b200/models``).

The reference fixes all of this in code for one model (``kindi/nanbeige.py:676-726``: the kernel sequence of a
layer; ``:245-260``: its sizes); the hybrid engines beside it show why it has to be data (``kindi/engine.py:228-232``:
some layers keep keys and values, others a recurrent state).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: its kind (registry key) and its parameters (sizes, constants, nested part specs)."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __getitem__(self, k):
        return self.params[k]

    def get(self, k, default=None):
        return self.params.get(k, default)


@dataclass(frozen=True)
class LayerSpec:
    """A layer: the block arrangement (kind + the specs of its parts) and the prefix of its tensors' names."""

    block: PartSpec
    prefix: str


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer. ``cache`` is the index of the cache entry (keys/values or state) this run owns;
    ``reads_cache_of`` names another schedule entry's cache entry whose keys and values this run attends to
    instead of writing its own."""

    layer: int
    cache: int
    reads_cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    """``embedding`` and ``head`` are parts like the layers' (kinds of the categories "embedding" and "head"): what
    turns token ids into the residual stream and the last hidden rows into logits is named by the architecture, with
    its tensors' names and constants (a scale, a soft cap) as parameters. ``may_ignore``: patterns (``fnmatch``) of
    tensor names a folder may hold that the model does not read. ``copies``: names a folder may hold only as a copy
    of another tensor it holds (a tied head stored twice): ``{name: the tensor it must equal}``."""

    architecture: str
    vocab_size: int
    width: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    final_norm_prefix: str
    embedding: PartSpec
    head: PartSpec
    stop_token_ids: Tuple[int, ...] = ()
    max_positions: Optional[int] = None     # the most positions a sequence may reach (None: only the cache bounds it)
    may_ignore: Tuple[str, ...] = ()
    copies: Mapping[str, str] = field(default_factory=dict)

    @property
    def n_cache_entries(self) -> int:
        return 1 + max((e.cache for e in self.schedule), default=-1)

    def validate(self) -> None:
        seen: Dict[int, int] = {}
        for i, e in enumerate(self.schedule):
            if not (0 <= e.layer < len(self.layers)):
                raise ValueError("schedule entry %d names layer %d of %d" % (i, e.layer, len(self.layers)))
            if e.reads_cache_of is None:
                if e.cache in seen:
                    raise ValueError("schedule entries %d and %d both own cache entry %d" % (seen[e.cache], i, e.cache))
                seen[e.cache] = i
            elif e.reads_cache_of not in seen:
                raise ValueError("schedule entry %d reads cache entry %d before any entry wrote it"
                                 % (i, e.reads_cache_of))


def default_schedule(n_layers: int) -> Tuple[ScheduleEntry, ...]:
    return tuple(ScheduleEntry(layer=i, cache=i) for i in range(n_layers))
