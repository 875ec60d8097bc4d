"""The generation loop above the step function.

Requests are taken in order and formed into batches that start together: all prompts of a batch run in one step,
then every live sequence brings one token a step. A sequence ends at a stop token (which is not part of its
output, ``kindi/nanbeige_gen.py:272-274``) or when it has ``max_new`` tokens, where ``max_new = max(1,
min(max_tokens, ctx - len(prompt)))`` and a prompt of ``ctx`` tokens or more is refused
(``kindi/nanbeige_gen.py:210-212,219-220``). A sequence that ends leaves the batch and gives back its slot at once;
when the batch is empty the next one starts, in slots and pages that were used before. The reference serves one
request at a time (``kindi/nanbeige_gen.py:261-283``); batches are this library's own.

Host and GPU overlap where the stepper allows it (``launch`` / ``collect``): while a step runs, the next one is
issued with its tokens taken on the device from the running step's picks, and only then are the running step's
tokens read (the reference's ``step_begin`` / ``step_end``, ``kindi/nanbeige.py:741-776``, used at
``kindi/nanbeige_gen.py:343-347``). A sequence that turns out to have ended at a stop token has then run one step
too many, whose result is dropped; the tokens of every sequence are the same as without the overlap.

The loop's decisions need no GPU: it talks to a *stepper* (``alloc``, ``free``, ``run``; optionally ``launch`` and
``collect``), which is the engine in production and a stand-in in the CPU tests.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

from ..cache.pages import PAGE, pages_for
from ..config.runtime import SamplingParams
from .batch import StepEntry


class PromptTooLong(ValueError):
    """the prompt alone fills the context (the reference's ContextOverflow, ``kindi/server.py:26-36``)"""


@dataclass
class GenerationStats:
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prompt_s: float = 0.0
    gen_s: float = 0.0
    steps: int = 0
    batches: int = 0

    @property
    def gen_tok_s(self) -> float:
        return self.generated_tokens / self.gen_s if self.gen_s > 0 else 0.0


@dataclass
class GenerationResult:
    tokens: List[List[int]]
    finish: List[str]                       # "stop" | "length" per request
    stats: GenerationStats = field(default_factory=GenerationStats)


def max_new_tokens(prompt_len: int, max_tokens: int, ctx: int) -> int:
    if prompt_len < 1:
        raise ValueError("a prompt needs at least one token")
    if prompt_len >= ctx:
        raise PromptTooLong("the prompt has %d tokens and the context holds %d: nothing could be generated"
                            % (prompt_len, ctx))
    return max(1, min(max_tokens, ctx - prompt_len))


def plan_batches(prompt_lens: Sequence[int], max_new: Sequence[int], ctx: int, max_batch: int) -> List[List[int]]:
    """request indices per batch, in order. A batch takes requests while it has room for another sequence and the
    cache can hold every member at its greatest possible length (prompt + max_new - 1 stored tokens, rounded up to
    a page each), so that a started batch can never run out of pages."""
    room = pages_for(ctx)
    batches: List[List[int]] = []
    cur: List[int] = []
    used = 0
    for i, (p, m) in enumerate(zip(prompt_lens, max_new)):
        need = pages_for(p + m - 1)
        if need > room:
            raise PromptTooLong("request %d needs %d tokens of cache and the context holds %d" % (i, need * PAGE, ctx))
        if cur and (len(cur) >= max_batch or used + need > room):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


def generate(stepper, prompts: Sequence[Sequence[int]], params: SamplingParams, *,
             stop_token_ids: Sequence[int] = (), on_tokens: Optional[Callable[[Dict[int, int]], None]] = None,
             cancel: Optional[Callable[[], bool]] = None) -> GenerationResult:
    """generate for every prompt; returns the new tokens of each (without the stop token).

    ``stepper`` offers ``ctx``, ``max_batch``, optionally ``max_positions``, ``alloc()``, ``free(slot)`` and ``run(entries, params, seq_ids,
    histories) -> [token per entry]`` (each entry wants exactly one place). ``on_tokens`` is called after each step
    with {request index: new token}; ``cancel()`` true ends all live sequences with finish "stop"
    (``kindi/nanbeige_gen.py:265-267``)."""
    stop = set(int(t) for t in stop_token_ids) | set(int(t) for t in params.stop_token_ids)
    n = len(prompts)
    prompts = [list(int(t) for t in p) for p in prompts]
    # one sequence can hold what the cache holds, and no more positions than the model's configuration allows
    limit = getattr(stepper, "max_positions", None)
    seq_ctx = stepper.ctx if limit is None else min(stepper.ctx, limit)
    max_new = [max_new_tokens(len(p), params.max_tokens, seq_ctx) for p in prompts]
    batches = plan_batches([len(p) for p in prompts], max_new, stepper.ctx, stepper.max_batch)
    out: List[List[int]] = [[] for _ in range(n)]
    finish: List[str] = ["length"] * n
    stats = GenerationStats(prompt_tokens=sum(len(p) for p in prompts), batches=len(batches))
    # issuing the next step before this step's tokens are read needs a stepper that splits a step, and a pick that
    # needs no tokens on the host (the repeat penalty reads the sequence's history)
    overlap = hasattr(stepper, "launch") and hasattr(stepper, "collect") and params.repeat_penalty == 1.0
    for batch in batches:
        slots = {i: stepper.alloc() for i in batch}
        rows = list(batch)                       # the sequences of the step in flight, in the order of its rows
        try:
            t0 = time.perf_counter()
            entries = [StepEntry(slots[i], tuple(prompts[i]), (len(prompts[i]) - 1,)) for i in rows]
            handle = stepper.launch(entries, params, rows, None) if overlap else None
            first = True
            while True:
                ahead = None
                if overlap and all(i in slots and len(out[i]) + 1 < max_new[i] for i in rows):
                    # every row is alive and nobody leaves after this step for its length: the next step has the same
                    # rows, so it can run on the tokens this step leaves on the device (a stop token shows only when
                    # they have been read)
                    nxt_entries = [StepEntry(slots[i], (0,), (0,)) for i in rows]
                    ahead = stepper.launch(nxt_entries, params, rows, None, tokens_from_previous=True)
                    stats.steps += 1
                if overlap:
                    toks = stepper.collect(handle)
                else:
                    hist = [prompts[i] if first else prompts[i] + out[i] for i in rows]
                    toks = stepper.run(entries, params, rows, hist)
                if first:
                    stats.prompt_s += time.perf_counter() - t0
                    stats.steps += 1
                    t0 = time.perf_counter()
                    first = False
                nxt: List[int] = []
                emitted: Dict[int, int] = {}
                for i, t in zip(rows, toks):
                    if i not in slots:
                        continue                 # ended earlier; this row of a step issued ahead is dropped
                    t = int(t)
                    if t in stop:
                        finish[i] = "stop"
                    else:
                        out[i].append(t)
                        emitted[i] = t
                        if len(out[i]) < max_new[i]:
                            nxt.append(i)
                            continue
                        finish[i] = "length"
                    stepper.free(slots.pop(i))
                stats.generated_tokens += len(emitted)
                if on_tokens is not None and emitted:
                    on_tokens(emitted)
                if cancel is not None and nxt and cancel():
                    for i in nxt:
                        finish[i] = "stop"
                        stepper.free(slots.pop(i))
                    nxt = []
                if ahead is not None:
                    # the step issued ahead is in flight with the old rows; rows that have ended meanwhile are dropped
                    # when it is collected
                    handle = ahead
                    if not nxt:
                        stepper.collect(handle)
                        break
                    continue
                if not nxt:
                    break
                rows = nxt
                entries = [StepEntry(slots[i], (out[i][-1],), (0,)) for i in rows]
                if overlap:
                    handle = stepper.launch(entries, params, rows, None)
                stats.steps += 1
            stats.gen_s += time.perf_counter() - t0
        finally:
            for s in slots.values():
                stepper.free(s)
    return GenerationResult(out, finish, stats)
