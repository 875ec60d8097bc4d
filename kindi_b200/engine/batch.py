"""Packing the sequences of one step: the host-side arithmetic that turns "these sequences bring these tokens" into
the arrays the kernels read. Pure Python + NumPy, so it is testable without a GPU.

Rows are the new tokens of all sequences, one sequence after another (unequal lengths, no padding). For row r of
sequence b: ``pos = length_before[b] + offset``, ``seq = b``. ``want`` places are offsets into a sequence's own
tokens; ``rows`` are the packed row numbers, in the order of the entries and of their ``want`` lists.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple

import numpy as np


@dataclass(frozen=True)
class StepEntry:
    """one sequence's share of a step: its slot, its next tokens, and the places among them whose logits are
    wanted"""

    slot: int
    tokens: Tuple[int, ...]
    want: Tuple[int, ...] = ()


@dataclass
class PackedStep:
    T: int                            # rows of the step, padding rows included
    B: int
    R: int
    meta: np.ndarray                  # int32, all segments one after another
    off: dict                         # segment name -> (start, length)
    h_slot: Tuple[int, ...]
    h_q_start: Tuple[int, ...]
    h_kv_len: Tuple[int, ...]
    decode: bool
    max_q: int
    max_kv: int


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


def layout(T: int, B: int, R: int) -> Tuple[dict, int]:
    """where each segment lies in the meta buffer; depends on the three counts only, so steps of the same shape
    share it"""
    off, at = {}, 0
    for name, n in (("tok", T), ("pos", T), ("seq", T), ("slot", B), ("q_start", B + 1), ("kv_len", B),
                    ("rows", R)):
        off[name] = (at, n)
        at += _align(max(n, 1))
    return off, at


def pack(entries: Sequence[StepEntry], length_before: Sequence[int], pad_rows_to: int = 0) -> PackedStep:
    """``pad_rows_to``: the step gets at least this many rows; the rows past the sequences' tokens are padding (token
    0, position -1, no sequence's row range holds them): they are computed and thrown away, change no cache and no
    other row, and let steps of different lengths share one recorded launch sequence"""
    if not entries:
        raise ValueError("a step needs at least one sequence")
    slots = [e.slot for e in entries]
    if len(set(slots)) != len(slots):
        raise ValueError("a slot appears twice in one step: %r" % (slots,))
    q_len = [len(e.tokens) for e in entries]
    if min(q_len) < 1:
        raise ValueError("every sequence of a step brings at least one token")
    B, T_real = len(entries), sum(q_len)
    T = max(T_real, pad_rows_to)
    rows: List[int] = []
    q_start = [0]
    for e, n in zip(entries, q_len):
        for w in e.want:
            if not (0 <= w < n):
                raise ValueError("want place %d lies outside the sequence's %d tokens of this step" % (w, n))
            rows.append(q_start[-1] + w)
        q_start.append(q_start[-1] + n)
    R = len(rows)
    off, total = layout(T, B, R)
    if T == B:
        # one token each (a decode step, every step of a long generation): the buffer is put together as one list
        kv_len = [n + 1 for n in length_before]
        flat = [0] * total
        for name, vals in (("tok", [e.tokens[0] for e in entries]), ("pos", list(length_before)), ("seq", range(B)),
                           ("slot", slots), ("q_start", q_start), ("kv_len", kv_len), ("rows", rows)):
            a, n = off[name]
            flat[a:a + n] = vals
        return PackedStep(T=T, B=B, R=R, meta=np.array(flat, dtype=np.int32), off=off, h_slot=tuple(slots),
                          h_q_start=tuple(q_start), h_kv_len=tuple(kv_len), decode=True, max_q=1, max_kv=max(kv_len))
    meta = np.zeros(total, dtype=np.int32)

    def seg(name):
        a, n = off[name]
        return meta[a:a + n]
    tok, pos, seq = seg("tok"), seg("pos"), seg("seq")
    pos[T_real:] = -1
    kv_len = []
    for b, (e, n) in enumerate(zip(entries, q_len)):
        a = q_start[b]
        tok[a:a + n] = e.tokens
        pos[a:a + n] = np.arange(length_before[b], length_before[b] + n, dtype=np.int32)
        seq[a:a + n] = b
        kv_len.append(length_before[b] + n)
    seg("slot")[:] = slots
    seg("q_start")[:] = q_start
    seg("kv_len")[:] = kv_len
    seg("rows")[:] = rows
    return PackedStep(T=T, B=B, R=R, meta=meta, off=off, h_slot=tuple(slots), h_q_start=tuple(q_start),
                      h_kv_len=tuple(kv_len), decode=max(q_len) == 1, max_q=max(q_len), max_kv=max(kv_len))


def split_step(entries: Sequence[StepEntry], chunk: int) -> List[List[Tuple[int, StepEntry]]]:
    """cut a step that brings more than ``chunk`` tokens into sub-steps of at most ``chunk`` tokens each: sequences
    are taken in order and a long one continues in the next sub-step (its later tokens read the earlier ones from
    the cache, as the reference's prompt chunks do, ``kindi/nanbeige.py:943-946,974``). Returns, per sub-step, a list
    of (index of the original entry, its share); ``want`` places are moved to the share that holds them. A slot
    appears at most once in a sub-step."""
    subs: List[List[Tuple[int, StepEntry]]] = [[]]
    room = chunk
    for i, e in enumerate(entries):
        at = 0
        n = len(e.tokens)
        while at < n:
            if room == 0 or any(j == i for j, _ in subs[-1]):
                subs.append([])
                room = chunk
            take = min(room, n - at)
            want = tuple(w - at for w in e.want if at <= w < at + take)
            subs[-1].append((i, StepEntry(e.slot, e.tokens[at:at + take], want)))
            at += take
            room -= take
    return subs
