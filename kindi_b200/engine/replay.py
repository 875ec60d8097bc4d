"""Trace replay: feed given token ids through the engine step by step and write the logits that are asked for.

It samples nothing and has no model code of its own: it calls ``Engine.step`` - the model, cache and kernels that
generation uses - and ``Engine.alloc`` / ``Engine.free`` for the requests' slots. The reference's nearest program is
``kindi verify`` (``kindi/nanbeige_cli.py:61-138``), which feeds stored ids and compares greedy tokens; its engine
exposes logits rows through ``check`` (``kindi/nanbeige.py:1126-1129``).

Input: one JSON object a line, ``{"step": n, "entries": [{"id", "tokens", "want"}], "end": [ids]}``. For a step in
which something is wanted, ``<out>/<step>.f32`` holds the logits at the wanted places, in the order of the entries
and of their ``want`` lists, little-endian float32 ``[wanted, vocab]``. After every step a line ``done <step>`` is
printed and flushed.
"""
from __future__ import annotations

import json
import os
import sys
from typing import Dict, IO

from .batch import StepEntry


def replay(engine, lines: IO[str], out_dir: str, out: IO[str] = sys.stdout) -> int:
    os.makedirs(out_dir, exist_ok=True)
    slots: Dict[str, int] = {}
    n = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries") or []:
            rid = str(e["id"])
            if rid not in slots:
                slots[rid] = engine.alloc()
            entries.append(StepEntry(slots[rid], tuple(int(t) for t in e["tokens"]),
                                     tuple(int(w) for w in e.get("want") or ())))
        if entries:
            logits = engine.step(entries)
            if logits is not None:
                host = logits.to("cpu").numpy().astype("<f4", copy=False)
                engine.check_status()
                tmp = os.path.join(out_dir, "%s.f32.tmp" % step)
                host.tofile(tmp)
                os.replace(tmp, os.path.join(out_dir, "%s.f32" % step))
            else:
                engine.check_status()
        for rid in rec.get("end") or []:
            rid = str(rid)
            if rid in slots:
                engine.free(slots.pop(rid))
        out.write("done %s\n" % step)
        out.flush()
        n += 1
    return n


def main(argv=None) -> int:
    import argparse
    p = argparse.ArgumentParser(prog="trace_run", description="replay a trace of token ids and write logits")
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=("bfloat16", "float32"))
    p.add_argument("--out", required=True, help="folder for <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True, dest="max_tokens",
                   help="most tokens live requests hold at any time (each rounded up to 64)")
    a = p.parse_args(argv)
    from .engine import Engine
    from ..cache.pages import pages_for
    engine = Engine(a.model, ctx=a.max_tokens, dtype=a.dtype, max_batch=min(max(1, pages_for(a.max_tokens)), 1024))
    replay(engine, sys.stdin, a.out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
