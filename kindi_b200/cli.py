"""kindi_b200 - command line.

  python -m kindi_b200 generate   generate token ids for prompts given as token ids
  python -m kindi_b200 verify     self-check: the same tokens twice, and from one multi-row pass as from single steps
  python -m kindi_b200 bench      measure writing (decode) and reading (prompt) speed
  python -m kindi_b200 info       show the configuration, the model and the GPU
  python -m kindi_b200 random     write a model folder with seeded random weights
Global options: --model DIR, --ctx N, --dtype bfloat16|float32.

The sub-commands and option names follow the reference's command line where it has them (``kindi/__main__.py:185-227``:
verify, bench, info, ``--ctx``; chat's ``--temperature`` and ``--max-tokens``; the config keys ``top_p``, ``top_k``,
``min_p``, ``repeat_penalty``, ``repeat_last_n`` of ``kindi/config.py:41-47`` as flags). Text in and out is not part
of this library: prompts and results are token ids.
"""
from __future__ import annotations

import argparse
import json
import sys
import time

from . import __version__


def log(msg):
    sys.stderr.write("[kindi_b200 %s] %s\n" % (time.strftime("%H:%M:%S"), msg))
    sys.stderr.flush()


def _engine(a, ctx=None):
    from .engine.engine import Engine
    if not a.model:
        raise SystemExit("kindi_b200: give the model folder with --model DIR")
    return Engine(a.model, ctx=ctx or a.ctx, dtype=a.dtype, max_batch=a.max_batch, log=log)


def _prompts(a):
    prompts = []
    for s in a.prompt_ids or []:
        prompts.append([int(t) for t in s.replace(",", " ").split()])
    if a.prompts_file:
        with open(a.prompts_file) as f:
            data = json.load(f)
        prompts += [[int(t) for t in p] for p in data]
    if not prompts:
        raise SystemExit("kindi_b200 generate: give --prompt-ids \"1,2,3\" (repeatable) or --prompts-file FILE.json")
    return prompts


def cmd_generate(a):
    from .config.runtime import SamplingParams
    eng = _engine(a)
    params = SamplingParams(temperature=a.temperature, top_p=a.top_p, top_k=a.top_k, min_p=a.min_p,
                            repeat_penalty=a.repeat_penalty, repeat_last_n=a.repeat_last_n, max_tokens=a.max_tokens,
                            seed=a.seed, stop_token_ids=tuple(a.stop_id or ()), order=a.sampler_order)
    res = eng.generate_batch(_prompts(a), params)
    for toks, fin in zip(res.tokens, res.finish):
        print(json.dumps({"tokens": toks, "finish": fin}))
    st = res.stats
    log("prompt %d tokens in %.2f s, %d tokens in %.2f s (%.1f tokens/s), %d batches"
        % (st.prompt_tokens, st.prompt_s, st.generated_tokens, st.gen_s, st.gen_tok_s, st.batches))
    return 0


def cmd_verify(a):
    """the reference's start-up self-check (``kindi/nanbeige_gen.py:156-179``): greedy generation twice gives the
    same tokens; one pass over several rows gives the tokens that single steps give; the run is not degenerate"""
    import random
    from .engine.batch import StepEntry
    eng = _engine(a, ctx=min(a.ctx, 4096))
    rng = random.Random(0)
    vocab = eng.spec.vocab_size
    ids = [rng.randrange(vocab) for _ in range(24)]
    first = eng.generate(ids, 10)
    again = eng.generate(ids, 10)
    slot = eng.alloc()
    rows = eng.step([StepEntry(slot, tuple(ids + first[:8]), tuple(range(len(ids) - 1, len(ids) + 8)))])
    one_pass = rows.argmax(dim=-1).tolist()
    eng.check_status()
    eng.free(slot)
    ok = first == again and one_pass[:9] == first[:9]
    log("steps %s, again %s, one pass %s" % (first, again, one_pass))
    if len(set(first)) <= 3:
        log("note: only %d distinct tokens (random weights give such runs)" % len(set(first)))
    log("PASS" if ok else "FAIL: the engine gives different tokens for the same prompt")
    return 0 if ok else 1


def cmd_bench(a):
    """the reference's own measurement (``kindi/nanbeige_cli.py:141-159``): writing speed at several depths (128
    timed steps after 5), reading speed for prompts of several lengths (after a 64-token warm-up)"""
    import random
    from .engine.batch import StepEntry
    eng = _engine(a)
    vocab = eng.spec.vocab_size
    rng = random.Random(1)
    for depth in [d for d in (0, 2048, 8192, 16384) if d + 140 < eng.ctx]:
        slot = eng.alloc()
        if depth:
            eng.step([StepEntry(slot, tuple(rng.randrange(vocab) for _ in range(depth)), ())])
        tok = 1000 % vocab
        for i in range(5):
            tok = int(eng.step([StepEntry(slot, (tok,), (0,))]).argmax())
        t0 = time.time()
        for i in range(128):
            tok = int(eng.step([StepEntry(slot, (tok,), (0,))]).argmax())
        log("writing at position %5d: %8.2f tokens/s" % (depth, 128 / (time.time() - t0)))
        eng.free(slot)
    for n in [x for x in (512, 2048, 8192, 16384) if x + 8 < eng.ctx]:
        ids = tuple(rng.randrange(vocab) for _ in range(n))
        slot = eng.alloc()
        eng.step([StepEntry(slot, ids[:64], (63,))]).argmax().item()
        eng.free(slot)
        slot = eng.alloc()
        t0 = time.time()
        eng.step([StepEntry(slot, ids, (n - 1,))]).argmax().item()
        log("reading a %5d-token prompt: %9.1f tokens/s" % (n, n / (time.time() - t0)))
        eng.free(slot)
    return 0


def cmd_info(a):
    print("kindi_b200 %s" % __version__)
    if a.model:
        import dataclasses
        import math
        from .config.registry import model_from_dir
        from .parts.model import cache_needs, expected_tensors
        cfg, spec = model_from_dir(a.model)
        shown = dataclasses.asdict(cfg) if dataclasses.is_dataclass(cfg) else dict(cfg)
        for k, v in sorted(shown.items()):
            print("  %-24s %s" % (k, v))
        shapes = expected_tensors(spec)
        n = sum(math.prod(s) for s in shapes.values())
        print("model: %s, %d layers, %d tensors, %.3f B parameters" % (spec.architecture, len(spec.layers),
                                                                        len(shapes), n / 1e9))
        import torch
        from .cache.sequence_cache import SequenceCache
        dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[a.dtype]
        print("cache for ctx %d (%s): %.1f MiB" % (a.ctx, a.dtype, SequenceCache.bytes_needed(
            cache_needs(spec), a.ctx, a.max_batch, dt) / 2 ** 20))
    try:
        import torch
        if torch.cuda.is_available():
            free, total = torch.cuda.mem_get_info()
            print("GPU: %s, compute %d.%d, %.0f of %.0f MiB free" % (
                (torch.cuda.get_device_name(0),) + torch.cuda.get_device_capability(0) + (free / 2 ** 20, total / 2 ** 20)))
        else:
            print("GPU: not available")
    except Exception as e:                               # noqa: BLE001
        print("GPU: not available (%s)" % e)
    return 0


def cmd_random(a):
    from .weights.random_init import write_random_model
    with open(a.config) as f:
        cfg = json.load(f)
    write_random_model(a.out, cfg, a.seed, std=a.std, dtype=a.store_dtype)
    log("wrote %s (config.json, model.safetensors), seed %d" % (a.out, a.seed))
    return 0


def main(argv=None):
    p = argparse.ArgumentParser(prog="kindi_b200", description="kindi_b200 %s - generation for the Llama-arch "
                                "Nanbeige decoder on one B200" % __version__)
    p.add_argument("--model", help="model folder (config.json + safetensors)")
    p.add_argument("--ctx", type=int, default=24576, help="most tokens all live sequences hold together")
    p.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    p.add_argument("--max-batch", dest="max_batch", type=int, default=64)
    p.add_argument("--version", action="version", version="kindi_b200 " + __version__)
    sub = p.add_subparsers(dest="cmd")
    s = sub.add_parser("generate", help="generate token ids")
    s.add_argument("--prompt-ids", dest="prompt_ids", action="append", help="token ids, comma or space separated")
    s.add_argument("--prompts-file", dest="prompts_file", help="JSON file: a list of lists of token ids")
    s.add_argument("--temperature", type=float, default=0.7)
    s.add_argument("--top-p", dest="top_p", type=float, default=0.8)
    s.add_argument("--top-k", dest="top_k", type=int, default=20)
    s.add_argument("--min-p", dest="min_p", type=float, default=0.0)
    s.add_argument("--repeat-penalty", dest="repeat_penalty", type=float, default=1.0)
    s.add_argument("--repeat-last-n", dest="repeat_last_n", type=int, default=64)
    s.add_argument("--max-tokens", dest="max_tokens", type=int, default=1024)
    s.add_argument("--seed", type=int)
    s.add_argument("--stop-id", dest="stop_id", type=int, action="append")
    s.add_argument("--sampler-order", dest="sampler_order", choices=("llama", "hf"), default="llama")
    sub.add_parser("verify", help="self-check of the engine")
    sub.add_parser("bench", help="measure speed")
    sub.add_parser("info", help="show configuration, model and GPU")
    s = sub.add_parser("random", help="write a model folder with seeded random weights")
    s.add_argument("--config", required=True, help="a config.json to take the sizes from")
    s.add_argument("--out", required=True)
    s.add_argument("--seed", type=int, default=0)
    s.add_argument("--std", type=float, default=0.02)
    s.add_argument("--store-dtype", dest="store_dtype", choices=("bfloat16", "float32"), default="bfloat16")
    a = p.parse_args(argv)
    if not a.cmd:
        p.print_help()
        return 1
    try:
        return {"generate": cmd_generate, "verify": cmd_verify, "bench": cmd_bench, "info": cmd_info,
                "random": cmd_random}[a.cmd](a)
    except BrokenPipeError:
        # whoever read the output has gone (`... | head`): leave quietly, without Python's complaint at exit
        import os
        try:
            os.dup2(os.open(os.devnull, os.O_WRONLY), sys.stdout.fileno())
        except OSError:
            pass
        return 0
