"""Random configurations under random schedules against the plain model.

Each case draws, from its number alone, a configuration of the architecture (head size 16 to 256, 1 to 4 key/value
heads with 1 to 17 query heads each, widths, feed-forward sizes and vocabularies that are no powers of two, 1 to 3
layers, eps, rope base, tied or not, windows on some layers), a dtype, a set of requests and one way of cutting them
into steps: whole, the last tokens one by one, batches that shrink, groups that decode for unequal numbers of steps,
or one request in portions of any size. The engine is given random limits too (the longest step, the longest
recorded prompt step). Every wanted row of logits is compared with the plain model's row of the whole sequence.
The wide cases run 24 to 48 sequences a step, where a decode step takes other kernels than below 25. The odd cases
draw sizes no kernel is tuned for: head sizes in steps of 8 and some that are no multiple of 8 (2 to 250), widths
like 33 and 101, a feed-forward of 8 or 333, a vocabulary of 3.
"""
from __future__ import annotations

import random

import numpy as np
import pytest

import plain_model as P
import tiny

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-5, "bfloat16": 1.5e-2}
LENGTHS = [1, 2, 5, 33, 64, 65, 100, 129, 200, 290]


def _draw_config(rng: random.Random, wide: bool, odd: bool = False) -> dict:
    if wide:
        hd, nkv, g = rng.choice([32, 64, 128, 128]), rng.choice([1, 2, 3, 4]), rng.choice([1, 2, 5])
    else:
        hd = rng.choice([16, 32, 48, 64, 64, 96, 128, 128, 128, 256])
        nkv, g = rng.choice([1, 1, 2, 3]), rng.choice([1, 2, 3, 5, 5, 7, 17])
    layers = rng.choice([1, 2, 3])
    cfg = dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=rng.choice([127, 256, 331, 777, 1001]),
               hidden_size=rng.choice([64, 72, 100, 136, 200, 328]), intermediate_size=rng.choice([96, 150, 264, 320, 1000]),
               num_hidden_layers=layers, num_attention_heads=nkv * g, num_key_value_heads=nkv, head_dim=hd,
               rms_norm_eps=rng.choice([1e-5, 1e-6, 3e-6]), rope_theta=rng.choice([1e4, 5e5, 7e7]),
               tie_word_embeddings=rng.random() < 0.5)
    if odd:
        cfg.update(head_dim=rng.choice(list(range(8, 264, 8)) + [12, 20, 36, 2, 6, 250]),
                   hidden_size=rng.choice([62, 70, 101, 64, 136, 264, 33]),
                   intermediate_size=rng.choice([97, 150, 333, 64, 8, 1000]), vocab_size=rng.choice([3, 17, 127, 1001, 257]))
    window = rng.choice([None, None, 33, 70, 130])
    if window:
        cfg["sliding_window"] = window
        cfg["layer_types"] = [rng.choice(["full_attention", "sliding_attention"]) for _ in range(layers)]
        if "sliding_attention" not in cfg["layer_types"]:
            cfg["layer_types"][0] = "sliding_attention"
    return cfg


def _portions(eng, reqs, want, rng):
    from kindi_b200.engine.batch import StepEntry
    worst = 0.0
    for _ in range(2):                                  # the second pass meets the shapes the first one recorded
        for rid, toks in reqs.items():
            slot, at, rows = eng.alloc(), 0, []
            while at < len(toks):
                n = min(len(toks) - at, rng.choice([1, 1, 2, 7, 64, 70, 128]))
                rows.append(eng.step([StepEntry(slot, tuple(toks[at:at + n]), tuple(range(n)))]).cpu().numpy())
                at += n
            eng.check_status()
            eng.free(slot)
            worst = max(worst, tiny.rel_err(np.concatenate(rows), want[rid]))
    return worst


@pytest.mark.parametrize("case", list(range(16)) + [1000 + i for i in range(8)] + [2000 + i for i in range(12)])
def test_random_configuration_and_schedule(tmp_path, case):
    from kindi_b200.engine.engine import Engine
    from kindi_b200.weights.random_init import write_random_model
    rng = random.Random(case)
    wide = 1000 <= case < 2000
    cfg = _draw_config(rng, wide, odd=case >= 2000)
    dtype = rng.choice(["float32", "bfloat16"])
    folder = write_random_model(str(tmp_path / "m"), cfg, case, dtype=dtype)
    model = P.load_model(folder)
    vocab = cfg["vocab_size"]
    n_req = rng.randint(30, 60) if wide else rng.randint(1, 9)
    reqs = tiny.random_requests(vocab, [rng.choice(LENGTHS) for _ in range(n_req)], seed=case)
    want = {rid: P.forward(model, toks).numpy() for rid, toks in reqs.items()}
    mode = rng.choice(["batched", "group"] if wide else ["whole", "last", "batched", "group", "portions"])
    max_batch = rng.randint(24, 48) if wide else rng.randint(1, 6)
    limits = dict(max_step_tokens=rng.choice([64, 128, 8192]), prompt_graph_tokens=rng.choice([0, 128, 512]))
    what = "case %d: %s %s %r batch %d %r" % (case, dtype, mode, cfg, max_batch, limits)
    if mode == "portions":
        eng = Engine(folder, ctx=4096, dtype=dtype, max_batch=max_batch, **limits)
        worst = _portions(eng, reqs, want, rng)
    else:
        if mode == "whole":
            steps = tiny.trace_whole(reqs)
        elif mode == "last":
            steps = tiny.trace_last_n(reqs, rng.choice([1, 8, 32]))
        elif mode == "batched":
            steps = tiny.trace_batched(reqs, batch=max_batch, decode=rng.choice([2, 5, 12]))
        else:
            ids, steps = list(reqs), []
            for b0 in range(0, len(ids), max_batch):
                grp = {r: reqs[r] for r in ids[b0:b0 + max_batch]}
                steps += tiny.trace_group(grp, {r: rng.randint(0, 20) for r in grp}, first_step=len(steps))
        eng = Engine(folder, ctx=tiny.max_live_tokens(steps), dtype=dtype, max_batch=max_batch, **limits)
        out = str(tmp_path / "out")
        tiny.run_replay(eng, steps, out)
        eng.check_status()
        got = tiny.collect(out, steps, vocab)
        worst = 0.0
        for rid in reqs:
            have = sorted(i for (r, i) in got if r == rid)
            worst = max(worst, tiny.rel_err(np.stack([got[(rid, i)] for i in have]), want[rid][have]))
    eng.cache.check()
    assert eng.cache.slots.n_held == 0 and all(g.pages.pool.n_held == 0 for g in eng.cache.groups), what
    assert worst <= TOL[dtype], "%s: differs from the plain model by %.3g" % (what, worst)


@pytest.mark.parametrize("case", list(range(10)))
def test_steps_that_mix_prompts_portions_and_single_tokens(tmp_path, case):
    """the step function's general use: in one step every live sequence brings its own number of tokens (a whole
    prompt, a portion that continues an earlier one, a single token), some sit the step out, new sequences join, and
    any subset of rows is wanted; each wanted row against the plain model's row of the whole sequence"""
    from kindi_b200.engine.batch import StepEntry
    from kindi_b200.engine.engine import Engine
    from kindi_b200.weights.random_init import write_random_model
    rng = random.Random(5000 + case)
    cfg = _draw_config(rng, False, odd=rng.random() < 0.3)
    dtype = rng.choice(["float32", "bfloat16"])
    folder = write_random_model(str(tmp_path / "m"), cfg, case, dtype=dtype)
    model = P.load_model(folder)
    reqs = tiny.random_requests(cfg["vocab_size"], [rng.choice([3, 17, 64, 65, 130, 200, 300])
                                                    for _ in range(rng.randint(2, 10))], seed=case)
    want = {rid: P.forward(model, toks).numpy() for rid, toks in reqs.items()}
    max_batch = rng.randint(2, 6)
    eng = Engine(folder, ctx=max_batch * 320 + 64, dtype=dtype, max_batch=max_batch,
                 max_step_tokens=rng.choice([64, 128, 8192]), prompt_graph_tokens=rng.choice([0, 128, 512]))
    waiting, live, worst = list(reqs), {}, 0.0                   # live: id -> [slot, tokens done]
    while waiting or live:
        while waiting and len(live) < max_batch and rng.random() < 0.7:
            live[waiting.pop(0)] = [eng.alloc(), 0]
        entries, who = [], []
        for rid, (slot, done) in live.items():
            if rng.random() < 0.2:
                continue
            k = min(len(reqs[rid]) - done, rng.choice([1, 1, 1, 2, 5, 33, 64, 100]))
            wanted = tuple(sorted(rng.sample(range(k), rng.randint(0, k)))) if rng.random() < 0.5 else tuple(range(k))
            entries.append(StepEntry(slot, tuple(reqs[rid][done:done + k]), wanted))
            who.append((rid, done, wanted, k))
        if not entries:
            continue
        out = eng.step(entries)
        eng.check_status()
        rows = out.cpu().numpy() if out is not None else None
        at = 0
        for rid, done, wanted, k in who:
            for w in wanted:
                worst = max(worst, float(np.abs(rows[at] - want[rid][done + w]).max() / np.abs(want[rid]).max()))
                at += 1
            live[rid][1] = done + k
            if live[rid][1] == len(reqs[rid]):
                eng.free(live.pop(rid)[0])
    eng.cache.check()
    assert eng.cache.slots.n_held == 0 and all(g.pages.pool.n_held == 0 for g in eng.cache.groups)
    assert worst <= TOL[dtype], "case %d (%s, %r): differs from the plain model by %.3g" % (case, dtype, cfg, worst)
