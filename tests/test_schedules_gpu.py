"""Schedules that the other engine tests do not reach, against the plain implementation:

* decode steps of 32 to 64 sequences (the serving kernels take other branches from 32 rows on: rotate-and-store as a
  kernel of its own, split-K planes followed by the SwiGLU kernel above 32 rows, wider activation tiles, one position
  split, and a recording of its own for that batch size), with unequal prompts, early ends and a second batch in the
  same slots and pages;
* a sequence of more than 8,200 positions: its prompt cut at ``max_step_tokens``, page numbers in the thousands, then
  its last tokens one by one alone (64 position splits) and inside a batch of 8;
* sampled generation end to end: the tokens are those of the plain model and the plain sampler fed the same uniform
  numbers.

The models here carry a planted key (``tiny.make_needle_model``): the rows decoded one by one are probe tokens whose
attention rests on one needle token far back in their sequence, so a far key that is dropped, a window one position
off or a page of another sequence changes the logits by ten to fifty times the tolerance
(``tests/test_plain_cpu.py`` measures that on the plain model), while rounding errors stay as with plain random
weights.
"""
import random

import numpy as np
import pytest
import torch

import plain_model as P
import tiny

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-5, "bfloat16": 1.5e-2}        # the tolerances of the replay tests

LAYER_SIZED = dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=3001, hidden_size=2560,
                   intermediate_size=10496, num_hidden_layers=2, num_attention_heads=20, num_key_value_heads=4,
                   head_dim=128, rms_norm_eps=1e-5, rope_theta=70000000.0, tie_word_embeddings=False)
# head size 128, 5 query heads per key/value head (the benchmark's group), two key/value heads, a narrow width
LONG = dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=311, hidden_size=192,
            intermediate_size=256, num_hidden_layers=2, num_attention_heads=10, num_key_value_heads=2, head_dim=128,
            rms_norm_eps=1e-5, rope_theta=70000000.0, tie_word_embeddings=False)


def _compare(got, reqs, want, tol, what):
    for rid, toks in reqs.items():
        mine = np.stack([got[(rid, i)] for i in range(len(toks))])
        err = tiny.rel_err(mine, want[rid])
        row = int(np.argmax(np.max(np.abs(mine - want[rid]), axis=1)))
        assert err <= tol, "%s %s: %.3g at position %d of %d" % (what, rid, err, row, len(toks))


def _wide_batches(vocab, n_first, n_second, longest, seed, window=None):
    """two batches that run one after the other in the same slots: unequal prompts (1 to `longest` tokens), each
    request decoding 8 to 19 of its tokens one by one, so the first batch shrinks from n_first through 32 to nothing.
    The decoded tokens are probes. The needle stands near the start of the request (far from the probes); in every
    third request it stands 62 positions before the first decoded token, so that it leaves a window of 70 positions
    while the request is decoded"""
    rng = random.Random(seed)
    lengths = [rng.randrange(9, longest) for _ in range(n_first + n_second)]
    lengths[0], lengths[1], lengths[2] = 9, longest, 64 + 9
    reqs, decode = {}, {}
    for i, n in enumerate(lengths):
        rid = "r%d" % i
        decode[rid] = min(n - 1, 8 + (i * 5) % 12)
        first = n - decode[rid]
        at = rng.randrange(0, max(1, first // 8))
        if window and i % 3 == 0 and first - (window - 8) >= 0:
            at = first - (window - 8)
        reqs[rid] = tiny.needle_request(vocab, n, at, first, rng)
    ids = list(reqs)
    first = {r: reqs[r] for r in ids[:n_first]}
    second = {r: reqs[r] for r in ids[n_first:]}
    steps = tiny.trace_group(first, decode)
    steps += tiny.trace_group(second, decode, first_step=len(steps))
    return reqs, steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,n_first", [("D", 48), ("E", 64)])
def test_wide_decode_batches_match_plain(tmp_path, name, n_first, dtype):
    from kindi_b200.engine.engine import Engine
    cfg = tiny.TINY[name][0]
    folder = tiny.make_needle_model(tmp_path, cfg, seed=31, dtype=dtype, name="needle" + name)
    vocab = cfg["vocab_size"]
    reqs, steps = _wide_batches(vocab, n_first, 37, longest=150, seed=17, window=cfg.get("sliding_window"))
    sizes = [len(s["entries"]) for s in steps]
    assert max(sizes) == n_first and any(32 <= b < n_first for b in sizes[1:]) and any(b < 32 for b in sizes)
    m = P.load_model(folder)
    want = {rid: P.forward(m, toks).numpy() for rid, toks in reqs.items()}
    eng = Engine(folder, ctx=tiny.max_live_tokens(steps), dtype=dtype, max_batch=n_first)
    out = str(tmp_path / "out")
    tiny.run_replay(eng, steps, out)
    eng.check_status()
    eng.cache.check()
    assert eng.cache.slots.n_held == 0 and all(g.pages.pool.n_held == 0 for g in eng.cache.groups)
    assert eng.graph_replays > 0                                   # batch sizes that lasted were recorded
    _compare(tiny.collect(out, steps, vocab), reqs, want, TOL[dtype], "%s %s" % (name, dtype))


def test_wide_decode_batch_at_layer_sizes(tmp_path):
    """64 sequences at the benchmark's layer sizes (two layers): the decode step that the batch-64 point of the
    benchmark times, checked against the plain model"""
    from kindi_b200.engine.engine import Engine
    folder = tiny.make_needle_model(tmp_path, LAYER_SIZED, seed=41, dtype="bfloat16", name="layer_sized")
    vocab = LAYER_SIZED["vocab_size"]
    reqs, steps = _wide_batches(vocab, 64, 8, longest=40, seed=23)
    m = P.load_model(folder, dtype=torch.float32)                  # (float64 would take minutes at this width)
    want = {rid: P.forward(m, toks).numpy() for rid, toks in reqs.items()}
    del m
    eng = Engine(folder, ctx=tiny.max_live_tokens(steps), dtype="bfloat16", max_batch=64)
    out = str(tmp_path / "out")
    tiny.run_replay(eng, steps, out)
    eng.check_status()
    eng.cache.check()
    _compare(tiny.collect(out, steps, vocab), reqs, want, TOL["bfloat16"], "layer-sized")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_context_of_more_than_8192_positions(tmp_path, dtype):
    """one request of 8,230 tokens: the prompt goes through pieces of max_step_tokens, the last 32 tokens one by one,
    alone (the most position splits) and inside a batch of 8 (fewer splits, other sequences' pages in between); its
    pages are numbered in the thousands"""
    from kindi_b200.engine.batch import StepEntry
    from kindi_b200.engine.engine import Engine
    folder = tiny.make_needle_model(tmp_path, LONG, seed=51, dtype=dtype, name="long")
    vocab = LONG["vocab_size"]
    n = 8230
    lengths = [n, 300, 77, 1000, 129, 64, 500, 40]
    rng = random.Random(29)
    # the needle at position 5 of each request, probes as its last 32 tokens (those that are decoded one by one)
    reqs = {"r%d" % i: tiny.needle_request(vocab, k, 5, k - min(32, k - 1), rng) for i, k in enumerate(lengths)}
    m = P.load_model(folder)
    long_id = "r0"
    want_long = P.forward(m, reqs[long_id]).numpy()
    tol = TOL[dtype]
    # ---- alone: prompt in pieces of 2,048, then 32 single tokens; low page numbers are taken by a parked slot
    eng = Engine(folder, ctx=200000, dtype=dtype, max_batch=8, max_step_tokens=2048)
    parked = eng.alloc()
    eng.cache.reserve(parked, 150000)                              # pages 0 .. 2343 are taken
    slot = eng.alloc()
    toks = reqs[long_id]
    k = n - 32
    logits = eng.step([StepEntry(slot, tuple(toks[:k]), (0, 1, 63, 64, 2047, 2048, 4095, 4096, 8191, k - 1))])
    assert eng.steps_run == 5                                      # 8,198 tokens in pieces of 2,048
    rows = [0, 1, 63, 64, 2047, 2048, 4095, 4096, 8191, k - 1]
    assert tiny.rel_err(logits.cpu().numpy(), want_long[rows]) <= tol
    assert min(eng.cache.groups[0].pages.rows[slot].values()) >= 2000
    got = [eng.step([StepEntry(slot, (t,), (0,))])[0].cpu().numpy() for t in toks[k:]]
    eng.check_status()
    err = tiny.rel_err(np.stack(got), want_long[k:])
    assert err <= tol, "alone, last 32: %.3g" % err
    eng.free(slot)
    eng.free(parked)
    eng.cache.check()
    del eng
    # ---- in a batch of 8 that starts together (one piece of up to 8,192 tokens a step), last 32 one by one
    want = {rid: (want_long if rid == long_id else P.forward(m, t).numpy()) for rid, t in reqs.items()}
    steps = tiny.trace_group(reqs, {r: min(32, len(t) - 1) for r, t in reqs.items()})
    eng = Engine(folder, ctx=tiny.max_live_tokens(steps), dtype=dtype, max_batch=8)
    out = str(tmp_path / "batch")
    for s in steps:                                                # logits of the long prompt's rows: only a few
        for e in s["entries"]:
            if len(e["tokens"]) > 256:
                e["want"] = [w for w in (0, 100, 4000, len(e["tokens"]) - 1) if w < len(e["tokens"])]
    tiny.run_replay(eng, steps, out)
    eng.check_status()
    got = tiny.collect(out, steps, vocab)
    for rid, t in reqs.items():
        have = sorted(i for (r, i) in got if r == rid)
        assert set(range(len(t) - min(32, len(t) - 1), len(t))) <= set(have)       # the tokens decoded one by one
        mine = np.stack([got[(rid, i)] for i in have])
        err = tiny.rel_err(mine, want[rid][have])
        assert err <= tol, "batch of 8, %s: %.3g" % (rid, err)
    eng.cache.check()


def test_sampled_generation_walks_the_plain_model_and_sampler(tmp_path):
    """configuration B, prompts of 1 / 7 / 16 / 23 tokens, temperature 0.8 with a fixed seed, 6 tokens each, in
    32-bit: every token is the one the plain sampler draws from the plain model's logits with the sequence's own
    uniform number. A token may differ only where the number falls within 1e-4 of the boundary between the two
    tokens' shares (then the walk goes on from the engine's token)."""
    from kindi_b200 import Engine
    from kindi_b200.sampling.sampler import SequenceRandom
    d = tiny.make_model(tmp_path, "B", "float32")
    m = P.load_model(d)
    eng = Engine(d, ctx=1024, dtype="float32", max_batch=4)
    prompts = list(tiny.random_requests(384, [1, 7, 16, 23], seed=1).values())
    for opts in (dict(temperature=0.8, top_p=1.0, top_k=0), dict(temperature=0.8, top_p=0.9, top_k=40)):
        res = eng.generate_batch(prompts, seed=4321, max_tokens=6, stop_token_ids=(), **opts)
        differ = 0
        for i, (p, got) in enumerate(zip(prompts, res.tokens)):
            assert len(got) == 6 or res.finish[i] == "stop"
            rng = SequenceRandom(4321, i)
            seq = list(p)
            for t in got:
                u = rng.next()
                z = P.forward(m, seq)[-1].numpy()
                mine = P.sample_with_u(z, u, opts["temperature"], opts["top_p"], opts["top_k"])
                if t != mine:
                    differ += 1
                    ids, prob = P.sampling_distribution(z, opts["temperature"], opts["top_p"], opts["top_k"])
                    o = np.argsort(ids)
                    ids, c = ids[o], np.cumsum(prob[o])
                    assert t in ids, (i, len(seq), t)
                    a, b = sorted((int(np.where(ids == t)[0][0]), int(np.where(ids == mine)[0][0])))
                    assert b == a + 1 and abs(c[a] - u) <= 1e-4, (i, len(seq), t, mine, u, c[a])
                seq.append(t)
        assert differ <= 1
        assert len({tuple(t) for t in res.tokens}) > 1                 # sampling, not one fixed run
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_in_portions_of_any_size_sees_the_needle(tmp_path, dtype):
    """a request brought in portions of 64, 2, 70, 1 and 33 tokens and then token by token (each portion reads the
    earlier ones from the cache; the two-token and one-token portions are prompt-shaped and decode-shaped steps in the
    middle of a prompt), in a slot and in pages that another request used before, with a window on one layer: every
    row equals the whole-sequence plain model, and the probe rows rest on the needle near the start"""
    from kindi_b200.engine.batch import StepEntry
    from kindi_b200.engine.engine import Engine
    cfg = tiny.TINY["E"][0]
    folder = tiny.make_needle_model(tmp_path, cfg, seed=31, dtype=dtype, name="needleE")
    vocab = cfg["vocab_size"]
    rng = random.Random(5)
    toks = tiny.needle_request(vocab, 190, 2, 120, rng)
    other = tiny.needle_request(vocab, 150, 7, 100, rng)
    want = P.forward(P.load_model(folder), toks).numpy()
    eng = Engine(folder, ctx=256, dtype=dtype, max_batch=1)
    slot = eng.alloc()
    eng.step([StepEntry(slot, tuple(other), ())])                  # leaves its keys in the pages that come next
    eng.free(slot)
    slot = eng.alloc()
    rows, at = [], 0
    for n in (64, 2, 70, 1, 33) + (1,) * 20:
        part = tuple(toks[at:at + n])
        rows.append(eng.step([StepEntry(slot, part, tuple(range(n)))]).cpu().numpy())
        at += n
    eng.check_status()
    assert at == 190
    err = tiny.rel_err(np.concatenate(rows), want)
    assert err <= TOL[dtype], err
    eng.free(slot)
    eng.cache.check()


def test_window_layers_keep_a_small_pool_over_a_long_sequence(tmp_path):
    """the layer with a window of 70 positions holds 14 pages while two sequences grow to 1,500 and 400 tokens (pages
    behind the window are given back and used again many times); the layers that keep every key hold them all"""
    from kindi_b200.engine.engine import Engine
    cfg = tiny.TINY["E"][0]
    folder = tiny.make_needle_model(tmp_path, cfg, seed=31, dtype="bfloat16", name="needleE")
    vocab = cfg["vocab_size"]
    rng = random.Random(11)
    reqs = {"a": tiny.needle_request(vocab, 1500, 1500 - 20 - 62, 1500 - 20, rng),
            "b": tiny.needle_request(vocab, 400, 4, 380, rng)}
    m = P.load_model(folder)
    want = {r: P.forward(m, t).numpy() for r, t in reqs.items()}
    steps = tiny.trace_group(reqs, {"a": 20, "b": 20})
    for e in steps[0]["entries"]:
        e["want"] = [0, 69, 70, 71, 127, 128, len(e["tokens"]) - 1]
    eng = Engine(folder, ctx=tiny.max_live_tokens(steps), dtype="bfloat16", max_batch=2, max_step_tokens=128)
    win = [g for g in eng.cache.groups if g.need.window][0]
    assert win.n_pool_pages == 2 * (2 + 4) + 2 and win.n_pool_pages < eng.cache.n_pages
    out = str(tmp_path / "out")
    tiny.run_replay(eng, steps, out)
    eng.check_status()
    got = tiny.collect(out, steps, vocab)
    for r in reqs:
        have = sorted(i for (rid, i) in got if rid == r)
        assert len(have) == 27
        err = tiny.rel_err(np.stack([got[(r, i)] for i in have]), want[r][have])
        assert err <= TOL["bfloat16"], (r, err)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_short_prompt_steps_are_recorded_and_padding_changes_nothing(tmp_path, dtype):
    """prompt steps of up to 512 tokens are padded to a multiple of 64 rows and replayed from a recording once their
    shape has been seen twice. Prompts of 100, 90, 128, 65 and 70 tokens share the 128-row recording, pairs of unequal
    prompts another; a step that wants no row is recorded too. Every logit equals the plain model; in 32-bit the
    recorded steps give the same bits as an engine that records nothing; the padding rows store nothing (the next
    tokens of each sequence still see exactly their own keys)"""
    from kindi_b200.engine.batch import StepEntry
    from kindi_b200.engine.engine import Engine
    cfg = tiny.TINY["E"][0]
    folder = tiny.make_needle_model(tmp_path, cfg, seed=31, dtype=dtype, name="needleE")
    vocab = cfg["vocab_size"]
    m = P.load_model(folder)
    rng = random.Random(9)
    eng = Engine(folder, ctx=4096, dtype=dtype, max_batch=4)
    plain_eng = Engine(folder, ctx=4096, dtype=dtype, max_batch=4, cuda_graphs=False)

    def run(e, groups, follow=3):
        """each group of prompts is one step that wants the last row of each; then `follow` tokens one by one"""
        out = []
        for group in groups:
            slots = [e.alloc() for _ in group]
            k = [len(t) - follow for t in group]
            logits = e.step([StepEntry(s, tuple(t[:n]), (n - 1,)) for s, t, n in zip(slots, group, k)])
            rows = [[logits[i].cpu().numpy()] for i in range(len(group))]
            for j in range(follow):
                lg = e.step([StepEntry(s, (t[n + j],), (0,)) for s, t, n in zip(slots, group, k)])
                for i in range(len(group)):
                    rows[i].append(lg[i].cpu().numpy())
            e.check_status()
            for s in slots:
                e.free(s)
            out.append([np.stack(r) for r in rows])
        return out

    lengths = [[103], [93], [131], [68], [73], [40, 71], [64, 9], [8, 100], [200], [260], [300]]
    groups = [[tiny.needle_request(vocab, n, 1, n - 5, rng) for n in g] for g in lengths]
    got = run(eng, groups)
    assert sum(1 for k in eng._graphs if k[0] == "prompt") >= 2 and eng.graph_replays >= 6
    same = run(plain_eng, groups)
    for g, mine, other in zip(groups, got, same):
        for toks, a, b in zip(g, mine, other):
            want = P.forward(m, toks).numpy()[len(toks) - 4:]
            assert tiny.rel_err(a, want) <= TOL[dtype], (len(toks), tiny.rel_err(a, want))
            if dtype == "float32":
                assert np.array_equal(a, b), len(toks)
    # a prompt brought in two steps, the first of which wants nothing (recorded at its second occurrence)
    for n in (150, 170, 190):
        toks = tiny.needle_request(vocab, n, 2, n - 20, rng)
        s = eng.alloc()
        assert eng.step([StepEntry(s, tuple(toks[:100]), ())]) is None
        lg = eng.step([StepEntry(s, tuple(toks[100:]), (n - 101,))])[0].cpu().numpy()
        eng.check_status()
        eng.free(s)
        assert tiny.rel_err(lg, P.forward(m, toks).numpy()[-1]) <= TOL[dtype]
    assert ("prompt", 128, 1, 0) in eng._graphs
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


def test_recorded_prompt_shapes_are_kept_up_to_a_limit(tmp_path):
    """only so many recorded prompt shapes are kept (each holds buffers of its own): the oldest makes room, and a shape
    that was dropped is recorded again when it comes back"""
    from kindi_b200.engine.batch import StepEntry
    from kindi_b200.engine.engine import Engine
    cfg = tiny.TINY["D"][0]
    folder = tiny.make_model(tmp_path, "D", "bfloat16")
    m = P.load_model(folder)
    eng = Engine(folder, ctx=2048, dtype="bfloat16", max_batch=2)
    eng.prompt_graphs_kept = 2
    rng = random.Random(3)
    for n in (50, 60, 100, 110, 150, 160, 40, 45, 130, 170, 55):
        toks = [rng.randrange(cfg["vocab_size"]) for _ in range(n)]
        s = eng.alloc()
        lg = eng.step([StepEntry(s, tuple(toks), (n - 1,))])[0].cpu().numpy()
        eng.check_status()
        eng.free(s)
        assert tiny.rel_err(lg, P.forward(m, toks).numpy()[-1]) <= TOL["bfloat16"], n
        assert sum(1 for k in eng._graphs if k[0] == "prompt") <= 2
    assert ("prompt", 64, 1, 1) in eng._graphs and ("prompt", 192, 1, 1) in eng._graphs
    assert ("prompt", 128, 1, 1) not in eng._graphs
