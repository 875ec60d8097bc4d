"""Generation through the Python entry point and the command line, the sampling kernel against the plain sampler,
long decoding, the first tokens of a sequence, and bin/trace_run as a program."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_model as P
import tiny

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _check_greedy(m, prompt, got, tie):
    """every generated token is the plain model's argmax, or differs from it only where the plain logits are within
    `tie` (relative to the largest logit) of each other"""
    seq = list(prompt)
    for t in got:
        z = P.forward(m, seq)[-1].numpy()
        best = int(np.argmax(z))
        assert t == best or z[best] - z[t] <= tie * np.abs(z).max(), (len(seq), t, best, z[best] - z[t])
        seq.append(t)


@pytest.mark.parametrize("dtype,tie", [("float32", 1e-5), ("bfloat16", 1.5e-2)])
@pytest.mark.parametrize("name", ["A", "D"])
def test_greedy_generation_through_the_entry_point(tmp_path, name, dtype, tie):
    from kindi_b200 import Engine
    d = tiny.make_model(tmp_path, name, dtype)
    m = P.load_model(d)
    eng = Engine(d, ctx=2048, dtype=dtype, max_batch=3)
    vocab = tiny.TINY[name][0]["vocab_size"]
    prompts = list(tiny.random_requests(vocab, [5, 9, 13, 1, 70], seed=3).values())
    res = eng.generate_batch(prompts, temperature=0.0, max_tokens=8, stop_token_ids=())
    assert res.stats.batches == 2 and eng.cache.slots.n_held == 0
    for p, got, fin in zip(prompts, res.tokens, res.finish):
        assert fin in ("length", "stop") and (len(got) == 8 or fin == "stop")
        _check_greedy(m, p, got, tie)
    # the reference-style call: exactly n greedy tokens of one prompt, the same as in the batch
    alone = eng.generate(prompts[1], 8)
    if dtype == "float32":
        assert alone[:len(res.tokens[1])] == res.tokens[1]
    _check_greedy(m, prompts[1], alone, tie)
    eng.cache.check()


def test_long_decoding_stays_on_the_plain_model(tmp_path):
    """300 tokens decoded one by one after a short prompt (five pages of cache, decode graphs replayed): the logits
    at the end still agree with the plain model run on the whole sequence"""
    from kindi_b200 import Engine, StepEntry
    for dtype, tol in (("float32", 2e-5), ("bfloat16", 1.5e-2)):
        d = tiny.make_model(tmp_path, "D", dtype)
        eng = Engine(d, ctx=1024, dtype=dtype, max_batch=2)
        toks = list(tiny.random_requests(500, [320], seed=8).values())[0]
        slot = eng.alloc()
        eng.step([StepEntry(slot, tuple(toks[:20]), ())])
        rows = []
        for t in toks[20:]:
            rows.append(eng.step([StepEntry(slot, (t,), (0,))])[0].cpu().numpy())
        eng.check_status()
        assert eng.graph_replays > 250
        want = P.forward(P.load_model(d), toks).numpy()[20:]
        assert tiny.rel_err(np.stack(rows), want) < tol
        eng.free(slot)


def test_first_tokens_of_a_sequence(tmp_path):
    """a one-token prompt, then tokens one by one: positions 0, 1, 2 ... each see exactly the tokens before them"""
    from kindi_b200 import Engine, StepEntry
    d = tiny.make_model(tmp_path, "E", "float32")
    eng = Engine(d, ctx=256, dtype="float32", max_batch=2)
    toks = [11, 700, 3, 3, 42, 0, 776]
    slot = eng.alloc()
    rows = [eng.step([StepEntry(slot, (t,), (0,))])[0].cpu().numpy() for t in toks]
    want = P.forward(P.load_model(d), toks).numpy()
    assert tiny.rel_err(np.stack(rows), want) < 2e-5
    assert np.abs(rows[0] - want[0]).max() / np.abs(want[0]).max() < 1e-5


def _plain_pick(z, u, params, history=None):
    if params.repeat_penalty != 1.0 and history is not None:
        from kindi_b200.sampling.sampler import recent_tokens
        z = P.penalize(z, params.repeat_penalty, recent_tokens(history, params.repeat_last_n))
    return P.sample_with_u(z, u, params.temperature, params.top_p, params.top_k, params.min_p, params.order)


@pytest.mark.parametrize("opts", [
    dict(temperature=0.0), dict(temperature=0.7, top_p=0.8, top_k=20), dict(temperature=1.3, top_p=1.0, top_k=0),
    dict(temperature=0.5, top_p=0.6, top_k=0, min_p=0.02), dict(temperature=1.0, top_p=0.9, top_k=7, order="hf"),
    dict(temperature=0.8, top_p=0.95, top_k=50, repeat_penalty=1.3, repeat_last_n=4),
    dict(temperature=0.0, repeat_penalty=1.5, repeat_last_n=-1), dict(temperature=0.9, top_p=0.3, top_k=1),
])
def test_sampling_kernel_against_the_plain_sampler(opts):
    from kindi_b200.config.runtime import SamplingParams
    from kindi_b200.sampling.sampler import Sampler
    params = SamplingParams(**opts)
    rng = np.random.RandomState(1)
    for V in (331, 4099):
        R = 7
        z = (rng.randn(R, V) * 2.5).astype(np.float32)
        z[2, 5] = z[2, 9] = z[2].max() + 1.0                        # an exact tie of the two best
        us = [0.0, 0.13, 0.5, 0.77, 0.999, 0.31, 0.62]
        hist = [list(rng.randint(0, V, size=9)) for _ in range(R)]
        hist[2] = [5, 5, 9, 1]
        got = Sampler("cuda").pick(torch.from_numpy(z).cuda(), params, us, hist).tolist()
        for r in range(R):
            assert got[r] == _plain_pick(z[r].astype(np.float64), us[r], params, hist[r]), (V, r, opts)


@pytest.mark.parametrize("R", [19, 21, 38, 75, 160])
def test_sampling_kernel_with_many_rows(R):
    """a row is shared by eight, four, two CTAs or has one to itself, depending on how many rows there are: the same
    picks as the plain sampler in every case, with ties and with a vocabulary that no slice divides"""
    from kindi_b200.config.runtime import SamplingParams
    from kindi_b200.sampling.sampler import Sampler
    rng = np.random.RandomState(R)
    for V, opts in ((1001, dict(temperature=0.8, top_p=0.9, top_k=40)), (4099, dict(temperature=1.2, top_p=0.7, top_k=0)),
                    (331, dict(temperature=0.6, top_p=1.0, top_k=5, min_p=0.1, order="hf"))):
        params = SamplingParams(**opts)
        z = np.round(rng.randn(R, V) * 10) / 4.0                    # multiples of 0.25: ties everywhere
        z = z.astype(np.float32)
        us = [float(u) for u in rng.rand(R)]
        got = Sampler("cuda").pick(torch.from_numpy(z).cuda(), params, us, None).tolist()
        want = [_plain_pick(z[r].astype(np.float64), us[r], params) for r in range(R)]
        assert got == want, (R, V, opts)


def test_sampling_kernel_takes_minus_zero_for_zero():
    """logits of -0 and +0 are one value: a cut that falls on a zero keeps both (rounded logits, so ties abound)"""
    from kindi_b200.config.runtime import SamplingParams
    from kindi_b200.sampling.sampler import Sampler
    params = SamplingParams(temperature=1.5, top_p=0.95, top_k=7, min_p=0.2, order="hf")
    z = np.array([-0.0, 0.5, 0.0, -0.75, 2.0 / 3, -0.75, 0.75, 0.0, 0.0, -0.5, -0.75, 0.25, -0.0, 0.75, 0.0, -1.0, 0.0],
                 dtype=np.float32)
    us = [0.0, 0.06, 0.2, 0.5, 0.74, 0.9, 0.999]
    got = Sampler("cuda").pick(torch.from_numpy(np.tile(z, (len(us), 1))).cuda(), params, us, [[]] * len(us)).tolist()
    want = [_plain_pick(z.astype(np.float64), u, params) for u in us]
    assert got == want and want[0] == 0 and 12 in want


def test_sampled_tokens_do_not_depend_on_the_batch(tmp_path):
    from kindi_b200 import Engine
    d = tiny.make_model(tmp_path, "B", "float32")
    eng = Engine(d, ctx=1024, dtype="float32", max_batch=4)
    prompts = list(tiny.random_requests(384, [1, 7, 16, 23], seed=1).values())
    kw = dict(temperature=0.8, top_p=0.9, top_k=0, max_tokens=6, seed=1234, stop_token_ids=())
    a = eng.generate_batch(prompts, **kw)
    b = eng.generate_batch(prompts, **kw)
    assert a.tokens == b.tokens                                        # the same seed gives the same tokens
    eng2 = Engine(d, ctx=1024, dtype="float32", max_batch=2)           # other batches: [0, 1] and [2, 3]
    c = eng2.generate_batch(prompts, **kw)
    assert c.tokens == a.tokens and c.stats.batches == 2
    assert eng.generate_batch(prompts, **dict(kw, seed=99)).tokens != a.tokens


def test_stop_tokens_and_context_limit(tmp_path):
    from kindi_b200 import Engine
    from kindi_b200.engine.generate import PromptTooLong
    d = tiny.make_model(tmp_path, "A", "float32")
    eng = Engine(d, ctx=128, dtype="float32", max_batch=2)
    p = [3, 1, 4, 1, 5]
    free = eng.generate(p, 6)
    res = eng.generate_batch([p], temperature=0.0, max_tokens=6, stop_token_ids=(free[3],))
    first = free.index(free[3])
    assert res.tokens[0] == free[:first] and res.finish == ["stop"]
    with pytest.raises(PromptTooLong):
        eng.generate_batch([[1] * 128], temperature=0.0)
    long = eng.generate_batch([[1] * 120], temperature=0.0, max_tokens=100, stop_token_ids=())
    assert len(long.tokens[0]) == 8 and eng.cache.slots.n_held == 0


def test_trace_run_and_command_line_as_programs(tmp_path):
    d = tiny.make_model(tmp_path, "A", "bfloat16")
    reqs = tiny.random_requests(256, [5, 40], seed=2)
    steps = tiny.trace_batched(reqs, batch=2, decode=4)
    out = str(tmp_path / "out")
    env = dict(os.environ, PYTHONDONTWRITEBYTECODE="1")
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", "bfloat16", "--out", out,
                        "--max-tokens", str(tiny.max_live_tokens(steps))],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, env=env,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.split("\n") if l] == ["done %d" % s["step"] for s in steps]
    got = tiny.collect(out, steps, 256)
    m = P.load_model(d)
    for rid, toks in reqs.items():
        mine = np.stack([got[(rid, i)] for i in range(len(toks))])
        assert tiny.rel_err(mine, P.forward(m, toks).numpy()) < 1.5e-2
    r = subprocess.run([sys.executable, "-m", "kindi_b200", "--model", d, "--ctx", "512", "generate", "--prompt-ids",
                        "1,2,3", "--prompt-ids", "9 8", "--temperature", "0", "--max-tokens", "5"],
                       capture_output=True, text=True, cwd=ROOT, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(l) for l in r.stdout.strip().split("\n")]
    assert len(lines) == 2 and all(len(l["tokens"]) <= 5 for l in lines)
    r = subprocess.run([sys.executable, "-m", "kindi_b200", "--model", d, "--ctx", "512", "verify"],
                       capture_output=True, text=True, cwd=ROOT, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
