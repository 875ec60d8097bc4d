"""Replay on the GPU against the plain implementation: each request whole; with its last 32 tokens one by one; in
batches of unequal lengths whose shorter requests end earlier, one batch after another so that slots and pages are
used again. In 32-bit and in bfloat16, for every tiny configuration."""
import numpy as np
import pytest
import torch

import plain_model as P
import tiny

pytestmark = pytest.mark.gpu

# max |engine - plain| / max |plain| over a request's logits. 32-bit: sums of a few hundred terms in another order
# than the float64 reference. bfloat16: activations and cached keys/values are rounded to 8 bits of mantissa between
# the operations (2^-9 relative each), a handful of roundings per layer.
TOL = {"float32": 2e-5, "bfloat16": 1.5e-2}
LENGTHS = [5, 9, 13, 1, 70, 130, 33, 64, 97]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {(n, d): tiny.make_model(root, n, d) for n in tiny.TINY for d in ("bfloat16", "float32")}


def _plain_logits(model_dir, reqs):
    m = P.load_model(model_dir)
    return {rid: P.forward(m, toks).numpy() for rid, toks in reqs.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_replay_modes_match_plain(models, tmp_path, name, dtype):
    from kindi_b200.engine.engine import Engine
    # the float32 run reads the folder stored in float32, the bfloat16 run the one stored in bfloat16
    model_dir = models[(name, dtype)]
    vocab = tiny.TINY[name][0]["vocab_size"]
    reqs = tiny.random_requests(vocab, LENGTHS, seed=11)
    want = _plain_logits(model_dir, reqs)
    traces = {"whole": tiny.trace_whole(reqs), "last32": tiny.trace_last_n(reqs, 32),
              "batched": tiny.trace_batched(reqs, batch=4, decode=12)}
    results = {}
    for mode, steps in traces.items():
        eng = Engine(model_dir, ctx=tiny.max_live_tokens(steps), dtype=dtype, max_batch=4)
        out = str(tmp_path / mode)
        tiny.run_replay(eng, steps, out)
        eng.cache.check()
        assert eng.cache.slots.n_held == 0 and all(g.pages.pool.n_held == 0 for g in eng.cache.groups)
        results[mode] = tiny.collect(out, steps, vocab)
        del eng
    worst = 0.0
    for mode, got in results.items():
        assert len(got) == sum(len(t) for t in reqs.values()), mode
        for rid, toks in reqs.items():
            mine = np.stack([got[(rid, i)] for i in range(len(toks))])
            err = tiny.rel_err(mine, want[rid])
            worst = max(worst, err)
            assert err <= TOL[dtype], "%s %s %s: %.3g" % (mode, rid, dtype, err)
    print("worst relative error %s %s: %.3g" % (name, dtype, worst))
    if dtype == "float32":
        # the 32-bit path sums in an order that depends on positions only: the three ways of cutting agree bit for bit
        for key, row in results["whole"].items():
            assert np.array_equal(row, results["last32"][key]), ("last32", key)
            assert np.array_equal(row, results["batched"][key]), ("batched", key)


@pytest.mark.parametrize("stored,run", [("float32", "bfloat16"), ("bfloat16", "float32")])
def test_folder_stored_in_the_other_dtype(models, tmp_path, stored, run):
    """a 32-bit folder run in bfloat16 keeps its tensors in 32-bit (the products then take 32-bit weights and bfloat16
    activations); a bfloat16 folder run in 32-bit is widened exactly"""
    from kindi_b200.engine.engine import Engine
    model_dir = models[("C", stored)]
    reqs = tiny.random_requests(331, [40, 3, 70], seed=5)
    m = P.load_model(model_dir)
    steps = tiny.trace_batched(reqs, batch=3, decode=8)
    eng = Engine(model_dir, ctx=tiny.max_live_tokens(steps), dtype=run, max_batch=3)
    want_dtype = torch.float32 if stored == "float32" or run == "float32" else torch.bfloat16
    assert eng.model.embedding.table.dtype == want_dtype and eng.model.blocks[0].mixer.wqkv.dtype == want_dtype
    out = str(tmp_path / "o")
    tiny.run_replay(eng, steps, out)
    got = tiny.collect(out, steps, 331)
    for rid, toks in reqs.items():
        mine = np.stack([got[(rid, i)] for i in range(len(toks))])
        assert tiny.rel_err(mine, P.forward(m, toks).numpy()) <= TOL[run]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_steps_run_in_pieces(models, tmp_path, dtype):
    """a step longer than max_step_tokens is run in pieces inside the step function; in 32-bit the logits are the
    same bits as from one whole step"""
    from kindi_b200.engine.engine import Engine
    model_dir = models[("D", dtype)]
    reqs = tiny.random_requests(500, [150, 9, 70, 33], seed=6)
    steps = tiny.trace_batched(reqs, batch=4, decode=5)
    m = P.load_model(model_dir)
    outs = {}
    for name, cap in (("whole", 8192), ("pieces", 64)):
        eng = Engine(model_dir, ctx=tiny.max_live_tokens(steps), dtype=dtype, max_batch=4, max_step_tokens=cap)
        out = str(tmp_path / name)
        tiny.run_replay(eng, steps, out)
        outs[name] = tiny.collect(out, steps, 500)
        if name == "pieces":
            assert eng.steps_run > len(steps)
        eng.cache.check()
    for rid, toks in reqs.items():
        mine = np.stack([outs["pieces"][(rid, i)] for i in range(len(toks))])
        assert tiny.rel_err(mine, P.forward(m, toks).numpy()) <= TOL[dtype]
    if dtype == "float32":
        for k, row in outs["whole"].items():
            assert np.array_equal(row, outs["pieces"][k]), k
