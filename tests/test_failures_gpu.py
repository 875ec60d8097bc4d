"""Failure paths, none of which faults, traps or hangs the GPU: a wait inside a kernel that runs out, a cache position
without a mapped page, a cache that is full in the middle of a step, and a model that does not fit the device. After
each the engine says what happened and goes on working: the next steps equal the plain model."""
import numpy as np
import pytest
import torch

import plain_model as P
import tiny

pytestmark = pytest.mark.gpu


def _engine(tmp_path, dtype="bfloat16", name="D", **kw):
    from kindi_b200.engine.engine import Engine
    d = tiny.make_model(tmp_path, name, dtype)
    kw.setdefault("ctx", 1024)
    kw.setdefault("max_batch", 4)
    return d, Engine(d, dtype=dtype, **kw)


def _healthy(eng, folder, dtype, seed):
    """a prompt and six single tokens equal the plain model"""
    from kindi_b200.engine.batch import StepEntry
    vocab = eng.spec.vocab_size
    toks = list(tiny.random_requests(vocab, [90], seed=seed).values())[0]
    slot = eng.alloc()
    rows = [eng.step([StepEntry(slot, tuple(toks[:84]), (83,))])[0].cpu().numpy()]
    rows += [eng.step([StepEntry(slot, (t,), (0,))])[0].cpu().numpy() for t in toks[84:]]
    eng.check_status()
    eng.free(slot)
    want = P.forward(P.load_model(folder), toks).numpy()[83:]
    assert tiny.rel_err(np.stack(rows), want) <= (2e-5 if dtype == "float32" else 1.5e-2)


def test_a_wait_that_runs_out_is_reported_and_the_engine_goes_on(tmp_path):
    from kindi_b200.engine.engine import EngineError
    from kindi_b200.kernels import fast, lib as K
    folder, eng = _engine(tmp_path)
    _healthy(eng, folder, "bfloat16", 1)
    # the library's bounded wait on a barrier nobody arrives at, with a limit of one millisecond
    timed_out, ns = K.wait_selftest(eng.status, 1_000_000)
    assert timed_out and 1_000_000 <= ns < 50_000_000
    assert int(eng.status.item()) & K.ST_WAIT_TIMEOUT
    # what a lost arrival can leave behind: a raised flag in the scratch of a product
    for _, flags in list(fast._SK_SCRATCH.values()):
        flags.fill_(1)
    with pytest.raises(EngineError) as e:
        eng.check_status()
    assert "wait" in str(e.value)
    assert int(eng.status.item()) == 0
    assert all(int(flags.sum()) == 0 for _, flags in fast._SK_SCRATCH.values())
    _healthy(eng, folder, "bfloat16", 2)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_position_without_a_page_is_reported_not_read(tmp_path, dtype):
    from kindi_b200.engine.batch import StepEntry
    from kindi_b200.engine.engine import EngineError
    folder, eng = _engine(tmp_path, dtype)
    toks = list(tiny.random_requests(500, [150], seed=3).values())[0]
    slot = eng.alloc()
    eng.step([StepEntry(slot, tuple(toks[:140]), ())])
    eng.check_status()
    table = eng.cache.groups[0].table
    keep = int(table[slot, 1])
    table[slot, 1] = -1                                        # positions 64..127 lose their page
    for t in toks[140:143]:                                    # (the third step of this shape is a recorded one)
        eng.step([StepEntry(slot, (t,), (0,))])
    with pytest.raises(EngineError) as e:
        eng.check_status()
    assert "page" in str(e.value)
    table[slot, 1] = keep
    eng.free(slot)
    eng.cache.check()
    _healthy(eng, folder, dtype, 4)


def test_a_full_cache_inside_a_step_leaves_slots_and_pages_consistent(tmp_path):
    from kindi_b200.cache.pages import CacheFull
    from kindi_b200.engine.batch import StepEntry
    folder, eng = _engine(tmp_path, "bfloat16", ctx=256)      # four pages in all
    vocab = eng.spec.vocab_size
    a, b = eng.alloc(), eng.alloc()
    ta = list(tiny.random_requests(vocab, [100], seed=5).values())[0]
    tb = list(tiny.random_requests(vocab, [140], seed=6).values())[0]
    eng.step([StepEntry(a, tuple(ta[:60]), ())])              # one page
    with pytest.raises(CacheFull) as e:
        eng.step([StepEntry(a, tuple(ta[60:100]), ()), StepEntry(b, tuple(tb), ())])      # needs 1 + 3 more pages
    assert "ctx = 256" in str(e.value)
    eng.cache.check()
    assert eng.length(a) == 60 and eng.length(b) == 0         # nothing of the failed step counts
    eng.free(b)
    eng.cache.check()
    # the sequence that was there goes on, and its logits are right
    got = eng.step([StepEntry(a, tuple(ta[60:100]), tuple(range(40)))]).cpu().numpy()
    eng.check_status()
    want = P.forward(P.load_model(folder), ta).numpy()[60:]
    assert tiny.rel_err(got, want) <= 1.5e-2
    eng.free(a)
    eng.cache.check()
    assert eng.cache.slots.n_held == 0 and all(g.pages.pool.n_held == 0 for g in eng.cache.groups)
    _healthy(eng, folder, "bfloat16", 7)


def test_a_model_that_does_not_fit_is_refused_before_anything_is_allocated(tmp_path):
    from kindi_b200.engine.engine import Engine, OutOfDeviceMemory
    d = tiny.make_model(tmp_path, "D", "bfloat16")
    said = []
    before = torch.cuda.memory_allocated()
    with pytest.raises(OutOfDeviceMemory) as e:
        Engine(d, ctx=2_000_000_000, dtype="bfloat16", max_batch=4, log=said.append)     # a terabyte of cache
    assert "cache" in str(e.value) and "GiB free" in str(e.value)
    assert torch.cuda.memory_allocated() == before
    assert any("memory plan" in s for s in said)
    eng = Engine(d, ctx=512, dtype="bfloat16", max_batch=4, log=said.append)
    assert eng.plan["total"] < eng.plan["free"] and eng.plan["cache"] > 0 and eng.plan["weights"] > 0


def test_position_limit_of_the_configuration(tmp_path):
    """max_position_embeddings bounds a sequence: the step function refuses to go past it, generation stops there"""
    from kindi_b200.engine.batch import StepEntry
    from kindi_b200.engine.engine import Engine, EngineError
    from kindi_b200.engine.generate import PromptTooLong
    from kindi_b200.weights.random_init import write_random_model
    cfg = dict(tiny.TINY_A, max_position_embeddings=40)
    d = write_random_model(str(tmp_path / "m"), cfg, 0, dtype="float32")
    eng = Engine(d, ctx=512, dtype="float32", max_batch=2)
    slot = eng.alloc()
    eng.step([StepEntry(slot, tuple(range(1, 40)), ())])
    eng.step([StepEntry(slot, (5,), (0,))])
    with pytest.raises(EngineError) as e:
        eng.step([StepEntry(slot, (6,), (0,))])
    assert "max_position_embeddings" in str(e.value) and eng.length(slot) == 40
    eng.free(slot)
    res = eng.generate_batch([list(range(1, 31))], temperature=0.0, max_tokens=100, stop_token_ids=())
    assert len(res.tokens[0]) == 10 and res.finish == ["length"]
    with pytest.raises(PromptTooLong):
        eng.generate_batch([list(range(1, 41))], temperature=0.0)
