"""The generation loop's decisions, driven by a stand-in stepper: batches, stop tokens, lengths, slots."""
import pytest

from kindi_b200.config.runtime import SamplingParams
from kindi_b200.engine.batch import StepEntry, layout, pack, split_step
from kindi_b200.engine.generate import PromptTooLong, generate, max_new_tokens, plan_batches


class FakeStepper:
    """the next token of a sequence is (sum of its tokens so far) mod 97; it records every step"""

    def __init__(self, ctx=4096, max_batch=4, n_slots=4):
        self.ctx, self.max_batch = ctx, max_batch
        self.free_slots = list(range(n_slots))
        self.held = {}
        self.steps = []
        self.sums = {}

    def alloc(self):
        s = self.free_slots.pop()
        assert s not in self.held
        self.held[s] = True
        self.sums[s] = 0
        return s

    def free(self, slot):
        assert self.held.pop(slot)                  # freeing twice fails here
        self.free_slots.append(slot)

    def run(self, entries, params, seq_ids, histories):
        assert len({e.slot for e in entries}) == len(entries) and all(e.slot in self.held for e in entries)
        self.steps.append([(e.slot, len(e.tokens)) for e in entries])
        out = []
        for e, h in zip(entries, histories):
            self.sums[e.slot] += sum(e.tokens)
            assert self.sums[e.slot] == sum(h)      # the loop fed every token exactly once
            out.append(self.sums[e.slot] % 97)
        return out


def _expect(prompt, n, stop=()):
    seq, out = list(prompt), []
    for _ in range(n):
        t = sum(seq) % 97
        if t in stop:
            return out, "stop"
        out.append(t)
        seq.append(t)
    return out, "length"


def test_unequal_prompts_stop_tokens_and_early_ends():
    st = FakeStepper()
    prompts = [[1, 2, 3], [50], [7] * 20, [9, 9]]
    p = SamplingParams(temperature=0.0, max_tokens=12, stop_token_ids=(31,))
    res = generate(st, prompts, p, stop_token_ids=[4])
    for i, pr in enumerate(prompts):
        want, fin = _expect(pr, 12, stop=(31, 4))
        assert res.tokens[i] == want and res.finish[i] == fin
    assert st.steps[0] == [(s, len(pr)) for (s, _), pr in zip(st.steps[0], prompts)]        # all prompts in one step
    assert all(n == 1 for step in st.steps[1:] for _, n in step)                              # then one token each
    sizes = [len(s) for s in st.steps]
    assert sizes == sorted(sizes, reverse=True) and not st.held                               # shrinking batch, all freed
    assert res.stats.generated_tokens == sum(len(t) for t in res.tokens) and res.stats.batches == 1


def test_batches_one_after_another_reuse_slots():
    st = FakeStepper(max_batch=2, n_slots=2)
    prompts = [[i + 1] * (i + 1) for i in range(5)]
    res = generate(st, prompts, SamplingParams(temperature=0.0, max_tokens=3))
    assert res.stats.batches == 3 and not st.held
    for i, pr in enumerate(prompts):
        assert res.tokens[i] == _expect(pr, 3)[0]
    firsts = [s for s in st.steps if any(n > 1 for _, n in s) or s == st.steps[0]]
    assert {slot for step in st.steps for slot, _ in step} == {0, 1}                          # the same two slots


def test_limits():
    assert max_new_tokens(10, 1024, 100) == 90 and max_new_tokens(10, 5, 100) == 5
    with pytest.raises(PromptTooLong):
        max_new_tokens(100, 5, 100)
    with pytest.raises(ValueError):
        max_new_tokens(0, 5, 100)
    # the cache holds 4 pages: two requests of 100 + 28 tokens fit (2 pages each), a third starts a new batch
    assert plan_batches([100, 100, 100], [28, 28, 28], ctx=256, max_batch=8) == [[0, 1], [2]]
    assert plan_batches([1] * 5, [1] * 5, ctx=4096, max_batch=2) == [[0, 1], [2, 3], [4]]
    st = FakeStepper(ctx=64)
    with pytest.raises(PromptTooLong):
        generate(st, [[1] * 64], SamplingParams(temperature=0.0))
    res = generate(st, [[1] * 60], SamplingParams(temperature=0.0, max_tokens=1000))
    assert len(res.tokens[0]) == 4 and res.finish == ["length"]                               # ctx - len(prompt)


def test_cancel_and_callback():
    st = FakeStepper()
    seen = []
    n = {"steps": 0}

    def cancel():
        n["steps"] += 1
        return n["steps"] >= 3
    res = generate(st, [[1, 2], [3]], SamplingParams(temperature=0.0, max_tokens=50), on_tokens=seen.append,
                   cancel=cancel)
    assert res.finish == ["stop", "stop"] and all(len(t) == 3 for t in res.tokens) and not st.held
    assert len(seen) == 3 and all(set(d) == {0, 1} for d in seen)


def test_slots_are_freed_when_a_step_fails():
    class Boom(FakeStepper):
        def run(self, *a):
            if len(self.steps) == 2:
                raise RuntimeError("boom")
            return super().run(*a)
    st = Boom()
    with pytest.raises(RuntimeError):
        generate(st, [[1], [2]], SamplingParams(temperature=0.0, max_tokens=9))
    assert not st.held


def test_pack_arithmetic():
    ps = pack([StepEntry(3, (5, 6, 7), (0, 2)), StepEntry(1, (9,), (0,))], length_before=[10, 64])
    seg = lambda n: ps.meta[ps.off[n][0]: ps.off[n][0] + ps.off[n][1]].tolist()         # noqa: E731
    assert seg("tok") == [5, 6, 7, 9] and seg("pos") == [10, 11, 12, 64] and seg("seq") == [0, 0, 0, 1]
    assert seg("slot") == [3, 1] and seg("q_start") == [0, 3, 4] and seg("kv_len") == [13, 65]
    assert seg("rows") == [0, 2, 3] and (ps.T, ps.B, ps.R) == (4, 2, 3) and not ps.decode and ps.max_kv == 65
    assert pack([StepEntry(0, (1,), (0,)), StepEntry(2, (1,), (0,))], [5, 6]).decode
    # one token each (the quick way through pack): the same segments, some sequences without a wanted place
    ps = pack([StepEntry(4, (11,), (0,)), StepEntry(0, (12,), ()), StepEntry(9, (13,), (0,))], [7, 0, 200])
    seg = lambda n: ps.meta[ps.off[n][0]: ps.off[n][0] + ps.off[n][1]].tolist()         # noqa: E731
    assert seg("tok") == [11, 12, 13] and seg("pos") == [7, 0, 200] and seg("seq") == [0, 1, 2]
    assert seg("slot") == [4, 0, 9] and seg("q_start") == [0, 1, 2, 3] and seg("kv_len") == [8, 1, 201]
    assert seg("rows") == [0, 2] and (ps.T, ps.B, ps.R) == (3, 3, 2) and ps.decode and ps.max_kv == 201
    assert ps.h_kv_len == (8, 1, 201) and ps.h_q_start == (0, 1, 2, 3) and ps.meta.dtype.name == "int32"
    assert layout(4, 2, 3) == layout(4, 2, 3) and all(a % 4 == 0 for a, _ in layout(5, 3, 2)[0].values())
    for bad in ([StepEntry(0, (), ())], [StepEntry(0, (1,), (1,))], [StepEntry(0, (1,)), StepEntry(0, (2,))], []):
        with pytest.raises(ValueError):
            pack(bad, [0] * len(bad))


def test_split_step_keeps_every_token_and_place():
    entries = [StepEntry(0, tuple(range(10)), (0, 9)), StepEntry(1, (7,), (0,)), StepEntry(2, tuple(range(100, 125)), (3, 24)),
               StepEntry(3, (1, 2), ())]
    for chunk in (4, 8, 11, 25, 64):
        subs = split_step(entries, chunk)
        assert all(sum(len(e.tokens) for _, e in sub) <= chunk for sub in subs)
        assert all(len({e.slot for _, e in sub}) == len(sub) for sub in subs)           # a slot once per sub-step
        seen = {i: [] for i in range(len(entries))}
        places = {i: [] for i in range(len(entries))}
        for sub in subs:
            for i, e in sub:
                places[i] += [len(seen[i]) + w for w in e.want]
                seen[i] += list(e.tokens)
        for i, e in enumerate(entries):
            assert tuple(seen[i]) == e.tokens and tuple(places[i]) == e.want
    assert len(split_step(entries, 64)) == 1


class OverlapStepper(FakeStepper):
    """a stepper that splits a step: ``launch`` computes at once what the device would (its picks are kept "on the
    device" for a following step that asks for them) and ``collect`` hands the tokens over; it checks that no step is
    ever issued on tokens of the host that the host has not collected yet, and that at most two steps are under way"""

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.last_picks = None
        self.in_flight = 0
        self.ahead = 0

    def launch(self, entries, params, seq_ids, histories, tokens_from_previous=False):
        assert histories is None and self.in_flight <= 1
        assert len({e.slot for e in entries}) == len(entries) and all(e.slot in self.held for e in entries)
        if tokens_from_previous:
            assert self.last_picks is not None and len(self.last_picks) == len(entries)
            assert all(len(e.tokens) == 1 for e in entries)
            toks = [(t,) for t in self.last_picks]
            self.ahead += 1
        else:
            assert self.in_flight == 0               # tokens from the host: everything before has been collected
            toks = [e.tokens for e in entries]
        self.steps.append([(e.slot, len(t)) for e, t in zip(entries, toks)])
        out = []
        for e, t in zip(entries, toks):
            self.sums[e.slot] += sum(t)
            out.append(self.sums[e.slot] % 97)
        self.last_picks = out
        self.in_flight += 1
        return list(out)

    def collect(self, handle):
        self.in_flight -= 1
        return handle


@pytest.mark.parametrize("max_tokens,stops", [(12, (31, 4)), (3, ()), (1, ()), (40, (5, 11, 60, 77))])
def test_overlapped_loop_gives_the_same_tokens(max_tokens, stops):
    prompts = [[1, 2, 3], [50], [7] * 20, [9, 9], [13, 1], [2] * 9]
    p = SamplingParams(temperature=0.0, max_tokens=max_tokens, stop_token_ids=stops)
    plain = generate(FakeStepper(max_batch=4, n_slots=4), prompts, p)
    st = OverlapStepper(max_batch=4, n_slots=4)
    seen = []
    res = generate(st, prompts, p, on_tokens=lambda d: seen.append(dict(d)))
    assert res.tokens == plain.tokens and res.finish == plain.finish
    for i, pr in enumerate(prompts):
        assert res.tokens[i] == _expect(pr, max_tokens, stop=stops)[0]
    assert not st.held and st.in_flight == 0
    assert sum(len(d) for d in seen) == sum(len(t) for t in res.tokens)
    if max_tokens > 3:
        assert st.ahead > 0                          # steps were issued ahead of the read


def test_overlap_is_off_when_the_pick_needs_the_history():
    st = OverlapStepper()
    p = SamplingParams(temperature=0.0, max_tokens=4, repeat_penalty=1.2)
    res = generate(st, [[1, 2, 3]], p)
    assert st.ahead == 0 and res.tokens[0] == _expect([1, 2, 3], 4)[0]


def test_cancel_with_a_step_under_way():
    st = OverlapStepper()
    calls = []

    def cancel():
        calls.append(1)
        return len(calls) >= 3
    res = generate(st, [[1, 2, 3], [4]], SamplingParams(temperature=0.0, max_tokens=50), cancel=cancel)
    assert res.finish == ["stop", "stop"] and len(res.tokens[0]) == 3 and not st.held and st.in_flight == 0


def test_pack_with_padding_rows():
    """a recorded prompt step is padded to a fixed number of rows: the padding rows carry token 0 and position -1, lie
    behind every sequence's row range, and the sequences' own numbers are what they are without padding"""
    entries = [StepEntry(3, (5, 6, 7), (2,)), StepEntry(1, (9,) * 10, (9,))]
    plain = pack(entries, [4, 0])
    padded = pack(entries, [4, 0], pad_rows_to=64)
    assert (plain.T, padded.T, padded.B, padded.R) == (13, 64, 2, 2) and not padded.decode
    seg = lambda ps, n: ps.meta[ps.off[n][0]: ps.off[n][0] + ps.off[n][1]].tolist()
    assert seg(padded, "tok")[:13] == seg(plain, "tok") and set(seg(padded, "tok")[13:]) == {0}
    assert seg(padded, "pos")[:13] == [4, 5, 6] + list(range(10)) and set(seg(padded, "pos")[13:]) == {-1}
    assert set(seg(padded, "seq")[13:]) == {0}
    for name in ("slot", "q_start", "kv_len", "rows"):
        assert seg(padded, name) == seg(plain, name)
    assert padded.h_kv_len == plain.h_kv_len == (7, 10) and padded.max_q == 10
    assert pack(entries, [4, 0], pad_rows_to=8).T == 13            # never fewer rows than tokens
