"""Each part alone against its plain function; and that parts defined outside the package (a mixer with state of its
own, a feed-forward with routing, another position encoding), a layer that runs twice and a layer that reads another
layer's keys and values can be registered, built and stepped without a change to the package."""
import math

import numpy as np
import pytest
import torch

import plain_model as P
import tiny

pytestmark = pytest.mark.gpu


def _engine(tmp_path, name, dtype, **kw):
    from kindi_b200.engine.engine import Engine
    return Engine(tiny.make_model(tmp_path, name, dtype), ctx=1024, dtype=dtype, max_batch=4, **kw)


def _ctx(eng, seqs):
    """a step context for whole sequences of the given lengths that start now"""
    from kindi_b200.engine.batch import StepEntry, pack
    entries = [StepEntry(eng.alloc(), tuple(range(n)), ()) for n in seqs]
    ps = pack(entries, [0] * len(entries))
    for e, n in zip(entries, ps.h_kv_len):
        eng.cache.reserve(e.slot, n)
    eng.cache.flush()
    ctx = eng._context(ps)
    ctx.entry = eng.spec.schedule[0]
    return ctx


def _rel(a, b):
    return float((a.double().cpu() - b.double()).abs().max() / (b.double().abs().max() + 1e-30))


TOL = {"float32": 3e-6, "bfloat16": 1.2e-2}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C", "E"])
def test_norm_mixer_feed_forward_block_alone(tmp_path, name, dtype):
    from kindi_b200.parts.base import Branch
    eng = _engine(tmp_path, name, dtype)
    m = P.load_model(tiny.make_model(tmp_path, name, dtype))
    seqs = [70, 1, 9]
    T, E = sum(seqs), eng.spec.width
    ctx = _ctx(eng, seqs)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(T, E, generator=g)
    planes = torch.randn(3, T, E, generator=g) * 0.1
    blk = eng.model.blocks[0]
    w = m["w"]
    # ---- norm, with three pending planes, all rows and then a subset of rows
    xd = x.cuda().clone()
    y = blk.norm1.add_norm(ctx, xd, Branch(planes.cuda()))
    xs = x.double() + planes.double().sum(0)
    want = P.rms_norm(xs, w["model.layers.0.input_layernorm.weight"], m["eps"])
    assert _rel(xd, xs) < 1e-6 and _rel(y.float(), want) < (1e-6 if dtype == "float32" else 6e-3)
    rows = torch.tensor([5, 70, 79, 0], dtype=torch.int32).cuda()
    y2 = blk.norm1.add_norm(ctx, xd, None, rows=rows)
    assert torch.equal(y2, y[rows.long()])
    # ---- mixer alone: whole sequences, so the plain attention of each sequence is the reference
    yin = (torch.randn(T, E, generator=g) * 0.5).to(eng.dtype)
    br = blk.mixer.forward(ctx, yin.cuda())
    got = br.parts.sum(0)
    H, KV, d = m["heads"], m["kv_heads"], m["head_dim"]
    at = 0
    for n in seqs:
        yy = yin[at:at + n].double()
        cos, sin = P.rope_tables(torch.arange(n), d, m["theta"], torch.float64)
        q = P.rope_rotate_half((yy @ w["model.layers.0.self_attn.q_proj.weight"].T).view(n, H, d), cos, sin)
        k = P.rope_rotate_half((yy @ w["model.layers.0.self_attn.k_proj.weight"].T).view(n, KV, d), cos, sin)
        v = (yy @ w["model.layers.0.self_attn.v_proj.weight"].T).view(n, KV, d)
        window = m["window"] if (m["window"] and (m["layer_types"] is None or m["layer_types"][0] == "sliding_attention")) else None
        a = P.attention(q, k, v, 1 / math.sqrt(d), window).reshape(n, H * d)
        assert _rel(got[at:at + n], a @ w["model.layers.0.self_attn.o_proj.weight"].T) < TOL[dtype]
        at += n
    # ---- feed-forward alone
    br = blk.feed_forward.forward(ctx, yin.cuda())
    want = P.swiglu_mlp(yin.double(), w["model.layers.0.mlp.gate_proj.weight"], w["model.layers.0.mlp.up_proj.weight"],
                        w["model.layers.0.mlp.down_proj.weight"])
    assert _rel(br.parts.sum(0), want) < TOL[dtype]
    # ---- the whole block: residual in, residual + pending out
    for s in list(ctx.h_slot):
        eng.free(s)
    ctx = _ctx(eng, seqs)
    xd = x.cuda().clone()
    pend = blk.forward(ctx, xd, None)
    got = xd + pend.parts.sum(0)
    at = 0
    for n in seqs:
        cos, sin = P.rope_tables(torch.arange(n), d, m["theta"], torch.float64)
        assert _rel(got[at:at + n], P.decoder_layer(m, 0, x[at:at + n].double(), cos, sin)) < TOL[dtype]
        at += n
    eng.check_status()


def test_embedding_and_position_encoding_alone(tmp_path):
    from kindi_b200.kernels import lib as K
    from kindi_b200.parts.rope import Rotary
    from kindi_b200.config.spec import PartSpec
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    table = torch.randn(37, 24).to(torch.bfloat16).cuda()
    tok = torch.tensor([0, 36, 5, 5], dtype=torch.int32).cuda()
    out = torch.empty(4, 24, device="cuda")
    K.embed(table, tok, out, st)
    assert torch.equal(out, table.float()[tok.long()]) and int(st.item()) == 0
    K.embed(table, torch.tensor([37, -1, 3, 0], dtype=torch.int32).cuda(), out, st)
    assert int(st.item()) == K.ST_BAD_TOKEN and float(out[:2].abs().sum()) == 0.0    # skipped, reported, no fault
    # rotary: the table of the part and the rotation of the kernel against the plain functions, partial rotation too
    for hd, rot, base in [(16, 16, 10000.0), (48, 32, 500000.0), (128, 128, 7e7)]:
        rp = Rotary(PartSpec("rotary", {"base": base, "rotary_dim": rot}), 0, None, dtype=torch.float32, device="cuda")
        i = torch.arange(rot // 2, dtype=torch.float64)
        assert torch.equal(rp.inv_freq.cpu(), (base ** (-2 * i / rot)).float())
        pos = torch.tensor([0, 1, 77, 8191, 40000], dtype=torch.int32)
        x = torch.randn(5, 3 * hd)
        xd = x.cuda().clone()
        seq = torch.zeros(5, dtype=torch.int32).cuda()
        table_ = torch.zeros(1, 1, dtype=torch.int32).cuda()
        st.zero_()
        K.rope_store(xd, xd, rp.inv_freq, rot, pos.cuda(), seq, seq[:1], 3, 0, hd, None, table_, 1, st)
        cos, sin = P.rope_tables(pos, rot, base, torch.float64)
        want = P.rope_rotate_half(x.double().view(5, 3, hd), cos, sin).reshape(5, 3 * hd)
        assert _rel(xd, want) < 1e-6


# ------------------------------------------------------------------------------------------------------------------
# a mixer defined here, not in the package: y_t = W * mean(x_0 .. x_t). Its state per sequence is the running sum and
# the count; it is written in plain PyTorch and uses the step's host-side numbers, so it declares graph_safe = False.
def _toy_parts():
    from kindi_b200.config.registry import register_part
    from kindi_b200.parts.base import Branch, Mixer, StateNeed

    class RunningMean(Mixer):
        graph_safe = False

        @classmethod
        def tensor_shapes(cls, spec, width):
            return {"mix.weight": (width, width)}

        @classmethod
        def cache_need(cls, spec, width):
            return StateNeed((width + 1,))

        def __init__(self, spec, width, weights, *, dtype, device):
            super().__init__(spec, width, weights, dtype=dtype, device=device)
            self.w = weights("mix.weight").float()

        def forward(self, ctx, y):
            state = ctx.cache.state_view(ctx.entry.cache)
            out = torch.empty((1, ctx.T, self.width), dtype=torch.float32, device=y.device)
            for b, slot in enumerate(ctx.h_slot):
                a, e = ctx.h_q_start[b], ctx.h_q_start[b + 1]
                run = state[slot, :-1] + torch.cumsum(y[a:e].float(), dim=0)
                cnt = state[slot, -1] + torch.arange(1, e - a + 1, device=y.device, dtype=torch.float32)
                out[0, a:e] = (run / cnt[:, None]) @ self.w.T
                state[slot, :-1] = run[-1]
                state[slot, -1] = cnt[-1]
            return Branch(out)

    register_part("mixer", "toy_running_mean", RunningMean, replace=True)


def _toy_spec(width=64, vocab=97):
    from kindi_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    norm = PartSpec("rmsnorm", {"eps": 1e-5})
    ffn = PartSpec("swiglu", {"intermediate": 96})
    att = PartSpec("attention", {"n_heads": 4, "n_kv_heads": 2, "head_dim": 16, "window": None,
                                 "position": PartSpec("rotary", {"base": 10000.0, "rotary_dim": 16})})
    toy = PartSpec("toy_running_mean", {})
    layers = (LayerSpec(PartSpec("prenorm", {"norm1": norm, "mixer": att, "norm2": norm, "feed_forward": ffn}), "l0."),
              LayerSpec(PartSpec("prenorm", {"norm1": norm, "mixer": toy, "norm2": norm, "feed_forward": ffn}), "l1."),
              LayerSpec(PartSpec("prenorm", {"norm1": norm, "mixer": att, "norm2": norm, "feed_forward": ffn}), "l2."))
    # layer 0 runs twice (its second run owns cache entry 2); layer 2 reads the keys and values of the first run
    schedule = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2), ScheduleEntry(2, 3, reads_cache_of=0))
    spec = ModelSpec(architecture="toy", vocab_size=vocab, width=width, layers=layers, schedule=schedule,
                     final_norm=norm, final_norm_prefix="fn.",
                     embedding=PartSpec("table", {"name": "emb", "vocab": vocab}),
                     head=PartSpec("linear", {"name": "head", "tied_to": "emb", "vocab": vocab}))
    spec.validate()
    return spec


def _toy_plain(spec, w, tokens):
    """the toy model on one whole sequence, in float64, from the plain part functions"""
    w = {k: v.double().cpu() for k, v in w.items()}
    n = len(tokens)
    x = P.embedding(w["emb"], tokens)
    cos, sin = P.rope_tables(torch.arange(n), 16, 10000.0, torch.float64)
    kv = {}
    for e in spec.schedule:
        p = spec.layers[e.layer].prefix
        y = P.rms_norm(x, w[p + "input_layernorm.weight"], 1e-5)
        if spec.layers[e.layer].block["mixer"].kind == "attention":
            q = P.rope_rotate_half((y @ w[p + "self_attn.q_proj.weight"].T).view(n, 4, 16), cos, sin)
            if e.reads_cache_of is None:
                k = P.rope_rotate_half((y @ w[p + "self_attn.k_proj.weight"].T).view(n, 2, 16), cos, sin)
                kv[e.cache] = (k, (y @ w[p + "self_attn.v_proj.weight"].T).view(n, 2, 16))
            k, v = kv[e.cache if e.reads_cache_of is None else e.reads_cache_of]
            a = P.attention(q, k, v, 0.25).reshape(n, 64) @ w[p + "self_attn.o_proj.weight"].T
        else:
            mean = torch.cumsum(y, 0) / torch.arange(1, n + 1, dtype=torch.float64)[:, None]
            a = mean @ w[p + "self_attn.mix.weight"].T
        x = x + a
        y = P.rms_norm(x, w[p + "post_attention_layernorm.weight"], 1e-5)
        x = x + P.swiglu_mlp(y, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return P.rms_norm(x, w["fn.weight"], 1e-5) @ w["emb"].T


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 1.5e-2)])
def test_toy_mixer_with_state_repeated_layer_and_shared_cache(tmp_path, dtype, tol):
    from kindi_b200.engine.engine import Engine
    from kindi_b200.parts.model import cache_needs, expected_tensors, tensor_inits
    from kindi_b200.weights.random_init import random_tensors
    _toy_parts()
    spec = _toy_spec()
    shapes = expected_tensors(spec)
    assert "l1.self_attn.mix.weight" in shapes and "l2.self_attn.k_proj.weight" in shapes
    needs = cache_needs(spec)
    assert [type(n).__name__ for n in needs] == ["KVNeed", "StateNeed", "KVNeed", "NoneType"]
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    w = random_tensors(shapes, seed=9, std=0.05, dtype=tdt, inits=tensor_inits(spec))
    eng = Engine(spec=spec, tensors=w, ctx=1024, dtype=dtype, max_batch=3)
    assert not eng.cuda_graphs                                   # the toy mixer is not graph-safe
    reqs = tiny.random_requests(97, [40, 7, 90, 3, 66], seed=4)
    want = {r: _toy_plain(spec, w, t).numpy() for r, t in reqs.items()}
    for steps in (tiny.trace_whole(reqs), tiny.trace_last_n(reqs, 32), tiny.trace_batched(reqs, batch=3, decode=10)):
        out = str(tmp_path / ("o%d" % len(steps)))
        tiny.run_replay(eng, steps, out)
        got = tiny.collect(out, steps, 97)
        for r, t in reqs.items():
            mine = np.stack([got[(r, i)] for i in range(len(t))])
            assert tiny.rel_err(mine, want[r]) < tol, (len(steps), r)
        eng.cache.check()
        assert eng.cache.slots.n_held == 0


# ------------------------------------------------------------------------------------------------------------------
# a feed-forward with routing and another position encoding, both defined here. The feed-forward sends each row to
# the one expert whose router logit (32-bit) is largest (ties: the lowest index) and returns relu(W1_e y) W2_e; it is
# written with device-side PyTorch only and uses no host numbers, so the decode steps of a model that holds it are
# still recorded. The position encoding rotates the first half of each head with frequencies 0.3 / (i + 1).
def _toy_routed_parts():
    from kindi_b200.config.registry import register_part
    from kindi_b200.parts import Branch, FeedForward, RotationEncoding

    class TopOneExperts(FeedForward):
        @classmethod
        def tensor_shapes(cls, spec, width):
            n, f = int(spec["experts"]), int(spec["intermediate"])
            out = {"router.weight": (n, width)}
            for e in range(n):
                out["experts.%d.w1.weight" % e] = (f, width)
                out["experts.%d.w2.weight" % e] = (width, f)
            return out

        def __init__(self, spec, width, weights, *, dtype, device):
            super().__init__(spec, width, weights, dtype=dtype, device=device)
            n = int(spec["experts"])
            self.router = weights("router.weight").float()
            self.w1 = torch.stack([weights("experts.%d.w1.weight" % e).float() for e in range(n)])
            self.w2 = torch.stack([weights("experts.%d.w2.weight" % e).float() for e in range(n)])

        def forward(self, ctx, y):
            yf = y.float()
            pick = torch.argmax(yf @ self.router.T, dim=1)                    # ties: the first (lowest) index
            h = torch.relu(torch.bmm(self.w1[pick], yf[:, :, None]))
            return Branch(torch.bmm(self.w2[pick], h)[None, :, :, 0].contiguous())

    class HarmonicRotation(RotationEncoding):
        def __init__(self, spec, width, weights, *, dtype, device):
            super().__init__(spec, width, weights, dtype=dtype, device=device)
            self.rotary_dim = int(spec["rotary_dim"])
            self.inv_freq = (0.3 / torch.arange(1, self.rotary_dim // 2 + 1, dtype=torch.float64)).float().to(device)

    register_part("feed_forward", "toy_top1_experts", TopOneExperts, replace=True)
    register_part("position", "toy_harmonic", HarmonicRotation, replace=True)


def _toy_routed_spec(width=64, vocab=101):
    from kindi_b200.config.spec import LayerSpec, ModelSpec, PartSpec, default_schedule
    norm = PartSpec("rmsnorm", {"eps": 2e-6})
    swiglu = PartSpec("swiglu", {"intermediate": 128})
    routed = PartSpec("toy_top1_experts", {"experts": 3, "intermediate": 40})
    att_h = PartSpec("attention", {"n_heads": 4, "n_kv_heads": 1, "head_dim": 16, "window": None,
                                   "position": PartSpec("toy_harmonic", {"rotary_dim": 8})})
    att_r = PartSpec("attention", {"n_heads": 4, "n_kv_heads": 1, "head_dim": 16, "window": None,
                                   "position": PartSpec("rotary", {"base": 10000.0, "rotary_dim": 16})})
    layers = (LayerSpec(PartSpec("prenorm", {"norm1": norm, "mixer": att_h, "norm2": norm, "feed_forward": routed}), "a."),
              LayerSpec(PartSpec("prenorm", {"norm1": norm, "mixer": att_r, "norm2": norm, "feed_forward": swiglu}), "b."))
    spec = ModelSpec(architecture="toy_routed", vocab_size=vocab, width=width, layers=layers,
                     schedule=default_schedule(2), final_norm=norm, final_norm_prefix="fn.",
                     embedding=PartSpec("table", {"name": "emb", "vocab": vocab}),
                     head=PartSpec("linear", {"name": "head", "vocab": vocab}))
    spec.validate()
    return spec


def _toy_routed_plain(w, tokens, run_dtype):
    """whole sequence, float64; the router sees the normalised row as the engine hands it over (rounded to the run
    dtype), so that both pick the same expert"""
    w = {k: v.double().cpu() for k, v in w.items()}
    n = len(tokens)
    x = P.embedding(w["emb"], tokens)
    pos = torch.arange(n, dtype=torch.float32)
    inv_h = (0.3 / torch.arange(1, 5, dtype=torch.float64)).float()
    ang = (pos[:, None] * inv_h[None, :]).double()
    tables = {"a.": (torch.cos(ang), torch.sin(ang)), "b.": P.rope_tables(torch.arange(n), 16, 10000.0, torch.float64)}
    for p in ("a.", "b."):
        cos, sin = tables[p]
        y = P.rms_norm(x, w[p + "input_layernorm.weight"], 2e-6)
        q = P.rope_rotate_half((y @ w[p + "self_attn.q_proj.weight"].T).view(n, 4, 16), cos, sin)
        k = P.rope_rotate_half((y @ w[p + "self_attn.k_proj.weight"].T).view(n, 1, 16), cos, sin)
        v = (y @ w[p + "self_attn.v_proj.weight"].T).view(n, 1, 16)
        x = x + P.attention(q, k, v, 0.25).reshape(n, 64) @ w[p + "self_attn.o_proj.weight"].T
        y = P.rms_norm(x, w[p + "post_attention_layernorm.weight"], 2e-6)
        if p == "a.":
            yr = y.to(run_dtype).double()
            pick = torch.argmax((yr.float() @ w["a.mlp.router.weight"].float().T), dim=1)
            out = torch.empty_like(x)
            for t in range(n):
                e = int(pick[t])
                out[t] = w["a.mlp.experts.%d.w2.weight" % e] @ torch.relu(w["a.mlp.experts.%d.w1.weight" % e] @ yr[t])
            x = x + out
        else:
            x = x + P.swiglu_mlp(y, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return P.rms_norm(x, w["fn.weight"], 2e-6) @ w["head"].T


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 1.5e-2)])
def test_toy_routed_feed_forward_and_another_position_encoding(tmp_path, dtype, tol):
    from kindi_b200.engine.engine import Engine
    from kindi_b200.parts.model import expected_tensors, tensor_inits
    from kindi_b200.weights.random_init import random_tensors
    _toy_routed_parts()
    spec = _toy_routed_spec()
    shapes = expected_tensors(spec)
    assert shapes["a.mlp.router.weight"] == (3, 64) and shapes["a.mlp.experts.2.w2.weight"] == (64, 40)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    w = random_tensors(shapes, seed=13, std=0.05, dtype=tdt, inits=tensor_inits(spec))
    # routing with wide margins, so that rounding cannot change an expert: token t carries a large value in feature
    # t % 3 and the router reads exactly these three features (all three experts are used by every request)
    w["emb"][:, :3] = 0
    w["emb"][torch.arange(101), torch.arange(101) % 3] = 4.0
    w["a.mlp.router.weight"].zero_()
    w["a.mlp.router.weight"][torch.arange(3), torch.arange(3)] = 8.0
    eng = Engine(spec=spec, tensors=w, ctx=1024, dtype=dtype, max_batch=3)
    reqs = tiny.random_requests(101, [50, 9, 77, 2], seed=6)
    want = {r: _toy_routed_plain(w, t, tdt).numpy() for r, t in reqs.items()}
    for steps in (tiny.trace_whole(reqs), tiny.trace_last_n(reqs, 32), tiny.trace_batched(reqs, batch=3, decode=10)):
        out = str(tmp_path / ("r%d" % len(steps)))
        tiny.run_replay(eng, steps, out)
        got = tiny.collect(out, steps, 101)
        for r, t in reqs.items():
            mine = np.stack([got[(r, i)] for i in range(len(t))])
            assert tiny.rel_err(mine, want[r]) < tol, (len(steps), r)
        eng.cache.check()
        assert eng.cache.slots.n_held == 0
    if eng.cuda_graphs:
        assert eng.graph_replays > 0                  # its decode steps were recorded and replayed


# ------------------------------------------------------------------------------------------------------------------
# a whole toy ARCHITECTURE defined here and loaded from a model folder: config.json keys of its own (no attention
# heads, a GELU feed-forward, an embedding scale, a logit scale and soft cap), registered with the package's registry;
# the folder is written by the random-weights mode and read back by the engine like any other.
def _toy_architecture():
    from kindi_b200.config import (ConfigError, ConfigReader, LayerSpec, ModelSpec, PartSpec, default_schedule,
                                   register_architecture, register_part)
    from kindi_b200.parts.base import Branch, FeedForward
    _toy_parts()                                                     # the running-mean mixer with state

    class GeluMLP(FeedForward):
        """gelu(W1 y + b1) W2, the tanh form, written with device-side PyTorch only (no host numbers)"""

        @classmethod
        def tensor_shapes(cls, spec, width):
            f = int(spec["inner"])
            return {"fc.weight": (f, width), "fc.bias": (f,), "proj.weight": (width, f)}

        @classmethod
        def tensor_init(cls, spec, width):
            return {"fc.bias": "zero"}

        def __init__(self, spec, width, weights, *, dtype, device):
            super().__init__(spec, width, weights, dtype=dtype, device=device)
            self.w1, self.b1, self.w2 = (weights(n).float() for n in ("fc.weight", "fc.bias", "proj.weight"))

        def forward(self, ctx, y):
            h = torch.nn.functional.gelu(y.float() @ self.w1.T + self.b1, approximate="tanh")
            return Branch((h @ self.w2.T)[None].contiguous())

    def read(raw):
        r = ConfigReader(raw)
        r.ignore("architectures", "model_type")
        if r.string("hidden_act") != "gelu_tanh":
            raise ConfigError("config.json: the toy architecture has a tanh-GELU feed-forward only")
        c = dict(width=r.integer("d_model"), layers=r.integer("n_layer"), vocab=r.integer("vocab_size"),
                 inner=r.integer("d_inner"), eps=r.number("layer_norm_epsilon"), emb_scale=r.number("emb_scale", 1.0),
                 logit_scale=r.number("logit_scale", 1.0), softcap=r.number("logit_softcap", None))
        r.finish()
        return c

    def build(c):
        norm = PartSpec("rmsnorm", {"eps": c["eps"]})
        block = PartSpec("prenorm", {"norm1": norm, "mixer": PartSpec("toy_running_mean", {}), "norm2": norm,
                                     "feed_forward": PartSpec("toy_gelu", {"inner": c["inner"]}),
                                     "names": {"norm1": "ln_1.", "mixer": "mix.", "norm2": "ln_2.", "feed_forward": "mlp."}})
        return ModelSpec(architecture="ToyMeanGeluLM", vocab_size=c["vocab"], width=c["width"],
                         layers=tuple(LayerSpec(block, "h.%d." % i) for i in range(c["layers"])),
                         schedule=default_schedule(c["layers"]), final_norm=norm, final_norm_prefix="ln_f.",
                         embedding=PartSpec("table", {"name": "wte.weight", "vocab": c["vocab"], "scale": c["emb_scale"]}),
                         head=PartSpec("linear", {"name": "head.weight", "vocab": c["vocab"], "scale": c["logit_scale"],
                                                  "softcap": c["softcap"]}))

    register_part("feed_forward", "toy_gelu", GeluMLP, replace=True)
    register_architecture("ToyMeanGeluLM", build, read, replace=True)


TOY_CONFIG = dict(architectures=["ToyMeanGeluLM"], hidden_act="gelu_tanh", d_model=48, n_layer=3, vocab_size=131,
                  d_inner=80, layer_norm_epsilon=1e-5, emb_scale=6.0, logit_scale=0.5, logit_softcap=4.0)


def _toy_architecture_plain(folder, tokens):
    """whole sequence, float64, from the folder's files alone"""
    from safetensors.torch import load_file
    w = {k: v.double() for k, v in load_file(folder + "/model.safetensors").items()}
    c = TOY_CONFIG
    n = len(tokens)
    x = P.embedding(w["wte.weight"], tokens) * c["emb_scale"]
    for i in range(c["n_layer"]):
        p = "h.%d." % i
        y = P.rms_norm(x, w[p + "ln_1.weight"], c["layer_norm_epsilon"])
        mean = torch.cumsum(y, 0) / torch.arange(1, n + 1, dtype=torch.float64)[:, None]
        x = x + mean @ w[p + "mix.mix.weight"].T
        y = P.rms_norm(x, w[p + "ln_2.weight"], c["layer_norm_epsilon"])
        h = torch.nn.functional.gelu(y @ w[p + "mlp.fc.weight"].T + w[p + "mlp.fc.bias"], approximate="tanh")
        x = x + h @ w[p + "mlp.proj.weight"].T
    z = (P.rms_norm(x, w["ln_f.weight"], c["layer_norm_epsilon"]) @ w["head.weight"].T) * c["logit_scale"]
    return c["logit_softcap"] * torch.tanh(z / c["logit_softcap"])


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 1.5e-2)])
def test_toy_architecture_from_a_model_folder(tmp_path, dtype, tol):
    """another architecture is a registry entry: its folder (own config.json keys, own tensor names, a mixer with
    state and no attention at all) is written by the random-weights mode, loaded by the engine, replayed whole, token
    by token and in unequal batches, and generates; nothing of the package knows it"""
    from kindi_b200 import Engine, write_random_model
    from kindi_b200.config import ConfigError, model_from_dir
    _toy_architecture()
    folder = write_random_model(str(tmp_path / "toy"), TOY_CONFIG, seed=3, std=0.05, dtype=dtype)
    cfg, spec = model_from_dir(folder)
    assert cfg["width"] == 48 and spec.architecture == "ToyMeanGeluLM" and spec.head["softcap"] == 4.0
    eng = Engine(folder, ctx=1024, dtype=dtype, max_batch=3)
    assert not eng.cuda_graphs                                   # the running-mean mixer reads host numbers
    reqs = tiny.random_requests(131, [40, 7, 90, 3, 66], seed=4)
    want = {r: _toy_architecture_plain(folder, t).numpy() for r, t in reqs.items()}
    assert max(np.abs(v).max() for v in want.values()) < 4.0     # the soft cap is at work
    for steps in (tiny.trace_whole(reqs), tiny.trace_last_n(reqs, 32), tiny.trace_batched(reqs, batch=3, decode=10)):
        out = str(tmp_path / ("a%d" % len(steps)))
        tiny.run_replay(eng, steps, out)
        got = tiny.collect(out, steps, 131)
        for r, t in reqs.items():
            mine = np.stack([got[(r, i)] for i in range(len(t))])
            assert tiny.rel_err(mine, want[r]) < tol, (len(steps), r, tiny.rel_err(mine, want[r]))
        eng.cache.check()
    res = eng.generate_batch([reqs["r0"][:9], reqs["r2"][:30]], temperature=0.0, max_tokens=5, stop_token_ids=())
    for prompt, toks in zip((reqs["r0"][:9], reqs["r2"][:30]), res.tokens):
        seq = list(prompt)
        for t in toks:
            z = _toy_architecture_plain(folder, seq)[-1].numpy()
            assert t == int(z.argmax()) or z.max() - z[t] < tol * np.abs(z).max()
            seq.append(t)
    # a key of another architecture in this folder's config.json is refused by this architecture's reader
    import json
    bad = dict(TOY_CONFIG, num_attention_heads=4)
    (tmp_path / "bad").mkdir()
    (tmp_path / "bad" / "config.json").write_text(json.dumps(bad))
    with pytest.raises(ConfigError):
        model_from_dir(str(tmp_path / "bad"))


# ------------------------------------------------------------------------------------------------------------------
# another norm and another block arrangement, defined here: a LayerNorm with bias (mean removed, gain and bias) and a
# block that runs mixer and feed-forward side by side on ONE normalised input (x += mixer(n(x)) + feed_forward(n(x))),
# around the package's own attention and SwiGLU parts.
def _toy_norm_and_block():
    from kindi_b200.config.registry import part_class, register_part
    from kindi_b200.parts.base import Block, Branch, Norm

    class BiasLayerNorm(Norm):
        @classmethod
        def tensor_shapes(cls, spec, width):
            return {"weight": (width,), "bias": (width,)}

        @classmethod
        def tensor_init(cls, spec, width):
            return {"weight": "gain", "bias": "zero"}

        def __init__(self, spec, width, weights, *, dtype, device):
            super().__init__(spec, width, weights, dtype=dtype, device=device)
            self.eps = float(spec["eps"])
            self.w, self.b = weights("weight").float(), weights("bias").float()

        def add_norm(self, ctx, x, pending, rows=None):
            if pending is not None:
                v = x + pending.parts.sum(0) if rows is not None else x.add_(pending.parts.sum(0))
            else:
                v = x
            if rows is not None:
                v = v[rows.long()]
            mu = v.mean(-1, keepdim=True)
            var = ((v - mu) ** 2).mean(-1, keepdim=True)
            return (((v - mu) * torch.rsqrt(var + self.eps)) * self.w + self.b).to(self.dtype)

    class ParallelBlock(Block):
        @classmethod
        def _parts(cls, spec):
            return (("norm", "norm", "ln."), ("mixer", "mixer", "attn."), ("feed_forward", "feed_forward", "ff."))

        @classmethod
        def tensor_shapes(cls, spec, width):
            out = {}
            for role, cat, sub in cls._parts(spec):
                for sfx, shape in part_class(cat, spec[role].kind).tensor_shapes(spec[role], width).items():
                    out[sub + sfx] = shape
            return out

        @classmethod
        def tensor_init(cls, spec, width):
            out = {}
            for role, cat, sub in cls._parts(spec):
                for sfx, kind in part_class(cat, spec[role].kind).tensor_init(spec[role], width).items():
                    out[sub + sfx] = kind
            return out

        @classmethod
        def cache_need(cls, spec, width):
            return part_class("mixer", spec["mixer"].kind).cache_need(spec["mixer"], width)

        def __init__(self, spec, width, weights, *, dtype, device):
            super().__init__(spec, width, weights, dtype=dtype, device=device)
            self.norm, self.mixer, self.ff = (
                part_class(cat, spec[role].kind)(spec[role], width, weights.sub(sub), dtype=dtype, device=device)
                for role, cat, sub in self._parts(spec))
            self.graph_safe = all(p.graph_safe for p in (self.norm, self.mixer, self.ff))

        def forward(self, ctx, x, pending):
            y = self.norm.add_norm(ctx, x, pending)
            a, f = self.mixer.forward(ctx, y), self.ff.forward(ctx, y)
            return Branch(torch.cat([a.parts, f.parts], dim=0))          # both branches are added by the next norm

    register_part("norm", "toy_bias_layernorm", BiasLayerNorm, replace=True)
    register_part("block", "toy_parallel", ParallelBlock, replace=True)


def _toy_parallel_spec(width=80, vocab=113):
    from kindi_b200.config.spec import LayerSpec, ModelSpec, PartSpec, default_schedule
    norm = PartSpec("toy_bias_layernorm", {"eps": 1e-5})
    att = PartSpec("attention", {"n_heads": 5, "n_kv_heads": 5, "head_dim": 16, "window": None,
                                 "position": PartSpec("rotary", {"base": 10000.0, "rotary_dim": 16})})
    ffn = PartSpec("swiglu", {"intermediate": 112})
    block = PartSpec("toy_parallel", {"norm": norm, "mixer": att, "feed_forward": ffn})
    return ModelSpec(architecture="toy_parallel", vocab_size=vocab, width=width,
                     layers=tuple(LayerSpec(block, "blk%d." % i) for i in range(2)), schedule=default_schedule(2),
                     final_norm=norm, final_norm_prefix="out_ln.",
                     embedding=PartSpec("table", {"name": "emb", "vocab": vocab}),
                     head=PartSpec("linear", {"name": "head", "tied_to": "emb", "vocab": vocab}))


def _toy_parallel_plain(w, tokens):
    w = {k: v.double().cpu() for k, v in w.items()}
    n = len(tokens)

    def ln(v, p):
        mu = v.mean(-1, keepdim=True)
        return (v - mu) / torch.sqrt(((v - mu) ** 2).mean(-1, keepdim=True) + 1e-5) * w[p + "weight"] + w[p + "bias"]
    x = P.embedding(w["emb"], tokens)
    cos, sin = P.rope_tables(torch.arange(n), 16, 10000.0, torch.float64)
    for i in range(2):
        p = "blk%d." % i
        y = ln(x, p + "ln.")
        q = P.rope_rotate_half((y @ w[p + "attn.q_proj.weight"].T).view(n, 5, 16), cos, sin)
        k = P.rope_rotate_half((y @ w[p + "attn.k_proj.weight"].T).view(n, 5, 16), cos, sin)
        v = (y @ w[p + "attn.v_proj.weight"].T).view(n, 5, 16)
        a = P.attention(q, k, v, 0.25).reshape(n, 80) @ w[p + "attn.o_proj.weight"].T
        f = P.swiglu_mlp(y, w[p + "ff.gate_proj.weight"], w[p + "ff.up_proj.weight"], w[p + "ff.down_proj.weight"])
        x = x + a + f
    return ln(x, "out_ln.") @ w["emb"].T


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 1.5e-2)])
def test_toy_norm_and_parallel_block(tmp_path, dtype, tol):
    """a norm with a bias and a block that runs attention and feed-forward side by side, both defined in this file: the
    engine, the cache (five key/value heads of size 16), the decode recordings and the replay modes take them as
    they are"""
    from kindi_b200.engine.engine import Engine
    from kindi_b200.parts.model import expected_tensors, tensor_inits
    from kindi_b200.weights.random_init import random_tensors
    _toy_norm_and_block()
    spec = _toy_parallel_spec()
    shapes = expected_tensors(spec)
    assert shapes["blk1.ln.bias"] == (80,) and tensor_inits(spec)["blk0.ln.bias"] == "zero"
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    w = random_tensors(shapes, seed=21, std=0.05, dtype=tdt, inits=tensor_inits(spec))
    for n in list(w):
        if n.endswith(".bias"):
            w[n] = (torch.randn(w[n].shape, generator=torch.Generator().manual_seed(len(n))) * 0.1).to(tdt)
    eng = Engine(spec=spec, tensors=w, ctx=1024, dtype=dtype, max_batch=3)
    reqs = tiny.random_requests(113, [50, 9, 77, 2], seed=6)
    want = {r: _toy_parallel_plain(w, t).numpy() for r, t in reqs.items()}
    for steps in (tiny.trace_whole(reqs), tiny.trace_last_n(reqs, 32), tiny.trace_batched(reqs, batch=3, decode=10)):
        out = str(tmp_path / ("p%d" % len(steps)))
        tiny.run_replay(eng, steps, out)
        got = tiny.collect(out, steps, 113)
        for r, t in reqs.items():
            mine = np.stack([got[(r, i)] for i in range(len(t))])
            assert tiny.rel_err(mine, want[r]) < tol, (len(steps), r, tiny.rel_err(mine, want[r]))
        eng.cache.check()
    if eng.cuda_graphs:
        assert eng.graph_replays > 0
