"""The plain implementation itself: properties its parts must have, and its sampler against the reference's own
sampling code (outputs stored under tests/golden)."""
import json
import math
import os

import numpy as np
import torch

import plain_model as P
import tiny


def test_rope_keeps_norms_and_depends_on_distance_only():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(6, 2, 16, generator=g, dtype=torch.float64)
    y = torch.randn(6, 2, 16, generator=g, dtype=torch.float64)
    c0, s0 = P.rope_tables(torch.arange(6), 16, 10000.0, torch.float64)
    c1, s1 = P.rope_tables(torch.arange(6) + 37, 16, 10000.0, torch.float64)
    a0, a1 = P.rope_rotate_half(x, c0, s0), P.rope_rotate_half(x, c1, s1)
    assert torch.allclose(a0.norm(dim=-1), x.norm(dim=-1))
    b0, b1 = P.rope_rotate_half(y, c0, s0), P.rope_rotate_half(y, c1, s1)
    d0 = torch.einsum("thd,shd->hts", a0, b0)
    d1 = torch.einsum("thd,shd->hts", a1, b1)
    assert torch.allclose(d0, d1, atol=1e-5)            # angles are rounded to 32-bit as the reference's are
    assert torch.equal(P.rope_rotate_half(x[:1], c0[:1], s0[:1]), x[:1])      # position 0 rotates nothing


def test_attention_is_causal_grouped_and_windowed():
    g = torch.Generator().manual_seed(1)
    q = torch.randn(9, 4, 8, generator=g, dtype=torch.float64)
    k = torch.randn(9, 2, 8, generator=g, dtype=torch.float64)
    v = torch.randn(9, 2, 8, generator=g, dtype=torch.float64)
    out = P.attention(q, k, v, 0.3)
    k2, v2 = k.clone(), v.clone()
    k2[5:], v2[5:] = 0, 0
    assert torch.allclose(P.attention(q, k2, v2, 0.3)[:5], out[:5])           # later keys never reach earlier rows
    full = P.attention(q, k.repeat_interleave(2, dim=1), v.repeat_interleave(2, dim=1), 0.3)
    assert torch.allclose(full, out)                                          # head h reads kv head h // G
    assert torch.allclose(out[0], v[0].repeat_interleave(2, dim=0))           # the first row sees only itself
    w = P.attention(q, k, v, 0.3, window=3)
    assert torch.allclose(w[:3], out[:3]) and not torch.allclose(w[8], out[8])
    assert torch.allclose(w[8], P.attention(q[6:], k[6:], v[6:], 0.3)[2])     # row 8 reads 6, 7, 8 only


def test_norm_and_mlp_formulas():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    y = P.rms_norm(x, w, 0.0)
    assert torch.allclose(y, torch.tensor([[3.0 / math.sqrt(12.5) * 2, 4.0 / math.sqrt(12.5) * 0.5]], dtype=torch.float64))
    g = torch.Generator().manual_seed(2)
    a = torch.randn(3, 4, generator=g, dtype=torch.float64)
    wg, wu, wd = (torch.randn(5, 4, generator=g, dtype=torch.float64), torch.randn(5, 4, generator=g, dtype=torch.float64),
                  torch.randn(4, 5, generator=g, dtype=torch.float64))
    want = (torch.nn.functional.silu(a @ wg.T) * (a @ wu.T)) @ wd.T
    assert torch.allclose(P.swiglu_mlp(a, wg, wu, wd), want)


def test_whole_model_prefix_property(tmp_path):
    d = tiny.make_model(tmp_path, "C")
    m = P.load_model(d)
    toks = list(range(3, 60))
    full = P.forward(m, toks)
    assert full.shape == (57, 331)
    assert torch.allclose(P.forward(m, toks[:20]), full[:20], atol=1e-12)      # logits of a prefix do not change


def test_sampler_matches_the_reference_outputs():
    with open(os.path.join(os.path.dirname(__file__), "golden", "sampling_golden.json")) as f:
        gold = json.load(f)
    assert gold["cases"]
    for c in gold["cases"]:
        ids, p = P.sampling_distribution(np.array(c["logits"]), c["temperature"], c["top_p"], c["top_k"], c["min_p"])
        assert ids.tolist() == c["ids"]
        assert np.allclose(p, np.array(c["p"]), rtol=1e-12, atol=0)
    pen = gold["penalize"]
    assert np.allclose(P.penalize(np.array(pen["logits"]), pen["rp"], pen["recent"]), np.array(pen["out"]))


def test_sample_with_u_walks_token_order():
    z = np.array([0.0, 2.0, 1.0, -1.0])
    ids, p = P.sampling_distribution(z, 1.0, 1.0, 0)
    order = np.argsort(ids)
    c = np.cumsum(p[order])
    for u in (0.0, 0.05, 0.3, 0.6, 0.95, 0.999999):
        assert P.sample_with_u(z, u, 1.0, 1.0, 0) == int(ids[order][np.searchsorted(c, u, side="right")])
    assert P.sample_with_u(z, 0.7, 0.0, 1.0, 0) == 1 and P.greedy(np.array([1.0, 3.0, 3.0])) == 1
    assert P.sample_with_u(z, 0.99, 1.0, 1.0, 1) == 1                                  # top_k 1 is greedy


def test_needle_models_show_a_dropped_key_and_a_window_off_by_one(tmp_path):
    """what makes the engine tests with a planted key able to fail: in the plain model itself, hiding the needle from
    the last row only (a window of T - 1 positions hides position 0 from row T - 1 and nothing else), or moving a
    layer's window by one position while the needle stands at its edge, changes that row's logits by several
    times the bfloat16 tolerance of the engine tests (eight times and more for the hidden key, four for the window)"""
    import random
    import numpy as np
    tol = 1.5e-2
    for name in ("D", "E"):
        cfg = tiny.TINY[name][0]
        folder = tiny.make_needle_model(tmp_path, cfg, seed=31, dtype="float32", name="needle" + name)
        m = P.load_model(folder)
        full = dict(m, window=None, layer_types=None)
        for seed, T in ((1, 100), (2, 400)):
            toks = tiny.needle_request(cfg["vocab_size"], T, 0, T - 8, random.Random(seed))
            whole = P.forward(full, toks).numpy()
            cut = P.forward(dict(full, window=T - 1), toks).numpy()
            assert np.array_equal(cut[:-1], whole[:-1])
            assert np.abs(cut[-1] - whole[-1]).max() / np.abs(whole).max() > 8 * tol, (name, T)
    cfg = tiny.TINY["E"][0]                                            # a window of 70 positions on its middle layer
    m = P.load_model(tiny.make_needle_model(tmp_path, cfg, seed=31, dtype="float32", name="needleE"))
    T = 120
    toks = tiny.needle_request(cfg["vocab_size"], T, T - 1 - 69, T - 8, random.Random(3))   # the last row's window edge
    a = P.forward(m, toks).numpy()
    b = P.forward(dict(m, window=cfg["sliding_window"] - 1), toks).numpy()
    assert np.abs(a[-1] - b[-1]).max() / np.abs(a).max() > 4 * tol       # (one layer of three has the window)
