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
