"""Configurations at the edges of what the kernels take: head sizes in steps of 16 other than the tensor-core ones,
widths that are no multiple of 8 (no TMA-aligned rows), a feed-forward size that is no multiple of 64 or 8, many
query heads per key/value head, a single head, prime vocabularies, a window. Every case is replayed whole, with its
last tokens one by one and in an unequal batch, in 32-bit and in bfloat16, against the plain implementation."""
import numpy as np
import pytest

import plain_model as P
import tiny

pytestmark = pytest.mark.gpu


def _cfg(**kw):
    base = dict(architectures=["LlamaForCausalLM"], model_type="llama", rms_norm_eps=1e-5, rope_theta=10000.0,
                tie_word_embeddings=False)
    base.update(kw)
    return base


ODD = {
    # head size 96 (general attention kernel), width 100 (no 16-byte rows: the general product), odd feed-forward
    "hd96_w100": _cfg(vocab_size=211, hidden_size=100, intermediate_size=150, num_hidden_layers=2,
                      num_attention_heads=3, num_key_value_heads=3, head_dim=96),
    # 24 query heads on one key/value head of size 64 (more than the decode kernel's 16 a group), width 136
    "g24_hd64": _cfg(vocab_size=307, hidden_size=136, intermediate_size=264, num_hidden_layers=2,
                     num_attention_heads=24, num_key_value_heads=1, head_dim=64, tie_word_embeddings=True),
    # one head of size 256 (the largest), width 64, feed-forward 72
    "one_head_256": _cfg(vocab_size=127, hidden_size=64, intermediate_size=72, num_hidden_layers=3,
                         num_attention_heads=1, num_key_value_heads=1, head_dim=256, rms_norm_eps=1e-6),
    # head size 112, 7 query heads per key/value head, width 392 (a multiple of 8), feed-forward 1000, window 33
    "hd112_g7_window": _cfg(vocab_size=401, hidden_size=392, intermediate_size=1000, num_hidden_layers=2,
                            num_attention_heads=7, num_key_value_heads=1, head_dim=112, sliding_window=33,
                            layer_types=["sliding_attention", "full_attention"], rope_theta=500000.0),
    # head size 128 with 17 query heads per key/value head (prompt kernel yes, decode kernel no), width 272
    "hd128_g17": _cfg(vocab_size=257, hidden_size=272, intermediate_size=320, num_hidden_layers=2,
                      num_attention_heads=17, num_key_value_heads=1, head_dim=128),
}
TOL = {"float32": 2e-5, "bfloat16": 1.5e-2}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ODD))
def test_odd_sizes_match_plain(tmp_path, name, dtype):
    from kindi_b200.engine.engine import Engine
    from kindi_b200.weights.random_init import write_random_model
    cfg = ODD[name]
    folder = str(tmp_path / name)
    write_random_model(folder, cfg, 5, dtype=dtype)
    vocab = cfg["vocab_size"]
    reqs = tiny.random_requests(vocab, [70, 3, 130, 41], seed=8)
    m = P.load_model(folder)
    want = {rid: P.forward(m, toks).numpy() for rid, toks in reqs.items()}
    for mode, steps in (("whole", tiny.trace_whole(reqs)), ("last8", tiny.trace_last_n(reqs, 8)),
                        ("batched", tiny.trace_batched(reqs, batch=3, decode=5))):
        eng = Engine(folder, ctx=tiny.max_live_tokens(steps), dtype=dtype, max_batch=3)
        out = str(tmp_path / (name + mode))
        tiny.run_replay(eng, steps, out)
        eng.check_status()
        eng.cache.check()
        got = tiny.collect(out, steps, vocab)
        for rid, toks in reqs.items():
            mine = np.stack([got[(rid, i)] for i in range(len(toks))])
            err = tiny.rel_err(mine, want[rid])
            assert err <= TOL[dtype], "%s %s %s %s: %.3g" % (name, mode, rid, dtype, err)
        del eng
