"""The engine at the layer sizes of the benchmark's 3B-shaped configuration (width 2560, 20 query heads over 4
key/value heads of size 128, feed-forward 10496; two layers and a small vocabulary so that the plain implementation
stays quick): prompts long enough for every prompt-sized kernel (two row tiles per weight tile, SwiGLU in the
product's epilogue, the row-in-registers norm, the tensor-core attention over several pages), then tokens one by one
through the split-K decode products, and a batch of unequal lengths. Compared with the plain implementation."""
import numpy as np
import pytest

import plain_model as P
import tiny

pytestmark = pytest.mark.gpu

LAYER_SIZED = dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=3001, hidden_size=2560,
                   intermediate_size=10496, num_hidden_layers=2, num_attention_heads=20, num_key_value_heads=4,
                   head_dim=128, rms_norm_eps=1e-5, rope_theta=70000000.0, tie_word_embeddings=False)
TOL = 1.5e-2            # the bfloat16 tolerance of the replay tests


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    from kindi_b200.weights.random_init import write_random_model
    d = str(tmp_path_factory.mktemp("layer_sized") / "m")
    write_random_model(d, LAYER_SIZED, 21, dtype="bfloat16")
    return d


def test_layer_sized_model_matches_plain(folder, tmp_path):
    from kindi_b200.engine.engine import Engine
    vocab = LAYER_SIZED["vocab_size"]
    reqs = tiny.random_requests(vocab, [700, 45, 150], seed=3)
    m = P.load_model(folder)
    want = {rid: P.forward(m, toks).numpy() for rid, toks in reqs.items()}
    del m
    traces = {"last8": tiny.trace_last_n(reqs, 8), "batched": tiny.trace_batched(reqs, batch=3, decode=6)}
    for mode, steps in traces.items():
        eng = Engine(folder, ctx=tiny.max_live_tokens(steps), dtype="bfloat16", max_batch=3)
        out = str(tmp_path / mode)
        tiny.run_replay(eng, steps, out)
        eng.check_status()
        eng.cache.check()
        got = tiny.collect(out, steps, vocab)
        for rid, toks in reqs.items():
            mine = np.stack([got[(rid, i)] for i in range(len(toks))])
            err = tiny.rel_err(mine, want[rid])
            # where in the request the worst row lies (a prompt's end and the first decoded token are the usual suspects)
            worst_row = int(np.argmax(np.max(np.abs(mine - want[rid]), axis=1)))
            assert err <= TOL, "%s %s: %.3g at position %d of %d" % (mode, rid, err, worst_row, len(toks))
        del eng
