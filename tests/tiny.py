"""Tiny configurations, model folders in temporary places, and trace builders shared by the tests."""
from __future__ import annotations

import json
import os
import random
from typing import Dict, List, Sequence, Tuple

import numpy as np

# three small configurations that differ in every size and option: head counts and groups, a head size that is no
# power of two, widths and vocabularies that are no powers of two, layer counts, eps, rope base, tied / untied,
# and (C) a window on alternating layers
TINY_A = dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=256, hidden_size=64,
              intermediate_size=192, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
              rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False, eos_token_id=2)
TINY_B = dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=384, hidden_size=96,
              intermediate_size=320, num_hidden_layers=3, num_attention_heads=3, num_key_value_heads=1, head_dim=32,
              rms_norm_eps=1e-6, rope_theta=500000.0, tie_word_embeddings=True, eos_token_id=[5, 7])
TINY_C = dict(architectures=["NanbeigeForCausalLM"], model_type="llama", vocab_size=331, hidden_size=72,
              intermediate_size=200, num_hidden_layers=4, num_attention_heads=6, num_key_value_heads=2, head_dim=48,
              rms_norm_eps=3e-6, rope_theta=1000000.0, tie_word_embeddings=False, sliding_window=40,
              layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"])
# D and E have the head sizes the tensor-core attention kernels take (64, 128) with 5 and 3 query heads per key/value
# head, so the bfloat16 runs of these two go through the serving kernels end to end
TINY_D = dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=500, hidden_size=160,
              intermediate_size=320, num_hidden_layers=2, num_attention_heads=5, num_key_value_heads=1, head_dim=64,
              rms_norm_eps=1e-5, rope_theta=70000000.0, tie_word_embeddings=False)
TINY_E = dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=777, hidden_size=200,
              intermediate_size=344, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=2, head_dim=128,
              rms_norm_eps=2e-6, rope_theta=250000.0, tie_word_embeddings=True, sliding_window=70,
              layer_types=["full_attention", "sliding_attention", "full_attention"])
TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2), "D": (TINY_D, 3), "E": (TINY_E, 4)}


def make_model(tmp_path, name: str, dtype: str = "bfloat16") -> str:
    from kindi_b200.weights.random_init import write_random_model
    cfg, seed = TINY[name]
    d = os.path.join(str(tmp_path), "tiny_%s_%s" % (name, dtype))
    if not os.path.isfile(os.path.join(d, "model.safetensors")):
        write_random_model(d, cfg, seed, dtype=dtype)
    return d


def random_requests(vocab: int, lengths: Sequence[int], seed: int) -> Dict[str, List[int]]:
    rng = random.Random(seed)
    return {"r%d" % i: [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}


# ------------------------------------------------------------------------------------------- traces
def trace_whole(reqs: Dict[str, List[int]]) -> List[dict]:
    """each request alone, all its tokens in one step, logits at every place"""
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
            for i, (rid, toks) in enumerate(reqs.items())]


def trace_last_n(reqs: Dict[str, List[int]], n: int = 32) -> List[dict]:
    """each request alone: all but the last n tokens in one step, then the last n one by one"""
    steps, s = [], 0
    for rid, toks in reqs.items():
        k = max(1, len(toks) - n)
        steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[:k], "want": list(range(k))}], "end": []})
        s += 1
        for j in range(k, len(toks)):
            steps.append({"step": s, "entries": [{"id": rid, "tokens": [toks[j]], "want": [0]}], "end": []})
            s += 1
        steps[-1]["end"] = [rid]
    return steps


def trace_batched(reqs: Dict[str, List[int]], batch: int, decode: int = 12) -> List[dict]:
    """batches of `batch` requests that start together: each brings all but its last min(decode, len - 1) tokens in
    the first step, then one token a step; shorter requests end earlier; one batch after another"""
    steps, s = [], 0
    ids = list(reqs)
    for b0 in range(0, len(ids), batch):
        group = ids[b0:b0 + batch]
        first = {r: max(1, len(reqs[r]) - min(decode + 3 * i, len(reqs[r]) - 1)) for i, r in enumerate(group)}
        at = dict(first)
        ent = [{"id": r, "tokens": reqs[r][:first[r]], "want": list(range(first[r]))} for r in group]
        live = list(group)
        while True:
            ended = [r for r in live if at[r] >= len(reqs[r])]
            steps.append({"step": s, "entries": ent, "end": ended})
            s += 1
            live = [r for r in live if r not in ended]
            if not live:
                break
            ent = [{"id": r, "tokens": [reqs[r][at[r]]], "want": [0]} for r in live]
            for r in live:
                at[r] += 1
    return steps


def max_live_tokens(steps: List[dict]) -> int:
    """the most tokens live requests hold at any time, each rounded up to 64"""
    held: Dict[str, int] = {}
    most = 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        most = max(most, sum((n + 63) // 64 * 64 for n in held.values()))
        for r in st["end"]:
            held.pop(r, None)
    return most


def collect(out_dir: str, steps: List[dict], vocab: int) -> Dict[Tuple[str, int], np.ndarray]:
    """(request id, position in the request) -> logits row, from the files a replay wrote"""
    got: Dict[Tuple[str, int], np.ndarray] = {}
    at: Dict[str, int] = {}
    for st in steps:
        n_want = sum(len(e["want"]) for e in st["entries"])
        path = os.path.join(out_dir, "%s.f32" % st["step"])
        if n_want == 0:
            assert not os.path.exists(path)
            for e in st["entries"]:
                at[e["id"]] = at.get(e["id"], 0) + len(e["tokens"])
            continue
        a = np.fromfile(path, dtype="<f4")
        assert a.size == n_want * vocab, (path, a.size, n_want, vocab)
        a = a.reshape(n_want, vocab)
        row = 0
        for e in st["entries"]:
            base = at.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], base + w)] = a[row]
                row += 1
            at[e["id"]] = base + len(e["tokens"])
        for r in st["end"]:
            at.pop(r, None)
    return got


def run_replay(engine, steps: List[dict], out_dir: str) -> None:
    import io
    from kindi_b200.engine.replay import replay
    text = io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n")
    sink = io.StringIO()
    n = replay(engine, text, out_dir, out=sink)
    assert n == len(steps)
    assert sink.getvalue().split("\n")[:-1] == ["done %s" % s["step"] for s in steps]


def rel_err(a: np.ndarray, b: np.ndarray) -> float:
    """max |a - b| over max |b|"""
    return float(np.max(np.abs(a.astype(np.float64) - b.astype(np.float64))) / (np.max(np.abs(b)) + 1e-30))


# ------------------------------------------------------------------------------------------- a planted key
NEEDLE, PROBE = 3, 4            # token ids: the needle's key stands out for every probe's query


def make_needle_model(tmp_path, cfg: dict, seed: int, dtype: str = "bfloat16", strength: float = 14.0,
                      name: str = "needle") -> str:
    """a model folder with random weights N(0, 0.02) in which ONE key stands out: the score of a PROBE token's query
    against a NEEDLE token's key is about `strength` above all others in the first layer (less in later layers),
    wherever the two stand in the sequence, for the query heads of the first key/value head. With plain random weights
    attention is nearly uniform, and a far key that a kernel drops, a window one position off or a page of another
    sequence moves the logits by less than the bfloat16 tolerance; here a probe row's attention output IS the
    needle's value, so any of these shows as an error many times the tolerance, while all other scores stay small
    and rounding errors as usual.

    How: the needle's embedding has one large feature (column 0), a probe's another (column 1); in every layer the
    key projection of the first key/value head reads column 0 into its last rotated pair's first dimension and the
    query projections of that group's heads read column 1 into the same dimension. That pair turns by less than a
    thousandth of a radian over ten thousand positions (the smallest rotary frequency), so the score does not depend on
    the distance."""
    import torch
    from kindi_b200.config.registry import model_from_config
    from kindi_b200.parts.model import expected_tensors, tensor_inits
    from kindi_b200.weights.random_init import random_tensors
    from kindi_b200.weights.safetensors_io import write_file
    d = os.path.join(str(tmp_path), "%s_%d_%s" % (name, seed, dtype))
    if os.path.isfile(os.path.join(d, "model.safetensors")):
        return d
    os.makedirs(d, exist_ok=True)
    _, spec = model_from_config(cfg)
    tdt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    t = random_tensors(expected_tensors(spec), seed, dtype=torch.float32, inits=tensor_inits(spec))
    width, hd = cfg["hidden_size"], cfg["head_dim"]
    group = cfg["num_attention_heads"] // cfg["num_key_value_heads"]
    w = (strength * hd ** 0.5 / width) ** 0.5          # q . k / sqrt(hd) = w^2 * width / sqrt(hd) = strength
    emb = t["model.embed_tokens.weight"]
    emb[:, 0:2] = 0.0
    emb[NEEDLE, 0] = 1.0
    emb[PROBE, 1] = 1.0
    dim = hd // 2 - 1
    for i in range(cfg["num_hidden_layers"]):
        p = "model.layers.%d.self_attn." % i
        t[p + "k_proj.weight"][dim, 0] = w
        for h in range(group):
            t[p + "q_proj.weight"][h * hd + dim, 1] = w
    t = {n: v.to(tdt) for n, v in t.items()}
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(dict(cfg, torch_dtype=dtype), f)
    write_file(os.path.join(d, "model.safetensors"), t, metadata={"format": "pt"})
    return d


def needle_request(vocab: int, length: int, needle_at: int, probes_from: int, rng: random.Random) -> List[int]:
    """random tokens (neither needle nor probe) with the needle at `needle_at` and probes from `probes_from` on"""
    toks = []
    for i in range(length):
        t = rng.randrange(vocab)
        while t in (NEEDLE, PROBE):
            t = rng.randrange(vocab)
        toks.append(NEEDLE if i == needle_at else PROBE if i >= probes_from and i != needle_at else t)
    return toks


def trace_group(reqs: Dict[str, List[int]], decode: Dict[str, int], first_step: int = 0) -> List[dict]:
    """one batch that starts together: request r brings all but its last decode[r] tokens in the first step (at least
    one), then one token a step; a request ends with its last token, so the batch shrinks as it goes"""
    first = {r: max(1, len(t) - decode[r]) for r, t in reqs.items()}
    at = dict(first)
    live = list(reqs)
    ent = [{"id": r, "tokens": reqs[r][:first[r]], "want": list(range(first[r]))} for r in live]
    steps, s = [], first_step
    while True:
        ended = [r for r in live if at[r] >= len(reqs[r])]
        steps.append({"step": s, "entries": ent, "end": ended})
        s += 1
        live = [r for r in live if r not in ended]
        if not live:
            return steps
        ent = [{"id": r, "tokens": [reqs[r][at[r]]], "want": [0]} for r in live]
        for r in live:
            at[r] += 1
