"""A plain, slow implementation of the Llama-arch Nanbeige decoder and of the sampler, for the tests.

Whole sequences, no cache, no batching, one function per part, float64 on the CPU by default. It shares no code
with the package: it reads config.json with ``json`` and the weights with the ``safetensors`` package, and every
function restates a formula of the reference (cited as file:line of ahtx/kindi).

The reference's model cannot be run here as a whole: its engine needs CuPy and a quantised GGUF file
(``kindi/nanbeige.py:240``), and its kernels take only head size 128 and 5 or 7 query heads per key/value head
(``kindi/nanbeige.py:260``). What can be run is pinned on the reference's own output, stored under ``tests/golden/``
with the scripts that made it: ``kindi/sampling.py`` (NumPy only) against ``sampling_distribution``
(``make_sampling_golden.py``), and the reference's CUDA kernels that take and give 32-bit tensors - add + RMS norm,
rotation with the key/value store, decode attention with its merge, prompt attention, argmax - compiled as they
stand for sm_100a and run on a B200, against ``rms_norm``, ``rope_rotate_half``, ``attention`` and ``greedy``
(``make_reference_kernel_golden.py``, ``tests/reference_kernels.py``). The matrix products, the SwiGLU and the order
of a layer's operations rest on the formulas (the reference's own are int8 x low-bit products).
"""
from __future__ import annotations

import json
import math
import os
from typing import Optional, Sequence

import numpy as np
import torch


# --------------------------------------------------------------------------------------------- loading
def load_model(model_dir: str, dtype=torch.float64) -> dict:
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    w = {}
    for n in sorted(os.listdir(model_dir)):
        if n.endswith(".safetensors"):
            w.update(load_file(os.path.join(model_dir, n)))
    w = {k: v.to(dtype) for k, v in w.items()}
    heads = cfg["num_attention_heads"]
    return {
        "cfg": cfg, "w": w, "dtype": dtype,
        "layers": cfg["num_hidden_layers"], "heads": heads, "kv_heads": cfg.get("num_key_value_heads", heads),
        "head_dim": cfg.get("head_dim") or cfg["hidden_size"] // heads,        # kindi/nanbeige.py:257
        "eps": cfg["rms_norm_eps"],                                            # kindi/nanbeige.py:255
        "theta": cfg.get("rope_theta", 10000.0),                               # kindi/nanbeige.py:256
        "tied": bool(cfg.get("tie_word_embeddings", False)),
        "window": cfg.get("sliding_window"), "layer_types": cfg.get("layer_types"),
    }


# --------------------------------------------------------------------------------------------- parts
def embedding(table: torch.Tensor, tokens: Sequence[int]) -> torch.Tensor:
    """x = table[tok], no scaling (kindi/nbq.cu:472-487; kindi/nanbeige.py:681)"""
    return table[torch.tensor(list(tokens), dtype=torch.long)]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """scale = 1 / sqrt(mean(x^2) + eps); y = (scale * x) * w (kindi/nbq.cu:412-432: ss / n + eps, rsqrt, then the
    two products); the weight multiplies as stored"""
    scale = 1.0 / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return (scale * x) * w


def rope_tables(positions: torch.Tensor, rot: int, theta: float, dtype) -> tuple:
    """angle = float32(pos) * float32(theta ** (-2 i / rot)) for pair i, the product rounded to 32-bit ("fp32 angle,
    as the reference (pos.float() * inv_freq)", kindi/dspine.cu:167-168; theta_scale in 32-bit, kindi/nanbeige.py:683)"""
    i = torch.arange(0, rot // 2, dtype=torch.float64)
    inv_freq = (theta ** (-2.0 * i / rot)).to(torch.float32)
    ang = (positions.to(torch.float32)[:, None] * inv_freq[None, :]).to(torch.float64)
    return torch.cos(ang).to(dtype), torch.sin(ang).to(dtype)


def rope_rotate_half(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [T, heads, head_dim]; pairs (i, i + rot/2): out[i] = a c - b s, out[i + rot/2] = b c + a s
    (kindi/dspine.cu:166-173; the same rotation on adjacent pairs of permuted rows: kindi/nbq.cu:127-130,497-520)"""
    half = cos.shape[-1]
    a, b, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([a * c - b * s, b * c + a * s, rest], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
              window: Optional[int] = None) -> torch.Tensor:
    """q: [T, heads, d]; k, v: [T, kv_heads, d]. Query head h uses key/value head h // (heads / kv_heads)
    (kindi/nbq.cu:525-633: a block takes the G query heads of one K/V head); scores (q * scale) . k with
    scale = 1 / sqrt(d) (kindi/nanbeige.py:684; kindi/nbq.cu:553); a row sees positions 0..its own
    (kindi/nbq.cu:536: n = pos + 1), or only the last `window` of them; softmax; weighted sum of v
    (kindi/nbq.cu:635-649: o / l)"""
    T, H, d = q.shape
    G = H // k.shape[1]
    out = torch.empty_like(q)
    idx = torch.arange(T)
    visible = idx[None, :] <= idx[:, None]
    if window:
        visible &= idx[None, :] > idx[:, None] - window
    for h in range(H):
        s = (q[:, h, :] * scale) @ k[:, h // G, :].T
        s = s.masked_fill(~visible, float("-inf"))
        out[:, h, :] = torch.softmax(s, dim=-1) @ v[:, h // G, :]
    return out


def swiglu_mlp(y: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    """g = Wg y, u = Wu y, h = g / (1 + exp(-g)) * u (kindi/nbq.cu:461-467), out = Wd h (kindi/nanbeige.py:710-718);
    no biases"""
    g, u = y @ wg.T, y @ wu.T
    return (g / (1.0 + torch.exp(-g)) * u) @ wd.T


def decoder_layer(m: dict, i: int, x: torch.Tensor, cos, sin) -> torch.Tensor:
    """pre-norm block: x += Wo attn(norm(x)); x += mlp(norm(x)) (kindi/nanbeige.py:688-718; the reference defers each
    add into the next fused add + norm, which is the same sum)"""
    w, p = m["w"], "model.layers.%d." % i
    T = x.shape[0]
    H, KV, d = m["heads"], m["kv_heads"], m["head_dim"]
    y = rms_norm(x, w[p + "input_layernorm.weight"], m["eps"])
    q = (y @ w[p + "self_attn.q_proj.weight"].T).view(T, H, d)
    k = (y @ w[p + "self_attn.k_proj.weight"].T).view(T, KV, d)
    v = (y @ w[p + "self_attn.v_proj.weight"].T).view(T, KV, d)
    q, k = rope_rotate_half(q, cos, sin), rope_rotate_half(k, cos, sin)
    window = m["window"]
    if window and m["layer_types"] is not None and m["layer_types"][i] != "sliding_attention":
        window = None
    a = attention(q, k, v, 1.0 / math.sqrt(d), window).reshape(T, H * d)
    x = x + a @ w[p + "self_attn.o_proj.weight"].T
    y = rms_norm(x, w[p + "post_attention_layernorm.weight"], m["eps"])
    return x + swiglu_mlp(y, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])


def forward(m: dict, tokens: Sequence[int]) -> torch.Tensor:
    """logits [T, vocab] of a whole sequence: embedding, the layers, final norm (kindi/nbq.cu:435-453), head
    (kindi/nanbeige.py:720-724); a tied head is the embedding table (kindi/tp.py:850-851)"""
    w = m["w"]
    x = embedding(w["model.embed_tokens.weight"], tokens)
    cos, sin = rope_tables(torch.arange(len(tokens)), m["head_dim"], m["theta"], m["dtype"])
    for i in range(m["layers"]):
        x = decoder_layer(m, i, x, cos, sin)
    y = rms_norm(x, w["model.norm.weight"], m["eps"])
    head = w["model.embed_tokens.weight"] if m["tied"] else w["lm_head.weight"]
    return y @ head.T


# --------------------------------------------------------------------------------------------- sampling
def greedy(logits: np.ndarray) -> int:
    """argmax, ties to the lowest id (kindi/nbq.cu:670-694)"""
    return int(np.argmax(logits))


def penalize(z: np.ndarray, rp: float, recent: Sequence[int]) -> np.ndarray:
    """a recent token's logit is divided by rp when positive, multiplied when negative (kindi/sampling.py:117-123)"""
    z = z.astype(np.float64).copy()
    for t in set(int(t) for t in recent):
        z[t] = z[t] / rp if z[t] > 0 else z[t] * rp
    return z


def sampling_distribution(z: np.ndarray, temperature: float, top_p: float, top_k: int, min_p: float = 0.0,
                          order: str = "llama"):
    """the token ids (best first) and probabilities the sampler draws from (kindi/sampling.py:91-114): keep the
    top_k best (0: all), then the shortest best-first prefix whose mass before each token is < top_p (probabilities
    at temperature 1, or at the temperature with order "hf"), then tokens with z >= z_max + ln(min_p), then
    p = softmax((z - z_max) / temperature). Exact ties at a cut: the reference takes an arbitrary one of the tied
    tokens (np.argpartition, kindi/sampling.py:97-98); this library keeps every token whose logit equals the last
    kept one, so that the result does not depend on an order among equals."""
    z = np.asarray(z, dtype=np.float64)
    ids = np.argsort(-z, kind="stable")
    if top_k and top_k < len(ids):
        ids = ids[z[ids] >= z[ids[top_k - 1]]]
    zs = z[ids]
    if top_p and top_p < 1.0:
        q = zs / temperature if order == "hf" else zs
        q = np.exp(q - q.max())
        q /= q.sum()
        keep = (np.cumsum(q) - q) < top_p
        keep = zs >= zs[keep][-1]
        ids, zs = ids[keep], zs[keep]
    if min_p and min_p > 0.0:
        keep = zs >= zs.max() + np.log(min_p)
        ids, zs = ids[keep], zs[keep]
    p = np.exp((zs - zs.max()) / temperature)
    return ids, p / p.sum()


def sample_with_u(z: np.ndarray, u: float, temperature: float, top_p: float, top_k: int, min_p: float = 0.0,
                  order: str = "llama") -> int:
    """the draw for a given uniform number u in [0, 1): the kept tokens are walked in token-id order and the first
    whose cumulative probability exceeds u is taken (the reference draws with NumPy's choice over the same
    distribution, kindi/sampling.py:86-88; the walk order is this library's own)"""
    if temperature <= 0:
        return greedy(z)
    ids, p = sampling_distribution(z, temperature, top_p, top_k, min_p, order)
    o = np.argsort(ids)
    ids, p = ids[o], p[o]
    c = np.cumsum(p)
    k = int(np.searchsorted(c, u * c[-1], side="right"))
    return int(ids[min(k, len(ids) - 1)])
