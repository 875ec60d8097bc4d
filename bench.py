#!/usr/bin/env python3
"""Measurement: decoded tokens a second of the 3B-shaped Nanbeige/Llama-arch model on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 8192] [--layers L]

The default run has the layer sizes of the benchmark's 3B-shaped configuration (32 layers, width 2560, 20 heads,
4 key/value heads of size 128, feed-forward 10496, vocabulary 166144, bfloat16) with seeded random weights, a batch
of 8 sequences each at a context of 8192 tokens. A "step" is one decode step of the whole batch. It prints ONE JSON
line: ``value`` = decoded tokens a second timed on the device with CUDA events around exactly K steps; ``e2e`` = the
same through ``Engine.generate_batch`` (token ids in and out as Python lists; every step's inputs are copied from
pinned host memory and its picked tokens read back); ``prefill`` = one 2048-token prompt; ``roofline`` = the bytes a decode
step has to read (every weight once, the live sequences' keys and values) over its time, against the measured
copy bandwidth; ``points`` = decoding at batch 1 and 64 (tokens a second); ``points_detail`` = the same and further
batch sizes and context lengths, each with its step time, the bytes it has to read and its fraction of the copy
bandwidth; ``kernels`` = device time per kind of launch of one decode step and one prompt pass issued launch by
launch (CUDA events around every launch, outside the timed regions). For more than one GPU it says so and exits with
2: this library runs on one GPU. ``--impl reference`` says why ahtx/kindi's engine cannot run here and, where its
kernel sources are at hand, times its two attention kernels at this configuration's shape.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the benchmark's 3B-shaped configuration
CONFIG_3B = dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=166144, hidden_size=2560,
                 intermediate_size=10496, num_hidden_layers=32, num_attention_heads=20, num_key_value_heads=4,
                 head_dim=128, rms_norm_eps=1e-5, rope_theta=70000000.0, tie_word_embeddings=False)
# the benchmark's two larger configurations (same architecture, other layer sizes), for runs with --preset
CONFIG_16B = dict(CONFIG_3B, hidden_size=5120, intermediate_size=13824, num_hidden_layers=48, num_attention_heads=40,
                  num_key_value_heads=8)
CONFIG_33B = dict(CONFIG_3B, hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=40,
                  num_key_value_heads=8)
PRESETS = {"3b": ("Nanbeige4-3B-shaped llama-arch", CONFIG_3B), "16b": ("16B-class llama-arch", CONFIG_16B),
           "33b": ("33B-class llama-arch", CONFIG_33B)}
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            with open(p) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            out.update({k: float(v) for k, v in d.items() if k in out and isinstance(v, (int, float))})
            out["source"] = "measured"
            return out
        except (OSError, ValueError):
            pass
    out = dict(FALLBACK_PEAKS)
    out["source"] = "fallback"
    return out


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 200 ms while a timed region runs"""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", "0", "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                       "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            out, _ = self.p.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
            out, _ = self.p.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def build_engine(layers: int, ctx: int, max_batch: int, base=None):
    import torch
    from kindi_b200.config import model_from_config
    from kindi_b200.engine.engine import Engine
    from kindi_b200.parts.model import expected_tensors, tensor_inits
    from kindi_b200.weights.random_init import random_tensors
    cfg = dict(base or CONFIG_3B)
    cfg["num_hidden_layers"] = layers
    mc, spec = model_from_config(cfg)
    tensors = random_tensors(expected_tensors(spec), seed=0, std=0.02, dtype=torch.bfloat16, device="cuda:0",
                             inits=tensor_inits(spec))
    eng = Engine(spec=spec, tensors=tensors, ctx=ctx, dtype="bfloat16", max_batch=max_batch)
    eng.config = mc
    return eng


def prefill_flops(mc, T: int) -> float:
    E, F, nh, nkv, hd, L = (mc.hidden_size, mc.intermediate_size, mc.num_attention_heads, mc.num_key_value_heads,
                            mc.head_dim, mc.num_hidden_layers)
    per_tok = 2.0 * (E * (nh + 2 * nkv) * hd + nh * hd * E + 3 * E * F)
    attn = 2.0 * 2.0 * nh * hd * (T * (T + 1) / 2.0)           # QK^T and PV over the causal half
    return L * (T * per_tok + attn) + 2.0 * E * mc.vocab_size  # the head runs on one row


def bench_prefill(eng, warmup: int, iters: int, tokens: int = 0, with_min: bool = False):
    import random
    import torch
    from kindi_b200.engine.batch import StepEntry
    rng = random.Random(3)
    tokens = tokens or PREFILL_TOKENS
    ids = tuple(rng.randrange(eng.spec.vocab_size) for _ in range(tokens))
    times = []
    for i in range(warmup + iters):
        slot = eng.alloc()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        eng.step([StepEntry(slot, ids, (tokens - 1,))])
        b.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(a.elapsed_time(b))
        eng.free(slot)
    eng.check_status()
    if with_min:
        return statistics.median(times), min(times)
    return statistics.median(times)


def bench_unequal(eng, n_prompts: int = 8, new_tokens: int = 256):
    """8 prompts of seeded random lengths 128..2048 that start together: one packed prompt step, then 256 greedy
    tokens each, through Engine.generate_batch (host tokens in and out every step)"""
    import random
    import torch
    rng = random.Random(11)
    prompts = [[rng.randrange(eng.spec.vocab_size) for _ in range(rng.randint(128, 2048))] for _ in range(n_prompts)]
    eng.generate_batch(prompts[:2], temperature=0.0, max_tokens=4)           # warm-up (graphs of other batch sizes aside)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    res = eng.generate_batch(prompts, temperature=0.0, max_tokens=new_tokens)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    made = sum(len(t) for t in res.tokens)
    return {"prompts": n_prompts, "prompt_tokens": sum(len(p) for p in prompts), "new_tokens": made,
            "seconds": round(dt, 4), "tokens_per_s": round(made / dt, 1),
            "prompt_s": round(res.stats.prompt_s, 4), "decode_s": round(res.stats.gen_s, 4),
            "decode_tokens_per_s": round(res.stats.gen_tok_s, 1), "steps": res.stats.steps}


def fill_context(eng, batch: int, context: int):
    """B sequences that each hold `context` tokens: pages are mapped and lengths set; the keys and values are
    synthetic (the whole pool is filled with N(0, 1) once), which costs a decode step exactly what real ones do"""
    slots = []
    for _ in range(batch):
        s = eng.alloc()
        eng.cache.reserve(s, context)
        eng.cache.commit(s, context)
        slots.append(s)
    eng.cache.flush()
    return slots


def bench_decode(eng, batch: int, context: int, steps: int, warmup: int, e2e: bool):
    """returns (device ms per step, e2e ms per step or None, launches in the device-timed region, bytes per step)"""
    import torch
    from kindi_b200.engine.batch import StepEntry
    from kindi_b200.kernels import lib as K
    slots = fill_context(eng, batch, context - 1)
    toks = [(17 * i + 5) % eng.spec.vocab_size for i in range(batch)]

    def one(toks):
        entries = [StepEntry(s, (t,), (0,)) for s, t in zip(slots, toks)]
        return eng.step(entries, greedy=True)[1]

    for _ in range(max(3, warmup)):
        one(toks)
    torch.cuda.synchronize()
    eng.check_status()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n0 = K.launch_count()
    a.record()
    for _ in range(steps):
        one(toks)
    b.record()
    torch.cuda.synchronize()
    dev_ms = a.elapsed_time(b) / steps
    launches = K.launch_count() - n0
    eng.check_status()
    e2e_ms = None
    bytes_step = eng.weight_bytes_per_step(batch) + batch * context * eng.kv_bytes_per_token()
    for s in slots:
        eng.free(s)
    if e2e:
        e2e_ms = bench_e2e(eng, batch, context, steps)
    return dev_ms, e2e_ms, launches, bytes_step


def bench_e2e(eng, batch: int, context: int, steps: int, warm: int = 48, sampling=None) -> float:
    """milliseconds per decode step through the call a user makes, ``Engine.generate_batch``: `batch` prompts of
    context - 1 token ids given as Python lists, greedy tokens returned as Python lists. Every step copies its inputs
    (positions, lengths, slots, row lists, tokens) from pinned host memory to the device and reads its picked tokens
    and the status word back. The first `warm` decode steps are not timed (right after the prompt pass the GPU still
    runs at the clocks its power limit forced during that pass: the first twenty to thirty steps take 3.2 ms instead
    of 2.65 at batch 8); the time is the wall clock between the token callbacks of the last `steps` steps."""
    import random
    import torch
    rng = random.Random(5)
    vocab = eng.spec.vocab_size
    prompts = [[rng.randrange(vocab) for _ in range(context - 1)] for _ in range(batch)]
    how = dict(sampling) if sampling else dict(temperature=0.0)       # greedy, unless sampling options are given
    eng.generate_batch([p[:64] for p in prompts], max_tokens=8, stop_token_ids=(), **how)       # warm-up
    torch.cuda.synchronize()
    stamps = []
    res = eng.generate_batch(prompts, max_tokens=warm + steps + 1, stop_token_ids=(),
                             on_tokens=lambda d: stamps.append(time.perf_counter()), **how)
    assert all(len(t) == warm + steps + 1 for t in res.tokens) and len(stamps) == warm + steps + 1
    return (stamps[-1] - stamps[-1 - steps]) * 1000.0 / steps


def kernel_times(eng, batch: int, context: int, prefill_tokens: int):
    """device time per kind of launch: one decode step of `batch` sequences at `context` and one prompt pass, each
    issued launch by launch (no recorded graph, launches strictly one after another) with CUDA events around every
    launch. The events cost about a microsecond a launch and nothing overlaps, so the sums are larger than the
    step times measured above: read them as shares."""
    import random
    from kindi_b200.engine.batch import StepEntry
    from kindi_b200.kernels import lib as K
    out = {}
    graphs, eng.cuda_graphs = eng.cuda_graphs, False
    K.set_pdl(False)
    try:
        slots = fill_context(eng, batch, context - 1)
        entries = [StepEntry(s, ((17 * i + 5) % eng.spec.vocab_size,), (0,)) for i, s in enumerate(slots)]
        eng.step(entries, greedy=True)
        for s in slots:
            eng.cache.commit(s, context - 1)
        with K.KernelTiming() as t:
            eng.step(entries, greedy=True)
        out["decode_step_b%d_ctx%d" % (batch, context)] = t.summary()
        for s in slots:
            eng.free(s)
        rng = random.Random(3)
        ids = tuple(rng.randrange(eng.spec.vocab_size) for _ in range(prefill_tokens))
        for timed in (False, True):
            slot = eng.alloc()
            if timed:
                with K.KernelTiming() as t:
                    eng.step([StepEntry(slot, ids, (prefill_tokens - 1,))])
                out["prompt_pass_%d" % prefill_tokens] = t.summary()
            else:
                eng.step([StepEntry(slot, ids, (prefill_tokens - 1,))])
            eng.free(slot)
        eng.check_status()
    finally:
        eng.cuda_graphs = graphs
        K.set_pdl(True)
    return out


REFERENCE_UNAVAILABLE = ("ahtx/kindi is not pip-installable offline (no setup.py or pyproject.toml); its Nanbeige engine "
                         "needs CuPy (not installed, no index) and a quantised GGUF model file, has no bf16 "
                         "safetensors path and serves one request at a time")


def reference_kernel_times(cfg, context: int, prefill_tokens: int):
    """the reference's own attention kernels (kindi/nbq.cu nbq_attn_part_g5 + nbq_attn_merge, kindi/nbq_fa.cu
    nbq_fa_prefill_g5: fp16 cache, mma.sync) compiled as they stand for sm_100a and timed at this configuration's
    shape: one decode query over `context` cached positions, and the attention of a `prefill_tokens` prompt. A
    kernel-level bar on the same GPU, not an end-to-end number. None when the sources or a GPU are not at hand."""
    import ctypes
    import math
    import tempfile
    ref = os.path.join(ROOT, "baseline", "_ref", "kindi")
    harness = os.path.join(ROOT, "tests", "golden", "reference_kernels_harness.cu")
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    if not all(os.path.isfile(os.path.join(ref, f)) for f in ("nbq.cu", "nbq_fa.cu", "nbq_grids.h")) \
            or not os.path.isfile(harness) or hd != 128 or nh != 5 * nkv:
        return None
    try:
        import torch
        if not torch.cuda.is_available():
            return None
        with tempfile.TemporaryDirectory() as tmp:
            so = os.path.join(tmp, "libref.so")
            r = subprocess.run(["nvcc", "-shared", "-Xcompiler", "-fPIC", "-std=c++14", "-use_fast_math", "-w", "-gencode",
                                "arch=compute_100a,code=sm_100a", "-I", ref, harness, "-o", so], capture_output=True,
                               text=True)
            if r.returncode != 0:
                return None
            lib = ctypes.CDLL(so)
            dev = "cuda"
            ctx = (max(context, prefill_tokens) + 255) // 256 * 256
            p = lambda t: ctypes.c_void_p(t.data_ptr())
            kc = (torch.randn(nkv * ctx * hd, device=dev) * 0.5).to(torch.float16)
            vc = (torch.randn(nkv * ctx * hd, device=dev) * 0.5).to(torch.float16)
            scale = ctypes.c_float(1.0 / math.sqrt(hd))
            nsplit = 16                                            # kindi/nanbeige.py:17
            q = torch.randn(1, nh * hd, device=dev)
            pos = torch.tensor([context - 1], dtype=torch.int32, device=dev)
            part_o = torch.zeros(nh * nsplit * hd, device=dev)
            part_ms = torch.zeros(nh * nsplit * 2, device=dev)
            o = torch.empty(1, nh * hd, device=dev)
            qp = torch.randn(prefill_tokens, nh * hd, device=dev)
            op = torch.empty(prefill_tokens, nh * hd, device=dev)
            flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)     # larger than the L2

            def timed(fn, n=10):
                best = []
                for i in range(3 + n):
                    flush.zero_()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    rc = fn()
                    b.record()
                    torch.cuda.synchronize()
                    if rc != 0:
                        raise RuntimeError("CUDA error %d" % rc)
                    if i >= 3:
                        best.append(a.elapsed_time(b) * 1000.0)
                return round(statistics.median(best), 1)
            dec = timed(lambda: lib.ref_attn_decode_g5(p(q), p(kc), p(vc), p(pos), ctx, scale, p(part_o), p(part_ms),
                                                       nh * hd, nkv, nsplit, 1, p(o)))
            pre = timed(lambda: lib.ref_fa_prefill_g5(p(qp), nh * hd, prefill_tokens, 0, p(kc), p(vc), ctx, scale, p(op),
                                                      nkv))
            return {"decode_attention_b1_ctx%d_us" % context: dec, "prefill_attention_%d_us" % prefill_tokens: pre,
                    "what": "kindi/nbq.cu nbq_attn_part_g5 + nbq_attn_merge and kindi/nbq_fa.cu nbq_fa_prefill_g5, "
                            "compiled unchanged for sm_100a, one layer, fp16 cache, L2 flushed before each launch, "
                            "host-synchronised launches (a few microseconds of launch time are inside)"}
    except Exception as e:                                          # noqa: BLE001
        return {"error": str(e)[:200]}


def bench_torch(cfg, layers: int, batch: int, context: int, steps: int, warmup: int, prefill_tokens: int):
    """a comparison arm that is NOT the reference and not this library: the same model (same seeded weights, same
    sizes) written with PyTorch's own operators - cuBLAS products, its fused attention over a dense bf16 cache, element
    by element kernels for norm, rotation and SwiGLU - with the decode step recorded as a CUDA graph. What library code
    gives on this GPU for the same metric; the formulas are those of tests/plain_model.py."""
    import math
    import torch
    import torch.nn.functional as F
    from kindi_b200.config import model_from_config
    from kindi_b200.parts.model import expected_tensors, tensor_inits
    from kindi_b200.weights.random_init import random_tensors
    c = dict(cfg)
    c["num_hidden_layers"] = layers
    mc, spec = model_from_config(c)
    w = random_tensors(expected_tensors(spec), seed=0, std=0.02, dtype=torch.bfloat16, device="cuda:0",
                       inits=tensor_inits(spec))
    E, nh, nkv, hd, eps = mc.hidden_size, mc.num_attention_heads, mc.num_key_value_heads, mc.head_dim, mc.rms_norm_eps
    wqkv = [torch.cat([w["model.layers.%d.self_attn.%s_proj.weight" % (i, n)] for n in "qkv"]) for i in range(layers)]
    wgu = [torch.cat([w["model.layers.%d.mlp.%s_proj.weight" % (i, n)] for n in ("gate", "up")]) for i in range(layers)]
    inv = (mc.rope_theta ** (-2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)).float().cuda()

    def norm(x, g):
        return (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)).to(torch.bfloat16) * g

    def rope(x, pos):                                        # x [B, T, heads, hd], pos [B, T]
        ang = pos[..., None].float() * inv
        cs, sn = torch.cos(ang)[:, :, None], torch.sin(ang)[:, :, None]
        a, b = x[..., : hd // 2].float(), x[..., hd // 2:].float()
        return torch.cat([a * cs - b * sn, b * cs + a * sn], -1).to(torch.bfloat16)

    def forward(tok, pos, kc, vc, lens):
        """tok, pos [B, T]; caches [layers][B, nkv, ctx, hd]; lens = keys each sequence holds after this step (int)"""
        B, T = tok.shape
        x = w["model.embed_tokens.weight"][tok].float()
        for i in range(layers):
            p = "model.layers.%d." % i
            y = norm(x, w[p + "input_layernorm.weight"])
            qkv = y @ wqkv[i].T
            q = rope(qkv[..., : nh * hd].view(B, T, nh, hd), pos)
            k = rope(qkv[..., nh * hd: (nh + nkv) * hd].view(B, T, nkv, hd), pos)
            v = qkv[..., (nh + nkv) * hd:].view(B, T, nkv, hd)
            kc[i][:, :, lens - T: lens] = k.transpose(1, 2)
            vc[i][:, :, lens - T: lens] = v.transpose(1, 2)
            att = F.scaled_dot_product_attention(q.transpose(1, 2), kc[i][:, :, :lens], vc[i][:, :, :lens],
                                                 is_causal=T > 1, enable_gqa=True)
            x = x + (att.transpose(1, 2).reshape(B, T, nh * hd) @ w[p + "self_attn.o_proj.weight"].T).float()
            y = norm(x, w[p + "post_attention_layernorm.weight"])
            gu = y @ wgu[i].T
            h = F.silu(gu[..., : gu.shape[-1] // 2].float()).to(torch.bfloat16) * gu[..., gu.shape[-1] // 2:]
            x = x + (h @ w[p + "mlp.down_proj.weight"].T).float()
        y = norm(x[:, -1], w["model.norm.weight"])
        return (y @ w["lm_head.weight"].T).float().argmax(-1)

    out = {}
    # ---- decode: B sequences that hold `context` keys after the step; the step recorded as a CUDA graph
    kc = [torch.randn(batch, nkv, context, hd, device="cuda").to(torch.bfloat16) for _ in range(layers)]
    vc = [torch.randn(batch, nkv, context, hd, device="cuda").to(torch.bfloat16) for _ in range(layers)]
    tok = torch.randint(0, mc.vocab_size, (batch, 1), device="cuda")
    pos = torch.full((batch, 1), context - 1, device="cuda", dtype=torch.int64)
    for _ in range(3):
        forward(tok, pos, kc, vc, context)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        picked = forward(tok, pos, kc, vc, context)
    for _ in range(max(3, warmup)):
        g.replay()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(steps):
        g.replay()
    b.record()
    torch.cuda.synchronize()
    out["decode_ms"] = a.elapsed_time(b) / steps
    del kc, vc, g
    # ---- prefill of one prompt (eager: launch by launch, as PyTorch runs a model)
    kc = [torch.zeros(1, nkv, prefill_tokens, hd, device="cuda", dtype=torch.bfloat16) for _ in range(layers)]
    vc = [torch.zeros(1, nkv, prefill_tokens, hd, device="cuda", dtype=torch.bfloat16) for _ in range(layers)]
    tok = torch.randint(0, mc.vocab_size, (1, prefill_tokens), device="cuda")
    pos = torch.arange(prefill_tokens, device="cuda")[None]
    ts = []
    for i in range(8):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        forward(tok, pos, kc, vc, prefill_tokens)
        b.record()
        torch.cuda.synchronize()
        if i >= 3:
            ts.append(a.elapsed_time(b))
    out["prefill_ms"] = statistics.median(ts)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference", "torch"),
                    help="ours; the reference (unavailable here, with its attention kernels timed); or 'torch': the same "
                         "model written with PyTorch's own operators, a comparison that is neither")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--preset", default="3b", choices=sorted(PRESETS),
                    help="layer sizes: the 3B-shaped configuration (default) or one of the two larger ones")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (0: all)")
    ap.add_argument("--unequal", action="store_true",
                    help="also generate for 8 prompts of random lengths 128 to 2048, 256 tokens each, through the "
                         "Python entry point (the 16B-class configuration's workload)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end measurement (for profiling runs)")
    ap.add_argument("--sampled", action="store_true",
                    help="also measure the end-to-end decode step with the reference's default sampling (temperature "
                         "0.7, top-p 0.8, top-k 20) and report it as e2e_sampled")
    ap.add_argument("--no-pdl", action="store_true", help="launch kernels strictly one after another")
    ap.add_argument("--prefill-only", action="store_true", help="measure only the prefill (for profiling)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                    help="prompt length of --prefill-only (the full run always measures 2048 tokens)")
    a = ap.parse_args(argv)
    if a.impl == "reference":
        line = {"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}
        kt = reference_kernel_times(PRESETS[a.preset][1], a.context, PREFILL_TOKENS)
        if kt is not None:
            line["kernel_level"] = kt
        print(json.dumps(line))
        return 0
    if a.impl == "torch" and a.gpus == 1:
        name, base = PRESETS[a.preset]
        layers = a.layers if a.layers > 0 else base["num_hidden_layers"]
        r = bench_torch(base, layers, a.batch, a.context, a.steps, max(3, a.warmup), PREFILL_TOKENS)
        print(json.dumps({"impl": "torch", "what": "the same model with PyTorch's own operators (cuBLAS, fused attention "
                          "over a dense bf16 cache, the decode step as a CUDA graph): not the reference, not this library",
                          "metric": "decode tokens/s (batch %d, context %d)" % (a.batch, a.context),
                          "value": round(a.batch * 1000.0 / r["decode_ms"], 1), "unit": "tokens/s",
                          "ms_per_step": round(r["decode_ms"], 4), "steps": a.steps, "layers": layers, "dtype": "bf16",
                          "prefill": {"tokens": PREFILL_TOKENS, "ms": round(r["prefill_ms"], 3),
                                      "value": round(PREFILL_TOKENS * 1000.0 / r["prefill_ms"], 1)}}))
        return 0
    if a.gpus != 1:
        print("kindi_b200 is a one-GPU library: bench.py measures N=1 only (asked for --gpus %d)" % a.gpus)
        return 2
    a.warmup = max(3, a.warmup)
    model_name, base = PRESETS[a.preset]
    if a.layers <= 0:
        a.layers = base["num_hidden_layers"]
    import torch
    from kindi_b200.engine.batch import layout
    pk = peaks()
    if a.no_pdl:
        from kindi_b200.kernels import lib as _K
        _K.set_pdl(False)
    point_batches = (1, 64) if a.preset == "3b" else (1,)          # 64 sequences of 8192 need too much cache beyond 3B
    max_b = max(a.batch, 1 if a.no_points else max(point_batches))
    ctx = max_b * (a.context + a.steps * 2 + a.warmup + 320) + PREFILL_TOKENS + 64
    if a.prefill_only:
        eng = build_engine(a.layers, a.prefill_tokens + 128, 2, base)
        pms = bench_prefill(eng, 2, max(1, min(a.steps, 3)), a.prefill_tokens)
        print(json.dumps({"prefill_only": True, "layers": a.layers, "tokens": a.prefill_tokens, "ms": round(pms, 3),
                          "value": round(a.prefill_tokens * 1000.0 / pms, 1)}))
        return 0
    eng = build_engine(a.layers, ctx, max_b, base)
    for g in eng.cache.groups:
        g.pool.normal_(0.0, 1.0)
    mc = eng.config
    clocks = ClockSampler()
    clocks.start()
    dev_ms, e2e_ms, launches, bytes_step = bench_decode(eng, a.batch, a.context, a.steps, a.warmup, not a.no_e2e)
    clk = clocks.stop()
    value = a.batch * 1000.0 / dev_ms
    out = {
        "metric": "decode tokens/s (batch %d, context %d)" % (a.batch, a.context), "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(dev_ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02) seed 0, synthetic token ids, cache filled with N(0,1)",
        "impl": "ours",
        "config": {"model": model_name, "global_batch": a.batch, "seq_len": a.context,
                   "parallelism": "none (1 GPU)", "layers": a.layers, "layers_of_config": base["num_hidden_layers"],
                   "hidden_size": mc.hidden_size, "heads": mc.num_attention_heads, "kv_heads": mc.num_key_value_heads,
                   "head_dim": mc.head_dim, "intermediate_size": mc.intermediate_size, "vocab_size": mc.vocab_size,
                   "rope_theta": mc.rope_theta, "rms_norm_eps": mc.rms_norm_eps, "tied": mc.tie_word_embeddings,
                   "prefill_tokens": PREFILL_TOKENS, "l2": "inputs larger than L2 (a step reads %.1f GB)" % (bytes_step / 1e9),
                   "cuda_graph": eng.graph_replays > 0},
        "clocks": clk,
        "gpu_launches": launches,
        "e2e": None if e2e_ms is None else {
            "value": round(a.batch * 1000.0 / e2e_ms, 1), "unit": "tokens/s",
            "h2d_bytes_per_step": 4 * layout(a.batch, a.batch, a.batch)[1], "d2h_bytes_per_step": 4 * a.batch + 4,
            "ms_per_step": round(e2e_ms, 4)},
        "roofline": {"bound": "hbm", "achieved": round(bytes_step / dev_ms / 1e6, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(bytes_step / dev_ms / 1e6 / pk["hbm_gbs"], 4),
                     "of": pk["source"], "bytes_per_step": int(bytes_step)},
    }
    if a.sampled:
        sms = bench_e2e(eng, a.batch, a.context, a.steps, sampling=dict(temperature=0.7, top_p=0.8, top_k=20, seed=1))
        out["e2e_sampled"] = {"value": round(a.batch * 1000.0 / sms, 1), "unit": "tokens/s", "ms_per_step": round(sms, 4),
                              "sampling": "temperature 0.7, top-p 0.8, top-k 20"}
    if not a.no_points:
        T = PREFILL_TOKENS
        # (the median of 20 passes back to back: under that sustained load the GPU runs slower than in a burst, which
        # is what the second fraction and the fastest pass are there to show)
        pms, pmin = bench_prefill(eng, 5, 20, with_min=True)
        fl = prefill_flops(mc, T)
        out["prefill"] = {"value": round(T * 1000.0 / pms, 1), "tokens": T, "ms": round(pms, 3),
                          "frac": round(fl / (pms / 1000.0) / (pk["bf16_tflops"] * 1e12), 4), "of": pk["source"],
                          "tflop": round(fl / 1e12, 3), "ms_fastest": round(pmin, 3),
                          "frac_of_sustained_peak": round(fl / (pms / 1000.0) / (pk["bf16_tflops_sustained"] * 1e12), 4)}
        pts, detail = {}, {}
        detail["decode_b%d_ctx%d" % (a.batch, a.context)] = {
            "tokens_per_s": round(value, 1), "ms": round(dev_ms, 4), "bytes_per_step": int(bytes_step),
            "frac": round(bytes_step / dev_ms / 1e6 / pk["hbm_gbs"], 4)}
        cache_room = eng.ctx
        for b in sorted(set(point_batches) | {a.batch}):
            for c in sorted({512, a.context, 32768}):
                if (b, c) == (a.batch, a.context) or b * (c + 2 * a.steps + 64) > cache_room:
                    continue                                       # (the headline; or more than the cache was sized for)
                ms, _, _, by = bench_decode(eng, b, c, max(16, a.steps // 2), a.warmup, False)
                detail["decode_b%d_ctx%d" % (b, c)] = {
                    "tokens_per_s": round(b * 1000.0 / ms, 1), "ms": round(ms, 4), "bytes_per_step": int(by),
                    "frac": round(by / ms / 1e6 / pk["hbm_gbs"], 4)}
                if c == a.context and b in point_batches:
                    pts["decode_b%d" % b] = round(b * 1000.0 / ms, 1)
        for b in (16, 32):                                         # batch sizes between the named points
            if b != a.batch and b <= max_b and b * (a.context + 2 * a.steps + 64) <= cache_room:
                ms, _, _, by = bench_decode(eng, b, a.context, max(16, a.steps // 2), a.warmup, False)
                detail["decode_b%d_ctx%d" % (b, a.context)] = {
                    "tokens_per_s": round(b * 1000.0 / ms, 1), "ms": round(ms, 4), "bytes_per_step": int(by),
                    "frac": round(by / ms / 1e6 / pk["hbm_gbs"], 4)}
        out["points"] = pts
        out["points_detail"] = detail
        out["kernels"] = kernel_times(eng, a.batch, a.context, PREFILL_TOKENS)
    if a.unequal:
        out["unequal_batch"] = bench_unequal(eng)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
