"""Each kernel alone against a plain PyTorch float32 reference of the same operation, at sizes other than the
engine's: odd widths, tile edges, head sizes in steps of 16, any number of heads and groups."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from kindi_b200.kernels import lib
    lib.load()
    return lib


def _status():
    return torch.zeros(1, dtype=torch.int32, device="cuda")


def _rel(a, b):
    return float((a.double() - b.double()).abs().max() / (b.double().abs().max() + 1e-30))


@pytest.mark.parametrize("M,N,K_", [(1, 7, 5), (3, 64, 64), (65, 130, 33), (128, 96, 200), (9, 331, 72)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_simt(K, M, N, K_, dtype):
    g = torch.Generator(device="cuda").manual_seed(M * 1000 + N)
    a = torch.randn(M, K_, device="cuda", generator=g).to(dtype)
    w = torch.randn(N, K_, device="cuda", generator=g).to(dtype)
    out = torch.empty(M, N, device="cuda", dtype=torch.float32)
    K.gemm_simt(a, w, out)
    ref = a.double() @ w.double().T
    assert _rel(out, ref) < 1e-6


# (M, N, K, swap, bn, splits): tile edges in every dimension, K tails that are no multiple of 64, both forms
TC_CASES = [
    (128, 256, 64, False, 256, 1), (128, 128, 128, False, 128, 1), (200, 300, 136, False, 128, 1),
    (2048, 512, 2560, False, 256, 1), (130, 72, 72, False, 64, 1), (257, 1000, 520, False, 256, 1),
    (300, 700, 200, False, 160, 1), (129, 500, 136, False, 192, 1), (512, 2560, 320, False, 224, 1),
    (260, 2560, 200, False, 144, 1), (140, 360, 72, False, 176, 1), (300, 3584, 264, False, 208, 1),
    (129, 1000, 136, False, 240, 1),
    # the prefill form with K split into planes (a few hundred rows: fewer tiles than SMs)
    (256, 2560, 10496, False, 256, 6), (300, 700, 1096, False, 128, 3), (129, 500, 4096, False, 192, 8),
    (1, 128, 64, True, 16, 1), (8, 384, 2560, True, 16, 1), (8, 384, 2560, True, 16, 5), (17, 200, 264, True, 32, 3),
    (64, 331 * 8, 1096, True, 64, 4), (100, 256, 4096, True, 128, 8), (5, 130, 72, True, 16, 2),
]


@pytest.mark.parametrize("M,N,K_,swap,bn,splits", TC_CASES)
def test_gemm_tc(K, M, N, K_, swap, bn, splits):
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K_)
    a = torch.randn(M, K_, device="cuda", generator=g).to(torch.bfloat16)
    w = torch.randn(N, K_, device="cuda", generator=g).to(torch.bfloat16)
    ref = a.double() @ w.double().T
    st = _status()
    S = K.gemm_tc_splits(K_, splits)
    if splits > 1:
        out = torch.full((S, M, N), float("nan"), device="cuda", dtype=torch.float32)
        K.gemm_tc(a, w, out, swap=swap, bn=bn, splits=splits, status=st)
        got = out.sum(dim=0)
    else:
        got = torch.full((M, N), float("nan"), device="cuda", dtype=torch.float32)
        K.gemm_tc(a, w, got, swap=swap, bn=bn, splits=1, status=st)
    assert int(st.item()) == 0
    assert _rel(got, ref) < 1e-5            # exact bf16 products, 32-bit accumulation
    if splits == 1:
        o16 = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        K.gemm_tc(a, w, o16, swap=swap, bn=bn, splits=1, status=st)
        assert int(st.item()) == 0
        assert _rel(o16.float(), ref) < 5e-3


# ------------------------------------------------------------------------------------------------ attention
def _make_cache(lengths, nkv, hd, dtype, seed, n_extra_pages=3):
    """a page pool with random keys and values for sequences of the given lengths, pages handed out in a shuffled
    order; returns pool [n_pages, 2, nkv, 64, hd], table, and the dense K, V of each sequence"""
    g = torch.Generator(device="cpu").manual_seed(seed)
    need = [(n + 63) // 64 for n in lengths]
    n_pages = sum(need) + n_extra_pages
    perm = torch.randperm(n_pages, generator=g).tolist()
    pool = (torch.randn(n_pages, 2, nkv, 64, hd, generator=g) * 3.0).to(dtype)       # unmapped space is NOT zero
    table = torch.full((len(lengths) + 2, n_pages), -1, dtype=torch.int32)
    dense = []
    slots = list(range(len(lengths), 0, -1))                # slots in another order than the batch
    for b, n in enumerate(lengths):
        k = torch.randn(n, nkv, hd, generator=g).to(dtype)
        v = torch.randn(n, nkv, hd, generator=g).to(dtype)
        for j in range(need[b]):
            pg = perm.pop()
            table[slots[b], j] = pg
            lo, hi = j * 64, min(n, j * 64 + 64)
            pool[pg, 0, :, : hi - lo] = k[lo:hi].transpose(0, 1)
            pool[pg, 1, :, : hi - lo] = v[lo:hi].transpose(0, 1)
        dense.append((k, v))
    return pool.cuda(), table.cuda(), dense, torch.tensor(slots, dtype=torch.int32).cuda(), n_pages


def _attn_ref(q, k, v, pos, scale, window):
    """q [nq, nh, hd] rows at positions pos (list); k, v [n, nkv, hd]; float64"""
    nq, nh, hd = q.shape
    G = nh // k.shape[1]
    out = torch.zeros(nq, nh, hd, dtype=torch.float64)
    for i, p in enumerate(pos):
        lo = max(0, p - window + 1) if window else 0
        for h in range(nh):
            s = (k[lo:p + 1, h // G].double() @ q[i, h].double()) * scale
            w = torch.softmax(s, dim=0)
            out[i, h] = w @ v[lo:p + 1, h // G].double()
    return out


def _run_attention(K, kind, dtype, nh, nkv, hd, q_lens, kv_lens, window, seed, boost=None):
    """kind: 'generic' | 'prefill' | 'decode'. Sequence b brings q_lens[b] rows that end at position kv_lens[b] - 1."""
    pool, table, dense, slots, n_pages = _make_cache(kv_lens, nkv, hd, dtype, seed)
    g = torch.Generator(device="cpu").manual_seed(seed + 1)
    T = sum(q_lens)
    q = torch.randn(T, nh, hd, generator=g).to(dtype)
    if boost is not None:
        # make one far key stand out for one row: scale that key and the row's query along the key's direction
        b, row, key = boost
        r0 = sum(q_lens[:b]) + row
        kvec = dense[b][0][key, 0].float()
        q[r0, 0] = (kvec / kvec.norm() * 12.0).to(dtype)
        page = int(table[slots[b], key // 64])
        pool[page, 0, 0, key % 64] = (kvec / kvec.norm() * 12.0).to(dtype).cuda()
        dense[b][0][key, 0] = (kvec / kvec.norm() * 12.0).to(dtype)
    scale = 1.0 / math.sqrt(hd)
    pos, seq, q_start = [], [], [0]
    for b, (ql, kl) in enumerate(zip(q_lens, kv_lens)):
        pos += list(range(kl - ql, kl))
        seq += [b] * ql
        q_start.append(q_start[-1] + ql)
    dev = lambda x: torch.tensor(x, dtype=torch.int32).cuda()      # noqa: E731
    qd = q.reshape(T, nh * hd).cuda()
    out = torch.full((T, nh * hd), float("nan"), dtype=dtype).cuda()
    st = _status()
    if kind == "generic":
        K.attn_generic(qd, out, dev(pos), dev(seq), slots, nh, nkv, hd, scale, window, pool, table, n_pages, st)
    elif kind == "tc":
        G = nh // nkv
        K.attn_tc(qd, out, slots, dev(q_start), dev(kv_lens), len(q_lens), nh, nkv, hd, scale, window, pool, table,
                  n_pages, grid_x=-(-max(q_lens) // (128 // G)), status=st)
    else:
        G = nh // nkv
        gx = 5 if kind == "decode" else -(-max(q_lens) * G // 64)
        K.attn_mma(qd, out, slots, dev(q_start), dev(kv_lens), len(q_lens), nh, nkv, hd, scale, window, pool, table,
                   n_pages, decode=kind == "decode", grid_x=gx, status=st)
    assert int(st.item()) == 0
    got = out.float().cpu().reshape(T, nh, hd)
    at = 0
    worst = 0.0
    for b, (ql, kl) in enumerate(zip(q_lens, kv_lens)):
        ref = _attn_ref(q[at:at + ql].float(), dense[b][0].float(), dense[b][1].float(), pos[at:at + ql], scale, window)
        worst = max(worst, float((got[at:at + ql].double() - ref).abs().max() / ref.abs().max()))
        at += ql
    return worst


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 16, 0), (3, 1, 48, 0), (6, 2, 80, 37), (2, 2, 256, 0)])
def test_attention_generic(K, dtype, tol, nh, nkv, hd, window):
    err = _run_attention(K, "generic", dtype, nh, nkv, hd, [5, 1, 70, 33], [5, 130, 70, 97], window, seed=hd)
    assert err < tol
    err = _run_attention(K, "generic", dtype, nh, nkv, hd, [1, 1], [300, 65], window, seed=hd + 1, boost=(0, 0, 3))
    assert err < tol


@pytest.mark.parametrize("nh,nkv,hd,window", [(20, 4, 128, 0), (3, 1, 64, 0), (8, 8, 128, 0), (6, 2, 64, 100),
                                              (10, 2, 128, 64), (16, 1, 128, 0)])
def test_attention_mma_prefill(K, nh, nkv, hd, window):
    # whole prompts, a chunk that continues an earlier part, single rows, lengths at and around page edges
    err = _run_attention(K, "prefill", torch.bfloat16, nh, nkv, hd, [64, 1, 130, 33, 7], [64, 129, 130, 97, 200],
                         window, seed=nh)
    assert err < 1e-2
    # one far key among hundreds decides a row
    err = _run_attention(K, "prefill", torch.bfloat16, nh, nkv, hd, [40, 3], [700, 65], window=0, seed=nh + 1,
                         boost=(0, 39, 5))
    assert err < 1e-2


@pytest.mark.parametrize("nh,nkv,hd,window", [(20, 4, 128, 0), (3, 1, 64, 0), (8, 8, 128, 0), (14, 2, 64, 100),
                                              (10, 2, 128, 64), (16, 1, 128, 0)])
def test_attention_mma_decode(K, nh, nkv, hd, window):
    err = _run_attention(K, "decode", torch.bfloat16, nh, nkv, hd, [1] * 6, [1, 64, 65, 700, 129, 320], window,
                         seed=nh + 7)
    assert err < 1e-2
    err = _run_attention(K, "decode", torch.bfloat16, nh, nkv, hd, [1, 1], [900, 65], window=0, seed=nh + 9,
                         boost=(0, 0, 3))
    assert err < 1e-2


def test_attention_mma_decode_with_a_cta_alone_on_its_sm(K):
    """a decode step of no more CTAs than SMs (one split, 30 sequences x 4 heads) asks for an SM per CTA: the same
    results as with any other launch shape"""
    kv_lens = [1 + (37 * i) % 700 for i in range(30)]
    pool, table, dense, slots, n_pages = _make_cache(kv_lens, 4, 128, torch.bfloat16, seed=5)
    g = torch.Generator(device="cpu").manual_seed(6)
    B, nh, nkv, hd = len(kv_lens), 20, 4, 128
    q = torch.randn(B, nh, hd, generator=g).to(torch.bfloat16)
    dev = lambda x: torch.tensor(x, dtype=torch.int32).cuda()      # noqa: E731
    st = _status()
    outs = []
    for splits in (1, 2):
        out = torch.full((B, nh * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
        K.attn_mma(q.reshape(B, nh * hd).cuda(), out, slots, dev(list(range(B + 1))), dev(kv_lens), B, nh, nkv, hd,
                   1.0 / math.sqrt(hd), 0, pool, table, n_pages, decode=True, grid_x=splits, status=st)
        assert int(st.item()) == 0
        outs.append(out.float().cpu().reshape(B, nh, hd))
    for b in range(B):
        ref = _attn_ref(q[b:b + 1].float(), dense[b][0].float(), dense[b][1].float(), [kv_lens[b] - 1],
                        1.0 / math.sqrt(hd), 0)
        for o in outs:
            assert float((o[b:b + 1].double() - ref).abs().max() / ref.abs().max()) < 1e-2


@pytest.mark.parametrize("nh,nkv,hd,window,planes", [(20, 4, 128, 0, 5), (3, 1, 64, 0, 1), (16, 1, 128, 0, 2),
                                                     (14, 2, 64, 100, 7), (10, 2, 128, 64, 3)])
def test_attention_decode_rotates_and_stores_by_itself(K, nh, nkv, hd, window, planes):
    """the decode attention that takes the QKV planes gives the same bits as the rotate-and-store kernel followed by
    the decode attention, leaves the same cache behind, and without storing reads what is there"""
    kv_lens = [1, 64, 65, 700, 129, 320, 128]
    B = len(kv_lens)
    pool, table, dense, slots, n_pages = _make_cache(kv_lens, nkv, hd, torch.bfloat16, seed=nh + hd)
    g = torch.Generator(device="cpu").manual_seed(nh)
    width = (nh + 2 * nkv) * hd
    qkv = torch.randn(B, width, generator=g)
    parts = torch.randn(planes, B, width, generator=g)
    parts[-1] = qkv - parts[:-1].sum(0)
    parts = parts.cuda().contiguous()
    inv = (250000.0 ** (-2 * torch.arange(hd // 2, dtype=torch.float64) / hd)).float().cuda()
    dev = lambda x: torch.tensor(x, dtype=torch.int32).cuda()      # noqa: E731
    pos, seq, q_start = dev([n - 1 for n in kv_lens]), dev(list(range(B))), dev(list(range(B + 1)))
    scale = 1.0 / math.sqrt(hd)
    st = _status()
    # the two kernels
    pool_a = pool.clone()
    q = torch.empty(B, nh * hd, dtype=torch.bfloat16, device="cuda")
    K.rope_store(parts, q, inv, hd, pos, seq, slots, nh, nkv, hd, pool_a, table, n_pages, st)
    want = torch.full((B, nh * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    K.attn_mma(q, want, slots, q_start, dev(kv_lens), B, nh, nkv, hd, scale, window, pool_a, table, n_pages,
               decode=True, grid_x=5, status=st)
    # the one kernel
    pool_b = pool.clone()
    got = torch.full((B, nh * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    K.attn_decode_rope(parts, inv, got, slots, q_start, dev(kv_lens), B, nh, nkv, hd, scale, window, pool_b, True,
                       table, n_pages, grid_x=5, status=st)
    assert int(st.item()) == 0
    assert torch.equal(pool_a, pool_b)
    assert torch.equal(got, want)
    # nothing stored: the newest key and value are the ones the cache already holds
    pool_c = pool_a.clone()
    got2 = torch.full((B, nh * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    K.attn_decode_rope(parts[:, :, : nh * hd].contiguous(), inv, got2, slots, q_start, dev(kv_lens), B, nh, nkv, hd,
                       scale, window, pool_c, False, table, n_pages, grid_x=3, status=st)
    assert int(st.item()) == 0 and torch.equal(pool_c, pool_a)
    assert _rel(got2.float(), want.float()) < 1e-2          # other splits: another order of the merge


@pytest.mark.parametrize("M,F,K_,bn", [(129, 64, 128, 128), (2048, 1024, 520, 256), (300, 320, 264, 256), (200, 192, 72, 128),
                                       (260, 176, 136, 160), (150, 48, 64, 224)])
def test_gemm_tc_finishes_swiglu_in_its_epilogue(K, M, F, K_, bn):
    g = torch.Generator(device="cuda").manual_seed(M + F + K_)
    a = (torch.randn(M, K_, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    wg = (torch.randn(F, K_, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    wu = (torch.randn(F, K_, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    wgu = torch.stack([wg.view(F // 16, 16, K_), wu.view(F // 16, 16, K_)], dim=1).reshape(2 * F, K_).contiguous()
    st = _status()
    out = torch.full((M, F), float("nan"), device="cuda", dtype=torch.bfloat16)
    K.gemm_tc(a, wgu, out, swap=False, bn=bn, splits=1, status=st, swiglu=True)
    gg, uu = a.double() @ wg.double().T, a.double() @ wu.double().T
    ref = gg / (1 + torch.exp(-gg)) * uu
    assert int(st.item()) == 0
    assert _rel(out.float(), ref) < 6e-3
    # the stand-alone kernel reads the same grouping, from bf16 rows and from 32-bit planes
    rows = torch.empty(M, 2 * F, device="cuda", dtype=torch.bfloat16)
    K.gemm_tc(a, wgu, rows, swap=False, bn=bn, splits=1, status=st)
    h = torch.empty(M, F, device="cuda", dtype=torch.bfloat16)
    K.swiglu(rows, h, 16)
    assert _rel(h.float(), ref) < 1.5e-2
    planes = rows.float()[None].contiguous()
    K.swiglu(planes, h, 16)
    assert _rel(h.float(), ref) < 1.5e-2


@pytest.mark.parametrize("nh,nkv,window,hd", [(20, 4, 0, 128), (3, 1, 0, 128), (8, 8, 0, 128), (10, 2, 64, 128),
                                              (16, 1, 0, 128), (6, 2, 100, 128), (5, 1, 0, 64), (8, 8, 0, 64),
                                              (14, 2, 100, 64), (12, 1, 64, 64)])
def test_attention_tc_prefill(K, nh, nkv, window, hd):
    # whole prompts, a chunk that continues an earlier part, single rows, lengths at and around page edges
    err = _run_attention(K, "tc", torch.bfloat16, nh, nkv, hd, [64, 1, 130, 33, 7], [64, 129, 130, 97, 200],
                         window, seed=nh)
    assert err < 1e-2
    # one far key among hundreds decides a row (the lazy maximum has to follow it)
    err = _run_attention(K, "tc", torch.bfloat16, nh, nkv, hd, [40, 3], [700, 65], window=0, seed=nh + 1,
                         boost=(0, 39, 5))
    assert err < 1e-2
    err = _run_attention(K, "tc", torch.bfloat16, nh, nkv, hd, [300], [300], window=window, seed=nh + 2,
                         boost=(0, 299, 250))
    assert err < 1e-2


@pytest.mark.parametrize("M,N,K_,bn", [(256, 256, 64, 256), (2048, 2560, 1096, 256), (300, 700, 200, 192),
                                       (513, 1000, 136, 128), (1000, 520, 264, 64), (1900, 2500, 520, 192),
                                       (2048, 3584, 200, 256), (100, 96, 72, 128), (2304, 2560, 328, 256)])
def test_gemm_pair_of_sms(K, M, N, K_, bn):
    """the product on pairs of SMs (tcgen05 with cta_group::2), tile by tile and with the K blocks of all tiles dealt
    out evenly (tiles finished by two pairs), both output types, and SwiGLU in the epilogue"""
    g = torch.Generator(device="cuda").manual_seed(M + N + K_)
    a = torch.randn(M, K_, device="cuda", generator=g).to(torch.bfloat16)
    w = torch.randn(N, K_, device="cuda", generator=g).to(torch.bfloat16)
    ref = a.double() @ w.double().T
    st = _status()
    tiles = -(-M // 256) * -(-N // bn)
    part = torch.full((tiles * 256 * bn,), float("nan"), device="cuda")
    flags = torch.zeros(8 * tiles, dtype=torch.int32, device="cuda")
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 5e-3)):
        out = torch.full((M, N), float("nan"), device="cuda", dtype=dtype)
        K.gemm_pair(a, w, out, bn=bn, status=st)
        assert int(st.item()) == 0
        assert _rel(out.float(), ref) < tol
        first = None
        for _ in range(2):          # twice: the flags of the first call have been lowered, and the bits are the same
            out2 = torch.full((M, N), float("nan"), device="cuda", dtype=dtype)
            K.gemm_pair(a, w, out2, bn=bn, status=st, part=part, flags=flags)
            assert int(st.item()) == 0 and int(flags.abs().sum().item()) == 0
            assert _rel(out2.float(), ref) < tol
            assert first is None or torch.equal(first, out2)
            first = out2
    if N % 32 == 0:
        F = N // 2
        wg, wu = w[:F], w[F:]
        wgu = torch.stack([wg.view(F // 16, 16, K_), wu.view(F // 16, 16, K_)], dim=1).reshape(N, K_).contiguous()
        h = torch.full((M, F), float("nan"), device="cuda", dtype=torch.bfloat16)
        K.gemm_pair(a * 0.1, wgu, h, bn=bn, status=st, swiglu=True)
        assert int(st.item()) == 0
        gg = (a * 0.1).double() @ wg.double().T
        uu = (a * 0.1).double() @ wu.double().T
        assert _rel(h.float(), gg / (1 + torch.exp(-gg)) * uu) < 1e-2


def test_prompt_products_as_the_engine_chooses_them(K):
    """the dispatch of prompt-sized products at the benchmark's layer sizes: the down product goes to pairs of SMs with
    its K blocks dealt out evenly (scratch and flags kept by the dispatcher, reused by the next call), gate/up to pairs
    tile by tile with SwiGLU in the epilogue, QKV to one CTA a unit; all against float64 products"""
    from kindi_b200.kernels import fast
    assert fast._prefill_tile(2048, 2560, 10496) == ("pair", 256, True)
    assert fast._prefill_tile(2048, 20992, 2560, True) == ("pair", 256, False)
    assert fast._prefill_tile(2048, 3584, 2560)[0] == "tc"
    g = torch.Generator(device="cuda").manual_seed(5)
    st = _status()
    M = 2048
    for N, K_ in ((2560, 10496), (3584, 2560)):
        a = (torch.randn(M, K_, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
        w = (torch.randn(N, K_, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
        ref = a.float() @ w.float().T               # (float32 on the GPU: float64 at this size takes too long)
        for _ in range(2):
            planes = fast.gemm_planes(a, w, st)
            assert planes is not None and int(st.item()) == 0
            assert _rel(planes.sum(0), ref) < 2e-5
        out = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
        assert fast.gemm_rows(a, w, out, st) and int(st.item()) == 0
        assert _rel(out.float(), ref) < 5e-3
    F, K_ = 9472, 1024
    a = (torch.randn(M, K_, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    wg = (torch.randn(F, K_, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    wu = (torch.randn(F, K_, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    wgu = torch.stack([wg.view(F // 16, 16, K_), wu.view(F // 16, 16, K_)], dim=1).reshape(2 * F, K_).contiguous()
    assert fast._prefill_tile(M, 2 * F, K_, True)[0] == "pair"
    h = torch.full((M, F), float("nan"), device="cuda", dtype=torch.bfloat16)
    assert fast.gemm_swiglu_rows(a, wgu, h, st) and int(st.item()) == 0
    gg, uu = a.float() @ wg.float().T, a.float() @ wu.float().T
    assert _rel(h.float(), gg / (1 + torch.exp(-gg)) * uu) < 1e-2
    assert all(int(f.abs().sum().item()) == 0 for _, f in fast._PAIR_SCRATCH.values())


def test_products_of_a_few_hundred_rows_split_k(K):
    """the output and down products of a short prompt (129 to 511 rows) come as several planes of a K split that fills
    the SMs; their sum is the product"""
    from kindi_b200.kernels import fast
    assert fast._prefill_split(256, 2560, 10496)[1] > 1 and fast._prefill_split(2048, 2560, 10496) is None
    g = torch.Generator(device="cuda").manual_seed(6)
    st = _status()
    for M, N, K_ in ((256, 2560, 10496), (129, 2560, 2560), (500, 2560, 10496), (384, 1000, 4104)):
        a = (torch.randn(M, K_, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
        w = (torch.randn(N, K_, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
        planes = fast.gemm_planes(a, w, st)
        assert int(st.item()) == 0 and planes.shape[1:] == (M, N)
        if fast._prefill_split(M, N, K_) is not None:
            assert planes.shape[0] > 1
        assert _rel(planes.sum(0), a.double() @ w.double().T) < 1e-5


@pytest.mark.parametrize("M,N,K_,bn", [(256, 256, 64, 128), (2048, 2560, 1096, 160), (300, 700, 200, 192),
                                       (513, 1000, 136, 224), (1000, 520, 264, 256), (2048, 2560, 328, 144),
                                       (300, 400, 72, 176), (2048, 3584, 200, 208), (257, 500, 136, 240)])
def test_gemm_tc_two_row_tiles(K, M, N, K_, bn):
    g = torch.Generator(device="cuda").manual_seed(M + N + K_)
    a = torch.randn(M, K_, device="cuda", generator=g).to(torch.bfloat16)
    w = torch.randn(N, K_, device="cuda", generator=g).to(torch.bfloat16)
    ref = a.double() @ w.double().T
    st = _status()
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 5e-3)):
        out = torch.full((M, N), float("nan"), device="cuda", dtype=dtype)
        K.gemm_tc(a, w, out, swap=False, bn=bn, splits=1, status=st, mt=2)
        assert int(st.item()) == 0
        assert _rel(out.float(), ref) < tol
    if bn % 32 == 0 and N % 32 == 0:
        F = N // 2
        wg, wu = w[:F], w[F:]
        wgu = torch.stack([wg.view(F // 16, 16, K_), wu.view(F // 16, 16, K_)], dim=1).reshape(N, K_).contiguous()
        h = torch.full((M, F), float("nan"), device="cuda", dtype=torch.bfloat16)
        K.gemm_tc(a * 0.1, wgu, h, swap=False, bn=bn, splits=1, status=st, swiglu=True, mt=2)
        gg, uu = (a * 0.1).double() @ wg.double().T, (a * 0.1).double() @ wu.double().T
        assert _rel(h.float(), gg / (1 + torch.exp(-gg)) * uu) < 6e-3


@pytest.mark.parametrize("M,F,K_", [(8, 10496, 2560), (1, 48, 64), (16, 64, 72), (17, 1008, 264), (64, 2656, 328),
                                    (100, 512, 1096), (5, 9488, 200), (3, 9472, 136)])
def test_decode_gate_up_product_finishes_swiglu_itself(K, M, F, K_):
    """the decode-sized gate/up product whose CTAs take equal stretches of all (tile, K block) pairs and meet in shared
    tiles: against the plain formula, twice in a row over the same scratch (flags are left as they were found), and
    with as many tiles as there are CTAs, fewer, and more"""
    from kindi_b200.kernels import fast
    g = torch.Generator(device="cuda").manual_seed(M + F + K_)
    a = (torch.randn(M, K_, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    wg = (torch.randn(F, K_, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    wu = (torch.randn(F, K_, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    wgu = torch.stack([wg.view(F // 16, 16, K_), wu.view(F // 16, 16, K_)], dim=1).reshape(2 * F, K_).contiguous()
    gg, uu = a.double() @ wg.double().T, a.double() @ wu.double().T
    ref = gg / (1 + torch.exp(-gg)) * uu
    st = _status()
    bn = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128
    tiles = -(-2 * F // 128)
    part = torch.full((tiles * bn * 128,), float("nan"), device="cuda")
    flags = torch.zeros(tiles, dtype=torch.int32, device="cuda")
    for _ in range(2):
        out = torch.full((M, F), float("nan"), device="cuda", dtype=torch.bfloat16)
        K.gemm_swiglu_decode(a, wgu, out, bn, part, flags, st)
        assert int(st.item()) == 0
        assert _rel(out.float(), ref) < 6e-3
        assert int(flags.abs().sum().item()) == 0
    # the engine's way in: the decode form (with scratch of its own) or the prompt form, whichever takes the shape
    out = torch.full((M, F), float("nan"), device="cuda", dtype=torch.bfloat16)
    took = [fast.gemm_swiglu_decode(a, wgu, out, st), False]
    if not took[0]:
        took[1] = fast.gemm_swiglu_rows(a, wgu, out, st)
    assert took == [fast._swiglu_in_decode_form(a), not fast._swiglu_in_decode_form(a)]
    assert int(st.item()) == 0 and _rel(out.float(), ref) < 6e-3


# ------------------------------------------------------------------------------------------------ small kernels
@pytest.mark.parametrize("T,E,planes", [(3, 50, 0), (8, 2560, 7), (5, 72, 3), (600, 2560, 1), (600, 96, 9), (70, 4100, 2),
                                        (520, 1000, 2), (513, 2048, 0), (600, 3200, 1), (601, 5120, 6), (701, 2560, 6),
                                        (2100, 2560, 3), (2049, 520, 1), (515, 5200, 2), (161, 2560, 7), (159, 2560, 7), (1791, 1024, 1),
                                        (1793, 1024, 2)])
@pytest.mark.parametrize("ydtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(K, T, E, planes, ydtype):
    g = torch.Generator(device="cuda").manual_seed(T + E)
    x0 = torch.randn(T, E, device="cuda", generator=g)
    d = torch.randn(planes, T, E, device="cuda", generator=g) * 0.3 if planes else None
    for wdtype in (torch.float32, torch.bfloat16):
        w = (1 + 0.1 * torch.randn(E, device="cuda", generator=g)).to(wdtype)
        x = x0.clone()
        y = torch.empty(T, E, device="cuda", dtype=ydtype)
        st = _status()
        K.add_rmsnorm(x, d, w, 1e-5, y, None, write_back=d is not None, status=st)
        v = x0.double() + (d.double().sum(0) if planes else 0)
        ref = v / torch.sqrt((v * v).mean(-1, keepdim=True) + 1e-5) * w.double()
        assert _rel(x, v) < 1e-6 and _rel(y.float(), ref) < (2e-6 if ydtype == torch.float32 else 6e-3)
        # a gather of rows, nothing written back
        rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32).cuda()
        x2 = x0.clone()
        y2 = torch.empty(3, E, device="cuda", dtype=ydtype)
        K.add_rmsnorm(x2, d, w, 1e-5, y2, rows, write_back=False, status=st)
        assert torch.equal(x2, x0) and _rel(y2.float(), ref[rows.long()]) < (2e-6 if ydtype == torch.float32 else 6e-3)
        K.add_rmsnorm(x2, None, w, 1e-5, y2, torch.tensor([T, -1, 0], dtype=torch.int32).cuda(), write_back=False, status=st)
        assert int(st.item()) == K.ST_BAD_ROW                     # reported, not a fault


@pytest.mark.parametrize("T,F,group,planes", [(3, 50, 0, 0), (9, 193, 0, 3), (8, 10496, 64, 5), (700, 320, 64, 0),
                                              (130, 64, 64, 1), (8, 10496, 16, 8), (600, 176, 16, 0), (5, 48, 16, 2)])
def test_swiglu(K, T, F, group, planes):
    g = torch.Generator(device="cuda").manual_seed(T + F)
    gate = torch.randn(T, F, device="cuda", generator=g) * 2
    up = torch.randn(T, F, device="cuda", generator=g)
    ref = gate.double() / (1 + torch.exp(-gate.double())) * up.double()
    gp = group or F
    gu = torch.stack([gate.view(T, F // gp, gp), up.view(T, F // gp, gp)], dim=2).reshape(T, 2 * F).contiguous()
    for dtype, tol in ((torch.float32, 2e-6), (torch.bfloat16, 1.5e-2)):
        out = torch.empty(T, F, device="cuda", dtype=dtype)
        K.swiglu(gu.to(dtype), out, group)
        assert _rel(out.float(), ref) < tol
    if planes:
        parts = torch.randn(planes, T, 2 * F, device="cuda", generator=g)
        parts[-1] = gu - parts[:-1].sum(0)
        out = torch.empty(T, F, device="cuda", dtype=torch.bfloat16)
        K.swiglu(parts.contiguous(), out, group)
        assert _rel(out.float(), ref) < 1.5e-2


@pytest.mark.parametrize("T,nh,nkv,hd,rot,planes", [(5, 3, 1, 48, 32, 0), (40, 20, 4, 128, 128, 0), (8, 20, 4, 128, 128, 5),
                                                    (33, 2, 2, 18, 6, 0), (64, 5, 1, 64, 32, 3), (36, 3, 1, 24, 12, 0),
                                                    (100, 20, 4, 128, 128, 0), (130, 5, 1, 64, 32, 3),
                                                    (97, 3, 1, 24, 12, 0), (150, 2, 2, 18, 6, 0)])
def test_rope_store_against_plain(K, T, nh, nkv, hd, rot, planes):
    """rotation of q in place or from planes, keys rotated into the cache pages, values copied; both kernels
    (one block per head for small steps, one block per row for larger ones) against the same formulas"""
    g = torch.Generator().manual_seed(T + hd)
    width = (nh + 2 * nkv) * hd
    qkv = torch.randn(T, width, generator=g)
    pos = torch.arange(100, 100 + T, dtype=torch.int32)
    i = torch.arange(rot // 2, dtype=torch.float64)
    inv = (10000.0 ** (-2 * i / rot)).float()
    ang = (pos.float()[:, None] * inv[None]).double()
    cos, sin = torch.cos(ang), torch.sin(ang)

    def rot_ref(x):                      # [T, heads, hd]
        a, b, rest = x[..., : rot // 2], x[..., rot // 2: rot], x[..., rot:]
        return torch.cat([a * cos[:, None] - b * sin[:, None], b * cos[:, None] + a * sin[:, None], rest], -1)
    n_pages = 4
    table = torch.tensor([[2, 0, 3, 1]], dtype=torch.int32).cuda()          # positions 100.. lie in blocks 1 to 3
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 6e-3)):
        given = qkv if planes else qkv.to(dtype).float()                    # what the kernel is handed
        q_ref = rot_ref(given[:, : nh * hd].double().view(T, nh, hd))
        k_ref = rot_ref(given[:, nh * hd: (nh + nkv) * hd].double().view(T, nkv, hd))
        v_ref = given[:, (nh + nkv) * hd:].double().view(T, nkv, hd)
        pool = torch.zeros(n_pages, 2, nkv, 64, hd, dtype=dtype, device="cuda")
        st = _status()
        seq = torch.zeros(T, dtype=torch.int32).cuda()
        slot = torch.zeros(1, dtype=torch.int32).cuda()
        if planes:
            if dtype == torch.float32:
                continue
            parts = torch.randn(planes, T, width, generator=g)
            parts[-1] = qkv - parts[:-1].sum(0)
            src = parts.cuda().contiguous()
            qout = torch.empty(T, nh * hd, dtype=dtype, device="cuda")
        else:
            src = qkv.to(dtype).cuda()
            qout = src
        K.rope_store(src, qout, inv.cuda(), rot, pos.cuda(), seq, slot, nh, nkv, hd, pool, table, n_pages, st)
        assert int(st.item()) == 0
        assert _rel(qout[:, : nh * hd].float().cpu().view(T, nh, hd), q_ref) < tol
        for t in range(T):
            p = 100 + t
            page = int(table[0, p // 64])
            assert _rel(pool[page, 0, :, p % 64].float().cpu(), k_ref[t]) < tol
            assert _rel(pool[page, 1, :, p % 64].float().cpu(), v_ref[t]) < tol


@pytest.mark.parametrize("kind,hd,dtype", [("generic", 48, torch.float32), ("generic", 128, torch.bfloat16),
                                           ("prefill", 64, torch.bfloat16), ("decode", 128, torch.bfloat16),
                                           ("decode", 64, torch.bfloat16), ("tc", 128, torch.bfloat16),
                                           ("tc", 64, torch.bfloat16)])
def test_attention_window_edge(K, kind, hd, dtype):
    """a key that stands out, placed on the last position a row may still see (pos - window + 1) and on the first it
    may not (pos - window): an off-by-one at the window's edge then changes the output grossly, not by a few per cent"""
    window, kv = 100, 300
    ql = 1 if kind == "decode" else 40
    row = ql - 1
    pos_row = kv - 1
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    for key in (pos_row - window + 1, pos_row - window):
        err = _run_attention(K, kind, dtype, 4, 2, hd, [ql, 1], [kv, 70], window, seed=hd + key, boost=(0, row, key))
        assert err < tol, (kind, key, err)


def test_embedding_scale_and_logit_scale_with_soft_cap(K):
    """the options of the embedding and head parts: rows times a scale; logits times a scale, then cap * tanh(z / cap)"""
    g = torch.Generator(device="cuda").manual_seed(3)
    st = _status()
    for dtype in (torch.float32, torch.bfloat16):
        table = torch.randn(53, 40, device="cuda", generator=g).to(dtype)
        tok = torch.tensor([0, 52, 7, 7, 31], dtype=torch.int32, device="cuda")
        out = torch.full((5, 40), float("nan"), device="cuda")
        K.embed(table, tok, out, st, 6.5)
        assert int(st.item()) == 0 and torch.equal(out, table.float()[tok.long()] * 6.5)
    z = torch.randn(7, 1001, device="cuda", generator=g) * 9.0
    for scale, cap in ((0.5, 0.0), (1.0, 4.0), (0.25, 30.0)):
        got = z.clone()
        K.logit_post(got, scale, cap)
        want = z.double() * scale
        if cap > 0:
            want = cap * torch.tanh(want / cap)
        assert _rel(got, want) < 1e-6
        if cap > 0:
            assert float(got.abs().max()) <= cap


def test_rotation_angles_of_a_step_are_the_kernels_own(K):
    """the cosines and sines a step computes once (rope_table) give the rotate-and-store kernel the same bits as its own
    computation, for rows and for 32-bit planes; rows with position -1 are left alone"""
    g = torch.Generator().manual_seed(11)
    T, nh, nkv, hd = 134, 5, 1, 128
    width = (nh + 2 * nkv) * hd
    qkv = torch.randn(T, width, generator=g).to(torch.bfloat16).cuda()
    pos = torch.arange(1000, 1000 + T, dtype=torch.int32)
    pos[-3:] = -1
    inv = (7e7 ** (-2 * torch.arange(hd // 2, dtype=torch.float64) / hd)).float().cuda()
    table = torch.arange(32, dtype=torch.int32)[None].contiguous().cuda()
    seq = torch.zeros(T, dtype=torch.int32).cuda()
    slot = torch.zeros(1, dtype=torch.int32).cuda()
    st = _status()
    res = []
    for use_table in (False, True):
        pool = torch.zeros(32, 2, nkv, 64, hd, dtype=torch.bfloat16, device="cuda")
        q = torch.full((T, nh * hd), 7.0, dtype=torch.bfloat16, device="cuda")
        ang = K.rope_table(pos.cuda(), inv, hd) if use_table else None
        K.rope_store(qkv.clone(), q, inv, hd, pos.cuda(), seq, slot, nh, nkv, hd, pool, table, 32, st, ang)
        assert int(st.item()) == 0
        res.append((q.clone(), pool.clone()))
    assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][1], res[1][1])
    assert bool((res[1][0][-3:] == 7.0).all())                       # padding rows: queries not written
    first_pad = 1000 + T - 3                                           # the first position that no row stores
    assert float(res[1][1][first_pad // 64, :, :, first_pad % 64:].abs().sum()) == 0.0
    assert float(res[1][1][first_pad // 64, :, :, first_pad % 64 - 1].abs().sum()) > 0.0
