"""Loading the kernel library and calling its entry points with torch tensors.

The library is plain C ABI (``extern "C"``): raw device pointers, sizes and a stream. It is loaded with ctypes from
the in-tree build folder; a missing or unbuildable library is an error, never a fallback to other code. Each
wrapper below checks what the kernel itself does not (contiguity, dtypes, size limits) and raises on a failed
launch.
"""
from __future__ import annotations

import ctypes
import functools
from ctypes import c_int, c_float, c_void_p, c_longlong
from typing import Optional

import torch

from . import build as _build

F32, BF16 = 0, 1
PAGE = 64                     # positions per cache page (KB_PAGE in csrc/common.cuh)

ST_BAD_TOKEN, ST_BAD_PAGE, ST_WAIT_TIMEOUT, ST_BAD_ROW = 1, 2, 4, 8

_lib = None


class KernelError(RuntimeError):
    pass


_SIGS = {
    "kb_embed": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    "kb_logit_post": [c_void_p, c_longlong, c_float, c_float, c_void_p],
    "kb_add_rmsnorm": [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_int, c_float, c_void_p, c_int, c_void_p,
                       c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "kb_gemm_simt": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                     c_void_p],
    "kb_rope_store": [c_void_p, c_int, c_int, c_longlong, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p,
                      c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p,
                      c_void_p, c_void_p],
    "kb_rope_table": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "kb_attn_generic": [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                        c_int, c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "kb_swiglu": [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "kb_gemm_tc": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                   c_longlong, c_void_p, c_void_p, c_int, c_int],
    "kb_gemm_tc_splits": [c_int, c_int],
    "kb_rope_table_min_rows": [],
    "kb_gemm_pair": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                     c_void_p, c_int, c_void_p, c_void_p],
    "kb_gemm_swiglu_decode": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                              c_void_p, c_void_p, c_void_p],
    "kb_attn_mma": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                    c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "kb_attn_decode_rope": [c_void_p, c_int, c_longlong, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_int, c_void_p,
                            c_int, c_int, c_int, c_void_p, c_void_p],
    "kb_attn_tc": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float,
                   c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    "kb_sample": [c_void_p, c_longlong, c_int, c_int, c_float, c_int, c_float, c_float, c_int, c_void_p, c_void_p,
                  c_void_p],
    "kb_penalize": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_int, c_float, c_void_p],
    "kb_wait_selftest": [ctypes.c_ulonglong, c_void_p, c_void_p, c_void_p],
}


def load(verbose: bool = True):
    """build (when needed) and load the kernel library; raises when that is not possible"""
    global _lib
    if _lib is not None:
        return _lib if _timing is None else _timing
    path = _build.library_path(build=True, verbose=verbose)
    lib = ctypes.CDLL(path)
    for name, args in _SIGS.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            raise KernelError("kindi_b200: the kernel library %s lacks %s" % (path, name))
        fn.argtypes = args
        fn.restype = c_int
    lib.kb_set_pdl.argtypes = [c_int]
    lib.kb_set_pdl.restype = None
    lib._path = path
    _lib = lib
    return lib


# ----------------------------------------------------------------------------------------------- per-kernel timing
_timing = None

# where an entry point's product sizes stand among its arguments (N, K), for the label of a timed launch
_GEMM_NK = {"kb_gemm_tc": (5, 6), "kb_gemm_pair": (5, 6), "kb_gemm_simt": (7, 8), "kb_gemm_swiglu_decode": (4, 5)}


class KernelTiming:
    """``with KernelTiming() as t: engine.step(...)``: every launch of the library inside the block is bracketed by
    CUDA events on the launching stream; ``t.summary()`` gives, per kind of launch (entry point, with the product's
    sizes for matrix products), the number of launches and the device time in microseconds. Meant for steps that are
    issued launch by launch (a recorded step is one launch to the host); the events themselves cost the device a
    microsecond or two per launch, so compare shares."""

    def __init__(self):
        self.records = []

    def __getattr__(self, name):                       # stands in for the library while timing is on
        fn = getattr(_lib, name)
        if not name.startswith("kb_") or name in ("kb_set_pdl", "kb_gemm_tc_splits", "kb_rope_table_min_rows"):
            return fn

        def timed(*args):
            label = name[3:]
            if name in _GEMM_NK:
                n, k = _GEMM_NK[name]
                label += " %dx%d" % ((2 * args[n], args[k]) if name == "kb_gemm_swiglu_decode" else (args[n], args[k]))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            rc = fn(*args)
            e1.record()
            self.records.append((label, e0, e1))
            return rc
        return timed

    def __enter__(self):
        global _timing
        load()
        _timing = self
        return self

    def __exit__(self, *exc):
        global _timing
        _timing = None
        return False

    def summary(self):
        torch.cuda.synchronize()
        out = {}
        for label, e0, e1 in self.records:
            d = out.setdefault(label, {"launches": 0, "us": 0.0})
            d["launches"] += 1
            d["us"] += e0.elapsed_time(e1) * 1000.0
        return {k: {"launches": v["launches"], "us": round(v["us"], 1)} for k, v in out.items()}


def set_pdl(on: bool) -> None:
    """launch kernels with programmatic dependent launch (the default) or strictly one after another"""
    load().kb_set_pdl(1 if on else 0)


def library_file() -> str:
    return load()._path


_launches = 0


def launch_count() -> int:
    """kernels of this library launched so far (replays of a recorded step count the launches they hold)"""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(rc: int, what: str) -> None:
    global _launches
    _launches += 1
    if rc != 0:
        raise KernelError("kindi_b200: launching %s failed with CUDA error %d (%s)"
                          % (what, rc, _err_name(rc)))


def _err_name(rc: int) -> str:
    try:
        return torch.cuda.cudart().cudaGetErrorString(rc)      # type: ignore[attr-defined]
    except Exception:                                          # noqa: BLE001
        return "?"


def dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError("kindi_b200: tensors must be float32 or bfloat16, found %s" % t.dtype)


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None) or torch.cuda.current_device


def _stream():
    """the current stream's handle (asked of torch directly: building a Stream object costs several microseconds,
    which a step of a hundred launches feels)"""
    if _raw_stream is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("kindi_b200: the kernels run on the GPU only; a tensor lives on %s" % t.device)


# ----------------------------------------------------------------------------------------------- wrappers
def embed(table: torch.Tensor, tok: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
          scale: float = 1.0) -> None:
    """out[t] (float32 [T, E]) = table[tok[t]] * scale"""
    _need_cuda(table, tok, out)
    T, E = out.shape
    assert table.is_contiguous() and out.is_contiguous() and out.dtype == torch.float32 and tok.dtype == torch.int32
    _check(load().kb_embed(_p(table), dt(table), _p(tok), _p(out), T, E, table.shape[0], float(scale), _p(status),
                           _stream()), "embed")


def wait_selftest(status: torch.Tensor, limit_ns: int = 1_000_000):
    """run the library's bounded wait on a barrier that nothing arrives at: it gives up after ``limit_ns`` (at most a
    tenth of a second), sets ST_WAIT_TIMEOUT in ``status`` and the kernel ends. Returns (timed out, nanoseconds waited)
    once the kernel has finished"""
    _need_cuda(status)
    out = torch.zeros(2, dtype=torch.int64, device=status.device)
    _check(load().kb_wait_selftest(int(limit_ns), _p(out), _p(status), _stream()), "wait_selftest")
    r = out.tolist()
    return bool(r[0]), int(r[1])


def logit_post(logits: torch.Tensor, scale: float = 1.0, softcap: float = 0.0) -> None:
    """logits (float32, contiguous) *= scale, then softcap * tanh(logits / softcap) when softcap > 0; in place"""
    _need_cuda(logits)
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    _check(load().kb_logit_post(_p(logits), logits.numel(), float(scale), float(softcap), _stream()), "logit_post")


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], w: torch.Tensor, eps: float, out: torch.Tensor,
                rows: Optional[torch.Tensor], write_back: bool, status: torch.Tensor) -> None:
    """x (float32 [T, E]) + sum of delta ([S, T, E] float32) -> RMS norm * w -> out ([R, E]); rows int32 or None"""
    _need_cuda(x, delta, w, out, rows)
    T, E = x.shape
    n_out = out.shape[0]
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and w.shape == (E,)
    nd, stride = 0, 0
    if delta is not None:
        assert delta.dtype == torch.float32 and delta.is_contiguous() and delta.shape[1:] == (T, E)
        nd, stride = delta.shape[0], T * E
    if rows is None:
        assert n_out == T
    else:
        assert rows.dtype == torch.int32 and rows.numel() == n_out
    if E * 4 > 200 * 1024:
        raise KernelError("kindi_b200: RMS norm supports a width up to 51200, found %d" % E)
    _check(load().kb_add_rmsnorm(_p(x), _p(delta), nd, stride, _p(w), dt(w), float(eps), _p(out), dt(out), _p(rows),
                                 n_out, T, E, 1 if write_back else 0, _p(status), _stream()), "add_rmsnorm")


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T with 32-bit accumulation in a fixed order (no tensor cores)"""
    _need_cuda(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(load().kb_gemm_simt(_p(a), dt(a), _p(w), dt(w), _p(out), dt(out), M, N, K, a.stride(0), w.stride(0),
                               out.stride(0), _stream()), "gemm_simt")


@functools.lru_cache(maxsize=1)
def rope_table_min_rows() -> int:
    """steps of fewer rows are rotated by kernels that compute their angles themselves and read no table"""
    return load().kb_rope_table_min_rows()


def rope_table(pos: torch.Tensor, inv_freq: torch.Tensor, rot: int) -> torch.Tensor:
    """(cos, sin) of float(pos[t]) * inv_freq[i] for every row and rotated pair: float32 [T, rot / 2, 2]. The angles of
    a step are the same in every layer, so a step makes this once and hands it to ``rope_store``"""
    _need_cuda(pos, inv_freq)
    T = pos.numel()
    assert pos.dtype == torch.int32 and inv_freq.dtype == torch.float32 and rot % 2 == 0
    assert inv_freq.numel() >= max(1, rot // 2)
    out = torch.empty((T, rot // 2, 2), dtype=torch.float32, device=pos.device)
    _check(load().kb_rope_table(_p(pos), _p(inv_freq), rot, T, _p(out), _stream()), "rope_table")
    return out


def rope_store(qkv: torch.Tensor, qout: torch.Tensor, inv_freq: torch.Tensor, rot: int, pos, seq, slot, nh: int,
               nkv: int, hd: int, pool: Optional[torch.Tensor], table: torch.Tensor, n_pages: int,
               status: torch.Tensor, angles: Optional[torch.Tensor] = None) -> None:
    """qkv: [T, (nh + 2 nkv) hd], or 32-bit planes [S, T, ...] that are summed. Query heads are rotated into qout
    ([T, >= nh hd]; may be qkv itself), keys are rotated and stored in the cache, values are stored. ``angles``: what
    ``rope_table`` made for these rows (optional: without it the kernel computes the cosines and sines itself)"""
    _need_cuda(qkv, qout, inv_freq, pool, table)
    planes = qkv.shape[0] if qkv.dim() == 3 else 1
    T = qkv.shape[-2]
    assert qkv.stride(-1) == 1 and inv_freq.dtype == torch.float32 and inv_freq.numel() >= max(1, rot // 2)
    assert rot % 2 == 0 and rot <= hd and qout.stride(1) == 1
    if pool is not None:
        assert pool.dtype == qout.dtype and pool.is_contiguous()
    pstride = qkv.stride(0) if qkv.dim() == 3 else 0
    if angles is not None:
        assert angles.dtype == torch.float32 and angles.is_contiguous() and angles.shape == (T, rot // 2, 2)
    _check(load().kb_rope_store(_p(qkv), dt(qkv), planes, pstride, qkv.stride(-2), _p(qout), dt(qout),
                                qout.stride(0), _p(inv_freq), rot, _p(pos), _p(seq), _p(slot), T, nh, nkv, hd,
                                _p(pool), _p(table), table.stride(0), n_pages, _p(status), _stream(), _p(angles)),
           "rope_store")


def attn_generic(q: torch.Tensor, out: torch.Tensor, pos, seq, slot, nh: int, nkv: int, hd: int, scale: float,
                 window: int, pool: torch.Tensor, table: torch.Tensor, n_pages: int, status: torch.Tensor) -> None:
    """attention of each row of q ([T, >= nh hd], row stride free) over its sequence's cached keys and values"""
    _need_cuda(q, out, pool, table)
    T = q.shape[0]
    if hd > 256:
        raise KernelError("kindi_b200: attention supports head sizes up to 256, found %d" % hd)
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == pool.dtype
    _check(load().kb_attn_generic(_p(q), dt(q), q.stride(0), _p(out), out.stride(0), _p(pos), _p(seq), _p(slot), T,
                                  nh, nkv, hd, float(scale), int(window), _p(pool), _p(table), table.stride(0),
                                  n_pages, _p(status), _stream()), "attn_generic")


def swiglu(gu: torch.Tensor, out: torch.Tensor, group: int = 0) -> None:
    """out[T, F] = silu(g) * u with gu [T, 2F] (or the sum of 32-bit planes gu [S, T, 2F]). The columns of gu come in
    groups of ``group`` gate columns followed by the ``group`` up columns of the same outputs (0: all gates, then
    all ups)"""
    _need_cuda(gu, out)
    T, F = out.shape
    planes = gu.shape[0] if gu.dim() == 3 else 1
    assert gu.shape[-2:] == (T, 2 * F) and gu.is_contiguous() and out.is_contiguous()
    _check(load().kb_swiglu(_p(gu), dt(gu), planes, T * 2 * F, _p(out), dt(out), T, F, group or F, _stream()),
           "swiglu")


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, swap: bool, bn: int, splits: int,
            status: torch.Tensor, swiglu: bool = False, mt: int = 1) -> None:
    """out = a[M, K] @ w[N, K]^T on the tensor cores (bf16 in, fp32 accumulate). ``out`` is [M, N] (bf16 or fp32)
    or, with K splits, fp32 [S, M, N] where S = gemm_tc_splits(K, splits). ``swiglu`` (prefill form, bn a multiple
    of 32): w holds 16 gate rows then the 16 up rows of the same outputs, group after group, and ``out`` is the bf16
    [M, N / 2] result silu(gate) * up. ``mt`` = 2 (prefill form): a unit is two 128-row tiles over the same columns"""
    _need_cuda(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == K
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.is_contiguous()
    if swiglu:
        assert out.shape == (M, N // 2) and out.dtype == torch.bfloat16 and not swap and splits == 1 and N % 32 == 0 and bn % 32 == 0
        stride, ldc = 0, N // 2
    elif out.dim() == 3:
        assert out.shape == (gemm_tc_splits(K, splits), M, N) and out.dtype == torch.float32
        stride, ldc = M * N, N
    else:
        assert out.shape == (M, N) and splits == 1
        stride, ldc = 0, N
    _check(load().kb_gemm_tc(_p(a), _p(w), _p(out), dt(out), M, N, K, a.stride(0), w.stride(0), ldc, 1 if swap else 0,
                             bn, splits, stride, _p(status), _stream(), 1 if swiglu else 0, mt), "gemm_tc")


def gemm_pair(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, bn: int, status: torch.Tensor,
              swiglu: bool = False, part: Optional[torch.Tensor] = None, flags: Optional[torch.Tensor] = None) -> None:
    """out = a[M, K] @ w[N, K]^T by pairs of SMs (tcgen05 with cta_group::2: a pair computes 256 rows x bn columns,
    each CTA holding half of the weight tile), bf16 in, fp32 accumulate, ``out`` [M, N] bf16 or fp32; bn 64, 128, 192
    or 256. ``swiglu``: as for gemm_tc, ``out`` is the bf16 [M, N / 2] result silu(gate) * up. With ``part`` (fp32, at
    least tiles * 256 * bn elements, tiles = ceil(M / 256) * ceil(N / bn)) and ``flags`` (int32 zeros, 8 a tile) the
    K blocks of all tiles are dealt out evenly to the pairs and a tile may be finished by two of them"""
    _need_cuda(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == K
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.is_contiguous() and bn in (64, 128, 192, 256)
    if swiglu:
        assert out.shape == (M, N // 2) and out.dtype == torch.bfloat16 and N % 32 == 0
        ldc = N // 2
    else:
        assert out.shape == (M, N)
        ldc = N
    if part is not None:
        tiles = -(-M // 256) * -(-N // bn)
        assert part.dtype == torch.float32 and part.numel() >= tiles * 256 * bn and part.is_contiguous()
        assert flags.dtype == torch.int32 and flags.numel() >= 8 * tiles and flags.is_contiguous()
    _check(load().kb_gemm_pair(_p(a), _p(w), _p(out), dt(out), M, N, K, a.stride(0), w.stride(0), ldc, bn, _p(status),
                               _stream(), 1 if swiglu else 0, _p(part), _p(flags)), "gemm_pair")


def gemm_swiglu_decode(a: torch.Tensor, w_grouped: torch.Tensor, out: torch.Tensor, bn: int, part: torch.Tensor,
                       flags: torch.Tensor, status: torch.Tensor) -> None:
    """out (bf16 [M, F]) = silu(g) * u with [g | u] = a[M, K] @ w_grouped[2F, K]^T (16 gate rows, then the 16 up rows
    of the same outputs), for M <= bn rows, SwiGLU finished inside the product. ``part`` (float32, at least
    ceil(2F / 128) * bn * 128) and ``flags`` (int32 zeros, at least ceil(2F / 128)) are scratch that calls on one
    stream may share"""
    _need_cuda(a, w_grouped, out, part, flags)
    M, K = a.shape
    F = w_grouped.shape[0] // 2
    tiles = -(-2 * F // 128)
    assert a.dtype == w_grouped.dtype == out.dtype == torch.bfloat16 and w_grouped.shape == (2 * F, K)
    assert a.stride(1) == 1 and w_grouped.stride(1) == 1 and out.shape == (M, F) and out.stride(1) == 1
    assert F % 16 == 0 and M <= bn and part.dtype == torch.float32 and part.numel() >= tiles * bn * 128
    assert flags.dtype == torch.int32 and flags.numel() >= tiles
    _check(load().kb_gemm_swiglu_decode(_p(a), _p(w_grouped), _p(out), M, F, K, a.stride(0), w_grouped.stride(0),
                                        out.stride(0), bn, _p(part), _p(flags), _p(status), _stream()),
           "gemm_swiglu_decode")


@functools.lru_cache(maxsize=4096)
def gemm_tc_splits(K: int, wanted: int) -> int:
    return load().kb_gemm_tc_splits(K, wanted)


def attn_mma(q: torch.Tensor, out: torch.Tensor, slot, q_start, kv_len, B: int, nh: int, nkv: int, hd: int,
             scale: float, window: int, pool: torch.Tensor, table: torch.Tensor, n_pages: int, *, decode: bool,
             grid_x: int, status: torch.Tensor) -> None:
    """tensor-core attention over the cache (bf16, head size 64 or 128). decode: one row per sequence, grid_x =
    position splits; else grid_x = ceil(most rows of a sequence * (nh / nkv) / 64)"""
    _need_cuda(q, out, pool, table)
    assert q.dtype == out.dtype == pool.dtype == torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    assert pool.is_contiguous()
    part_o = part_ml = None
    if decode and grid_x > 1:
        part_o = torch.empty((B, nh, grid_x, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((B, nh, grid_x, 2), dtype=torch.float32, device=q.device)
    _check(load().kb_attn_mma(_p(q), q.stride(0), _p(out), out.stride(0), _p(part_o), _p(part_ml), _p(slot),
                              _p(q_start), _p(kv_len), B, nh, nkv, hd, float(scale), int(window), _p(pool), _p(table),
                              table.stride(0), n_pages, 1 if decode else 0, grid_x, _p(status), _stream()),
           "attn_mma")
    if decode and grid_x > 1:
        add_launches(1)         # the merge of the position splits


def attn_decode_rope(qkv: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor, slot, q_start, kv_len, B: int,
                     nh: int, nkv: int, hd: int, scale: float, window: int, pool: torch.Tensor, store: bool,
                     table: torch.Tensor, n_pages: int, *, grid_x: int, status: torch.Tensor) -> None:
    """decode attention that takes the QKV product as 32-bit planes [S, rows, (nh + 2 nkv) hd], rotates the queries
    and the newest key over the whole head, stores the newest key and value (``store``) and attends; grid_x =
    position splits"""
    _need_cuda(qkv, out, pool, table, inv_freq)
    assert qkv.dtype == torch.float32 and qkv.dim() == 3 and qkv.stride(2) == 1 and qkv.stride(1) == qkv.shape[2]
    assert out.dtype == pool.dtype == torch.bfloat16 and out.stride(1) == 1 and pool.is_contiguous()
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() == hd // 2
    part_o = part_ml = None
    if grid_x > 1:
        part_o = torch.empty((B, nh, grid_x, hd), dtype=torch.float32, device=out.device)
        part_ml = torch.empty((B, nh, grid_x, 2), dtype=torch.float32, device=out.device)
    _check(load().kb_attn_decode_rope(_p(qkv), qkv.shape[0], qkv.stride(0), qkv.stride(1), _p(inv_freq), _p(out),
                                      out.stride(0), _p(part_o), _p(part_ml), _p(slot), _p(q_start), _p(kv_len), B, nh,
                                      nkv, hd, float(scale), int(window), _p(pool), 1 if store else 0, _p(table),
                                      table.stride(0), n_pages, grid_x, _p(status), _stream()), "attn_decode_rope")
    if grid_x > 1:
        add_launches(1)         # the merge of the position splits


def attn_tc(q: torch.Tensor, out: torch.Tensor, slot, q_start, kv_len, B: int, nh: int, nkv: int, hd: int,
            scale: float, window: int, pool: torch.Tensor, table: torch.Tensor, n_pages: int, *, grid_x: int,
            status: torch.Tensor) -> None:
    """tcgen05 attention for prompt-sized steps (bf16, head size 64 or 128): grid_x = ceil(most rows of a sequence /
    (128 // (nh / nkv)))"""
    _need_cuda(q, out, pool, table)
    assert q.dtype == out.dtype == pool.dtype == torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    assert pool.is_contiguous() and hd in (64, 128)
    _check(load().kb_attn_tc(_p(q), q.stride(0), _p(out), out.stride(0), _p(slot), _p(q_start), _p(kv_len), B, nh, nkv,
                             hd, float(scale), int(window), _p(pool), _p(table), table.stride(0), n_pages, grid_x,
                             _p(status), _stream()), "attn_tc")
