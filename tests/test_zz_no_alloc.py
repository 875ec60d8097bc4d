"""The entry point that allocates nothing, kb_attn_decode_static, called through its exported C symbol.

Who needs it: a host that may not allocate device memory while it runs (a plug-in inside another program's CUDA
context with a fixed memory limit, a real-time loop, a process whose memory pool belongs to somebody else). The usual
decode attention (kb_attn_mma) takes the scratch for its position splits from its caller; this one keeps it in a
static device array of the library (4 MiB per GPU). The test checks, on two calls in a row with different inputs,
that it gives what the usual entry point gives with scratch from the allocator, that device memory in use does not
change across a call, and that a call too large for the array is refused without launching anything.

This file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(lengths, nh, nkv, hd, seed):
    from test_kernels_gpu import _make_cache
    pool, table, dense, slots, n_pages = _make_cache(lengths, nkv, hd, torch.bfloat16, seed)
    B = len(lengths)
    g = torch.Generator().manual_seed(seed + 100)
    q = torch.randn(B, nh * hd, generator=g).to(torch.bfloat16).cuda()
    q_start = torch.arange(B + 1, dtype=torch.int32).cuda()
    kv_len = torch.tensor(lengths, dtype=torch.int32).cuda()
    return q, pool, table, slots, n_pages, q_start, kv_len


def test_static_scratch_entry_point_matches_the_allocating_one():
    from kindi_b200.kernels import lib as K
    dll = ctypes.CDLL(K.library_file())
    fn = dll.kb_attn_decode_static
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float,
                   c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]
    nh, nkv, hd = 20, 4, 128
    scale = 1.0 / math.sqrt(hd)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def both(lengths, splits, seed, window):
        q, pool, table, slots, n_pages, q_start, kv_len = _inputs(lengths, nh, nkv, hd, seed)
        B = len(lengths)
        want = torch.full((B, nh * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
        K.attn_mma(q, want, slots, q_start, kv_len, B, nh, nkv, hd, scale, window, pool, table, n_pages, decode=True,
                   grid_x=splits, status=status)
        got = torch.full((B, nh * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        used, free = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        rc = fn(q.data_ptr(), q.stride(0), got.data_ptr(), got.stride(0), slots.data_ptr(), q_start.data_ptr(),
                kv_len.data_ptr(), B, nh, nkv, hd, scale, window, pool.data_ptr(), table.data_ptr(), table.stride(0),
                n_pages, splits, status.data_ptr(), stream)
        torch.cuda.synchronize()
        assert rc == 0 and int(status.item()) == 0
        return got, want, (used, free), (torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0])

    # first call on this device: it also looks up the array's address
    got, want, _, _ = both([1, 64, 65, 700, 129, 320], splits=5, seed=21, window=0)
    assert not torch.isnan(got.float()).any()
    err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
    assert err < 1e-2 and torch.equal(got, want)                  # the same kernels: in fact bit for bit
    # second call, straight after, other inputs and fewer splits: nothing of the first call's scratch may show
    got, want, before, after = both([900, 33, 2, 200], splits=3, seed=22, window=150)
    err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
    assert err < 1e-2 and torch.equal(got, want)
    assert before == after                                        # no device memory was taken or given back
    # too large for the static array: refused, nothing launched
    q, pool, table, slots, n_pages, q_start, kv_len = _inputs([10] * 64, 128, 8, hd, 23)
    out = torch.full((64, 128 * hd), 7.0, dtype=torch.bfloat16, device="cuda")
    rc = fn(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), slots.data_ptr(), q_start.data_ptr(),
            kv_len.data_ptr(), 64, 128, 8, hd, scale, 0, pool.data_ptr(), table.data_ptr(), table.stride(0), n_pages,
            64, status.data_ptr(), stream)
    torch.cuda.synchronize()
    assert rc == 1 and bool((out == 7.0).all())                   # cudaErrorInvalidValue; the output is untouched
