"""The decode-attention entry point that allocates nothing, called through its exported C symbol
as a host without this package's Python layer would call it, against the regular entry point.

Why it exists: some users of the library cannot allocate device memory when they need the kernel
(all memory already given to a cache pool; a loop that must not synchronise; a foreign runtime
that only sees C symbols), so the scratch memory of the split-KV form is built into the library.
This file is collected last so that a failure here cannot hide another test's result.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _lib():
    from transformers_neuronx_b200.kernels import build
    lib = ctypes.CDLL(build.build("attention_decode"))        # the exported symbols, nothing else
    lib.tnx_attention_decode_noalloc_last_error.restype = ctypes.c_char_p
    return lib


def _case(seed):
    from test_kernels_gpu import PagedCase
    lens = [(0, 1), (31, 1), (250, 1), (511, 1), (77, 1)]
    return PagedCase(lens, n_heads=6, n_kv=3, d=64, dtype=torch.bfloat16, seed=seed)


def _call(lib, case, out, n_splits, max_kv_len, scale):
    pages = -(-max_kv_len // 16)
    pps = -(-pages // n_splits)
    n_splits = -(-pages // pps)
    p = lambda t: c_void_p(t.data_ptr())
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib.tnx_attention_decode_noalloc(
        p(case.q_flat), c_int(case.q_flat.stride(0)), p(case.cache), p(case.bt), c_int(case.bt.stride(0)),
        c_void_p(0), p(case.tok_req), p(case.positions), p(out), c_int(out.stride(0)), c_int(case.N), c_int(6),
        c_int(3), c_int(64), c_int(16), c_int(0), c_float(scale), c_int(n_splits), c_int(pps), stream), n_splits


def test_matches_the_allocating_entry_point_twice_in_a_row():
    from transformers_neuronx_b200.kernels import ops
    lib = _lib()
    scale = 1.0 / math.sqrt(64)
    for seed in (21, 22):                                   # two calls in a row share the built-in scratch
        case = _case(seed)
        got = torch.zeros(case.N, 6 * 64, dtype=torch.bfloat16, device=DEV)
        rc, n_splits = _call(lib, case, got, n_splits=4, max_kv_len=512, scale=scale)
        assert rc == 0, lib.tnx_attention_decode_noalloc_last_error()
        want = torch.zeros_like(got)
        ops.attention_decode(case.q_flat, case.cache, case.bt, case.tok_req, case.positions, want, 6, scale, 0,
                             max_kv_len=512, n_splits=n_splits)
        torch.cuda.synchronize()
        err = float((got.float() - want.float()).abs().max()) / float(want.float().abs().max())
        assert err <= 1e-2
        plain = case.want(scale, None)
        assert float((got.float() - plain).abs().max()) / float(plain.abs().max()) <= 1e-2
    assert lib.tnx_attention_decode_noalloc_last_error() == b""


def test_sizes_beyond_the_built_in_scratch_are_refused():
    lib = _lib()
    case = _case(23)
    out = torch.zeros(case.N, 6 * 64, dtype=torch.bfloat16, device=DEV)
    p = lambda t: c_void_p(t.data_ptr())
    rc = lib.tnx_attention_decode_noalloc(
        p(case.q_flat), c_int(case.q_flat.stride(0)), p(case.cache), p(case.bt), c_int(case.bt.stride(0)),
        c_void_p(0), p(case.tok_req), p(case.positions), p(out), c_int(out.stride(0)),
        c_int(4096), c_int(64), c_int(64), c_int(128), c_int(16), c_int(0), c_float(0.1), c_int(8), c_int(16),
        c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -2
    msg = lib.tnx_attention_decode_noalloc_last_error().decode()
    assert "exceed" in msg and "floats" in msg
    torch.cuda.synchronize()
    assert float(out.float().abs().max()) == 0.0            # nothing ran
