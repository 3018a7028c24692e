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


def _call(lib, case, out, scale, n_splits=4, max_kv_len=512, rows=None, n_rows=None, n_heads=6, n_kv=3, d=64, page=16,
          pps=None):
    pages = -(-max_kv_len // 16)
    if pps is None:
        pps = -(-pages // n_splits)
        n_splits = -(-pages // pps)
    p = lambda t: c_void_p(0 if t is None else t.data_ptr())
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib.tnx_attention_decode_noalloc(
        p(case.q_flat), c_int(case.q_flat.stride(0)), p(case.cache), p(case.bt), c_int(case.bt.stride(0)),
        p(rows), p(case.tok_req), p(case.positions), p(out), c_int(out.stride(0)),
        c_int(case.N if n_rows is None else n_rows), c_int(n_heads), c_int(n_kv), c_int(d), c_int(page), c_int(0),
        c_float(scale), c_int(n_splits), c_int(pps), stream)


@pytest.mark.parametrize("n_splits", [4, 1])
def test_matches_the_allocating_entry_point_twice_in_a_row(n_splits):
    """Two calls back to back on one stream (they share the built-in scratch: the second starts from
    what the first left), compared after a single synchronisation with the allocating entry point
    and with the plain attention; with several splits (the scratch is used) and with one (it is not)."""
    from transformers_neuronx_b200.kernels import ops
    lib = _lib()
    scale = 1.0 / math.sqrt(64)
    cases = [_case(21), _case(22)]
    got = [torch.zeros(c.N, 6 * 64, dtype=torch.bfloat16, device=DEV) for c in cases]
    for c, g in zip(cases, got):
        assert _call(lib, c, g, scale, n_splits=n_splits) == 0, lib.tnx_attention_decode_noalloc_last_error()
    torch.cuda.synchronize()
    assert lib.tnx_attention_decode_noalloc_last_error() == b""
    for c, g in zip(cases, got):
        want = torch.zeros_like(g)
        ops.attention_decode(c.q_flat, c.cache, c.bt, c.tok_req, c.positions, want, 6, scale, 0, max_kv_len=512,
                             n_splits=n_splits)
        torch.cuda.synchronize()
        assert float((g.float() - want.float()).abs().max()) / float(want.float().abs().max()) <= 1e-2
        plain = c.want(scale, None)
        assert float((g.float() - plain).abs().max()) / float(plain.abs().max()) <= 1e-2


def test_a_row_list_with_a_padded_entry():
    """Rows named by a list, one entry of which is -1 (the padding of a batch of fixed size): only the
    named rows are written."""
    lib = _lib()
    scale = 1.0 / math.sqrt(64)
    case = _case(24)
    rows = torch.tensor([3, -1, 0, 4], dtype=torch.int32, device=DEV)
    out = torch.zeros(case.N, 6 * 64, dtype=torch.bfloat16, device=DEV)
    assert _call(lib, case, out, scale, rows=rows, n_rows=4) == 0, lib.tnx_attention_decode_noalloc_last_error()
    torch.cuda.synchronize()
    plain = case.want(scale, None)
    named = torch.tensor([3, 0, 4], device=DEV)
    assert float((out[named].float() - plain[named]).abs().max()) / float(plain[named].abs().max()) <= 1e-2
    assert float(out[torch.tensor([1, 2], device=DEV)].float().abs().max()) == 0.0


def test_refusals_say_why_and_run_nothing():
    lib = _lib()
    case = _case(23)
    out = torch.zeros(case.N, 6 * 64, dtype=torch.bfloat16, device=DEV)
    msg = lambda: lib.tnx_attention_decode_noalloc_last_error().decode()
    # sizes beyond the built-in scratch
    assert _call(lib, case, out, 0.1, n_splits=8, pps=16, n_rows=4096, n_heads=64, n_kv=64, d=128) == -2
    assert "exceed" in msg() and "floats" in msg()
    # counts that are not positive; heads that the key/value heads do not divide; sizes the kernel does not take
    assert _call(lib, case, out, 0.1, n_splits=2, pps=0) == -1 and "pages_per_split" in msg()
    assert _call(lib, case, out, 0.1, n_heads=6, n_kv=4) == -1 and "multiple of n_kv_heads" in msg()
    assert _call(lib, case, out, 0.1, page=32) == -2 and "page_size must be 16" in msg()
    assert _call(lib, case, out, 0.1, d=72) == -2 and "head_dim" in msg()
    torch.cuda.synchronize()
    assert float(out.float().abs().max()) == 0.0            # nothing ran
    assert _call(lib, case, out, 1.0 / 8) == 0 and msg() == ""
    torch.cuda.synchronize()
    assert float(out.float().abs().max()) > 0.0
