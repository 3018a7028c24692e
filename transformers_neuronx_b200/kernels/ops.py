"""Python faces of the CUDA entry points: they check devices, types, shapes and strides, then pass
raw pointers and the current CUDA stream.  Nothing here computes; there is no fallback: on a tensor
that is not on a CUDA device every function raises."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p
from typing import Optional

import torch

from . import build as _build

_ERRORS = {-1: "bad argument", -2: "unsupported size", -3: "a bounded wait inside the kernel ran out"}


class KernelError(RuntimeError):
    pass


_launches = 0


def launch_count() -> int:
    """How many of this package's kernels have been launched by this process (kernels replayed
    from a CUDA graph are added by the code that replays it)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += int(n)


def _check(code: int, what: str) -> None:
    global _launches
    if code == 0:
        _launches += 1
        return
    if code < 0:
        raise KernelError(f"{what}: {_ERRORS.get(code, 'error')} (code {code})")
    raise KernelError(f"{what}: CUDA error {code} at launch")


_scoped_stream = None


def _stream() -> c_void_p:
    if _scoped_stream is not None:
        return _scoped_stream
    return c_void_p(torch.cuda.current_stream().cuda_stream)


class stream_scope:
    """Looks the current CUDA stream up once for all kernel launches inside the block (asking torch
    for it costs a few microseconds per launch, which a model step of a few tokens notices).  Enter
    it where the stream is already the one to launch on, e.g. inside a graph capture."""

    def __enter__(self):
        global _scoped_stream
        self._prev = _scoped_stream
        _scoped_stream = c_void_p(torch.cuda.current_stream().cuda_stream)
        return self

    def __exit__(self, *exc):
        global _scoped_stream
        _scoped_stream = self._prev
        return False


def _p(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, name: str, dtype=None, ndim=None, contiguous=True) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor: the engine has no CPU path")
    if dtype is not None:
        ok = t.dtype in dtype if isinstance(dtype, (tuple, list)) else t.dtype == dtype
        if not ok:
            raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name} has {t.dim()} dimensions, expected {ndim}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


_H16 = (torch.bfloat16, torch.float16)          # the 16-bit types: one library flavour each (kernels/build.py)
_FLOATS = (torch.float32,) + _H16

# Activations a product's epilogue applies, by the names the reference looks up
# (src/transformers_neuronx/hlo.py:485-501 -> activations.py) -> the kernels' codes (csrc/common.cuh).
ACTIVATIONS = {None: 0, "none": 0, "relu": 1, "gelu_new": 2, "gelu_new_legacy": 2, "gelu_pytorch_tanh": 2,
               "silu": 3, "swish": 3, "sigmoid": 4, "gelu": 5}


def activation_code(name) -> int:
    if name not in ACTIVATIONS:
        raise KernelError(f"activation {name!r} is not built into the products' epilogues; "
                          f"available: {sorted(k for k in ACTIVATIONS if k)}")
    return ACTIVATIONS[name]


def _is_h16(t: torch.Tensor) -> int:
    return 1 if t.dtype in _H16 else 0


def _lib(name: str, *tensors):
    """The library `name` in the flavour of the 16-bit type among `tensors` (they must agree)."""
    kinds = {t.dtype for t in tensors if t is not None and t.dtype in _H16}
    if len(kinds) > 1:
        raise KernelError(f"{name}: bfloat16 and float16 tensors in one call")
    return _build.load(name, next(iter(kinds)) if kinds else None)


def _rows_2d(t: torch.Tensor, name: str):
    """A 2-D tensor whose rows are contiguous (a column slice of a wider buffer is allowed)."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{name} must be 2-D with contiguous rows")
    return t.shape[0], t.shape[1], t.stride(0)


# ---------------------------------------------------------------------------------------------
def embed(tok_table, pre, ids, pos_table, positions, pos_offset, out_f32, out_act):
    """out[n] = (tok_table[ids[n]] or pre[n]) + pos_table[positions[n] + pos_offset]."""
    lib = _lib("embedding", tok_table, pos_table, out_act)
    N = ids.shape[0]
    _need(ids, "ids", torch.int32, 1)
    ref = out_f32 if out_f32 is not None else out_act
    H = ref.shape[1]
    table_bf16 = 0
    if tok_table is not None:
        _need(tok_table, "tok_table", _FLOATS, 2)
        if tok_table.shape[1] != H:
            raise KernelError("tok_table width differs from the output width")
        table_bf16 = _is_h16(tok_table)
    else:
        _need(pre, "pre", torch.float32, 2)
    if pos_table is not None:
        _need(pos_table, "pos_table", _FLOATS, 2)
        _need(positions, "positions", torch.int32, 1)
        if tok_table is not None and pos_table.dtype != tok_table.dtype:
            raise KernelError("token and position tables must have one dtype")
        table_bf16 = _is_h16(pos_table)
        if pos_table.shape[1] != H:
            raise KernelError("pos_table width differs from the output width")
    if out_f32 is not None:
        _need(out_f32, "out_f32", torch.float32, 2)
    act_bf16 = 0
    if out_act is not None:
        _need(out_act, "out_act", _FLOATS, 2)
        act_bf16 = _is_h16(out_act)
    _check(lib.tnx_embed(_p(tok_table), _p(pre), _p(ids), _p(pos_table), _p(positions), c_int(pos_offset),
                         _p(out_f32), _p(out_act), c_int(N), c_int(H), c_int(table_bf16), c_int(act_bf16),
                         _stream()), "embed")


def patch_tokens(tokens, src, sampled):
    """tokens[i] = sampled[src[i]] wherever src[i] >= 0 (all int32, on the device)."""
    lib = _build.load("embedding")
    for t, nm in ((tokens, "tokens"), (src, "src"), (sampled, "sampled")):
        _need(t, nm, torch.int32, 1)
    if src.shape[0] < tokens.shape[0]:
        raise KernelError("src is shorter than tokens")
    _check(lib.tnx_patch_tokens(_p(tokens), _p(src), _p(sampled), c_int(tokens.shape[0]), _stream()), "patch_tokens")


def gather_rows(table, ids, out):
    lib = _lib("embedding", table, out)
    _need(table, "table", _FLOATS, 2)
    _need(ids, "ids", torch.int32, 1)
    _need(out, "out", _FLOATS, 2)
    _check(lib.tnx_gather_rows(_p(table), _p(ids), _p(out), c_int(ids.shape[0]), c_int(table.shape[1]),
                               c_int(_is_h16(table)), c_int(_is_h16(out)), _stream()), "gather_rows")


def layer_norm(x, gamma, beta, eps, out_f32=None, out_act=None, rows=None):
    """Rows of the 32-bit x normalised; `rows` (int32) picks input rows."""
    lib = _lib("layernorm", out_act)
    _need(x, "x", torch.float32, 2)
    H = x.shape[1]
    n_rows = rows.shape[0] if rows is not None else x.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
    for t, nm in ((gamma, "gamma"), (beta, "beta")):
        if t is not None:
            _need(t, nm, torch.float32, 1)
            if t.shape[0] != H:
                raise KernelError(f"{nm} has {t.shape[0]} elements, the rows have {H}")
    act_bf16 = 0
    for t, nm in ((out_f32, "out_f32"), (out_act, "out_act")):
        if t is not None:
            _need(t, nm, torch.float32 if nm == "out_f32" else _FLOATS, 2)
            if t.shape[0] < n_rows or t.shape[1] != H:
                raise KernelError(f"{nm} has shape {tuple(t.shape)}, needs [{n_rows}, {H}]")
    if out_act is not None:
        act_bf16 = _is_h16(out_act)
    _check(lib.tnx_layer_norm(_p(x), _p(rows), _p(gamma), _p(beta), c_float(eps), _p(out_f32), _p(out_act),
                              c_int(n_rows), c_int(H), c_int(act_bf16), _stream()), "layer_norm")


def pick_rows(x, rows, out_f32=None, out_act=None):
    lib = _lib("layernorm", out_act)
    _need(x, "x", torch.float32, 2)
    n_rows = rows.shape[0] if rows is not None else x.shape[0]
    act_bf16 = _is_h16(out_act) if out_act is not None else 0
    _check(lib.tnx_pick_rows(_p(x), _p(rows), _p(out_f32), _p(out_act), c_int(n_rows), c_int(x.shape[1]),
                             c_int(act_bf16), _stream()), "pick_rows")


def gemm_simt(a, w, out, bias=None, residual=None, activation=None):
    """out = epilogue(a @ w^T) on CUDA cores with 32-bit FMA; a [M, K], w [N, K], out [M, N]; each of
    them 32-bit or 16-bit (a 16-bit matrix is widened exactly as it is loaded)."""
    lib = _lib("gemm_simt", a, w, out)
    act = activation_code(activation)
    _need(a, "a", _FLOATS, None, contiguous=False)
    _need(w, "w", _FLOATS, None, contiguous=False)
    _need(out, "out", _FLOATS, None, contiguous=False)
    M, K, lda = _rows_2d(a, "a")
    N, Kw, ldw = _rows_2d(w, "w")
    Mo, No, ldc = _rows_2d(out, "out")
    if Kw != K or Mo != M or No != N:
        raise KernelError(f"gemm shapes do not fit: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != N:
            raise KernelError("bias length differs from the output width")
    if residual is not None:
        _need(residual, "residual", torch.float32, None, contiguous=False)
        if tuple(residual.shape) != (M, N) or _rows_2d(residual, "residual")[2] != ldc or out.dtype != torch.float32:
            raise KernelError("residual must be float32 with the shape and row stride of a float32 out")
    _check(lib.tnx_gemm_simt(_p(a), _p(w), _p(bias), _p(residual), _p(out), c_int(M), c_int(N), c_int(K),
                             c_int(lda), c_int(ldw), c_int(ldc), c_int(act), c_int(_is_h16(a)),
                             c_int(_is_h16(w)), c_int(_is_h16(out)), _stream()), "gemm_simt")


def kv_append(k_src, v_src, slot_mapping, cache, page_size):
    """k_src, v_src: [N, n_kv_heads * head_dim] views (rows contiguous, one row stride);
    cache: [pages, 2, n_kv_heads, page_size, head_dim]."""
    lib = _lib("kv_cache", cache, k_src, v_src)
    _need(cache, "cache", _FLOATS, 5)
    _need(slot_mapping, "slot_mapping", torch.int32, 1)
    N, width, stride = _rows_2d(k_src, "k_src")
    if _rows_2d(v_src, "v_src") != (N, width, stride) or k_src.dtype != cache.dtype or v_src.dtype != cache.dtype:
        raise KernelError("k_src and v_src must agree in shape, stride and dtype with the cache")
    _, two, n_kv, ps, d = cache.shape
    if two != 2 or ps != page_size or n_kv * d != width:
        raise KernelError(f"cache shape {tuple(cache.shape)} does not fit rows of width {width}")
    _check(lib.tnx_kv_append(_p(k_src), _p(v_src), c_int(stride), _p(slot_mapping), _p(cache), c_int(N),
                             c_int(n_kv), c_int(d), c_int(ps), c_int(_is_h16(cache)), _stream()), "kv_append")


def copy_rows(tensor, pairs):
    """Rows (first axis) of a contiguous tensor copied within it: for each (source, destination) of the
    int32 tensor `pairs` [n, 2], row destination takes the contents of row source.  No row may be both."""
    lib = _build.load("kv_cache")
    if not tensor.is_cuda or not tensor.is_contiguous() or tensor.dim() < 1:
        raise KernelError("copy_rows needs a contiguous tensor on the GPU")
    _need(pairs, "pairs", torch.int32, 2)
    if pairs.shape[1] != 2:
        raise KernelError("pairs must be [n, 2]")
    row_bytes = tensor[0].numel() * tensor.element_size() if tensor.shape[0] else 0
    _check(lib.tnx_copy_rows(_p(tensor), _p(pairs), c_int(pairs.shape[0]), ctypes.c_longlong(row_bytes), _stream()), "copy_rows")


def attention_simt(q, cache, block_tables, token_request, positions, out, n_heads, scale, window=0):
    """q: [N, n_heads * head_dim] view; out likewise; cache as in kv_append."""
    lib = _lib("attention_simt", cache, q, out)
    _need(cache, "cache", _FLOATS, 5)
    N, width, q_stride = _rows_2d(q, "q")
    No, wo, out_stride = _rows_2d(out, "out")
    _, _, n_kv, ps, d = cache.shape
    if width != n_heads * d or (No, wo) != (N, width) or q.dtype != cache.dtype or out.dtype != cache.dtype:
        raise KernelError("q/out do not fit the cache's head size or dtype")
    _need(block_tables, "block_tables", torch.int32, 2)
    _need(token_request, "token_request", torch.int32, 1)
    _need(positions, "positions", torch.int32, 1)
    _check(lib.tnx_attention_simt(_p(q), c_int(q_stride), _p(cache), _p(block_tables), c_int(block_tables.stride(0)),
                                  _p(token_request), _p(positions), _p(out), c_int(out_stride), c_int(N),
                                  c_int(n_heads), c_int(n_kv), c_int(d), c_int(ps), c_int(window or 0),
                                  c_float(scale), c_int(_is_h16(cache)), _stream()), "attention_simt")


def sample(logits, out, temperature=None, top_k=None, top_p=None, seeds=None, counters=None, suppress_id=-1,
           min_keep=None, deterministic=False):
    """out[r] = next token of row r; per-row float32 temperature (<= 0: greedy), int32 top_k
    (0: off), float32 top_p (1: off), int32 min_keep (the fewest tokens top-p keeps; None: 1), int64
    seeds and counters for the Philox draw.  deterministic: no draw; the kept tokens are taken from
    the most likely down and the first at which the summed probability reaches one half is chosen."""
    lib = _build.load("sampling")
    _need(logits, "logits", torch.float32, None, contiguous=False)
    R, V, ld = _rows_2d(logits, "logits")
    _need(out, "out", torch.int32, 1)
    for t, nm, dt in ((temperature, "temperature", torch.float32), (top_k, "top_k", torch.int32),
                      (top_p, "top_p", torch.float32), (min_keep, "min_keep", torch.int32),
                      (seeds, "seeds", torch.int64), (counters, "counters", torch.int64)):
        if t is not None:
            _need(t, nm, dt, 1)
            if t.shape[0] < R:
                raise KernelError(f"{nm} has fewer entries than there are rows")
    _check(lib.tnx_sample(_p(logits), c_int(ld), c_int(R), c_int(V), _p(temperature), _p(top_k), _p(top_p),
                          _p(min_keep), c_int(1 if deterministic else 0), _p(seeds), _p(counters),
                          c_int(suppress_id), _p(out), _stream()), "sample")


def sample_packed(logits, packed, with_top_p, out, err_word=None):
    """sample() with every row's parameters packed, 16 int32 words a row (csrc/sampling.cu):
    temperature, top_k, top_p, min_keep, seed (2), counter (2), flags, up to four suppressed ids.
    err_word: a device int32 whose value is written to out[rows] (out then needs rows + 1 entries)."""
    lib = _build.load("sampling")
    _need(logits, "logits", torch.float32, None, contiguous=False)
    R, V, ld = _rows_2d(logits, "logits")
    _need(out, "out", torch.int32, 1)
    _need(packed, "packed", torch.int32, None)
    words = lib.tnx_sample_row_words()
    if packed.numel() < R * words:
        raise KernelError(f"packed holds {packed.numel()} words, {R} rows need {R * words}")
    if out.shape[0] < R + (1 if err_word is not None else 0):
        raise KernelError("out is too short for the rows (and the error word)")
    if err_word is not None:
        _need(err_word, "err_word", torch.int32, 1)
    _check(lib.tnx_sample_packed(_p(logits), c_int(ld), c_int(R), c_int(V), _p(packed), c_int(1 if with_top_p else 0),
                                 _p(err_word), _p(out), _stream()), "sample")


def sample_force_blocks_per_row(blocks=None) -> None:
    """The sampling kernel with 1, 2, 4 or 8 thread blocks a row whatever the sizes (None: its own rule
    again).  For the test that draws the same tokens with each; not for serving."""
    _check(_build.load("sampling").tnx_sample_force_blocks_per_row(c_int(int(blocks or 0))), "sample_force_blocks_per_row")


def error_word(device) -> torch.Tensor:
    """The device word that kernels with bounded waits set when a wait ran out (0: none did)."""
    return _state(device)["err"]


def raise_if_error_code(code: int, where: str = "") -> None:
    """Raises for a value of the error word that was read along with a step's results."""
    if code:
        for st in _dev_state.values():
            st["err"].zero_()
        raise KernelError(f"a bounded wait ran out inside a kernel{where} (where: {code}); its results, and "
                          "everything computed from them, are invalid")


# ---------------------------------------------------------------------------------------------
# Tensor-core kernels (bfloat16).
_attention_impls = {}
_gemm_plans = {}          # (M, N, K, SMs) -> (splits, scratch bytes, counters) as the library plans them
_dev_state = {}          # per device: error word, split-K scratch and counters, SM count


def _state(device):
    key = device.index if device.index is not None else torch.cuda.current_device()
    st = _dev_state.get(key)
    if st is None:
        st = {"err": torch.zeros(1, dtype=torch.int32, device=device),
              "scratch": None, "counters": torch.zeros(1024, dtype=torch.int32, device=device),
              "sms": torch.cuda.get_device_properties(device).multi_processor_count}
        _dev_state[key] = st
    return st


def _grow(st, key, need, dtype, device, minimum, zero=False):
    """Scratch buffer `key` with at least `need` elements.  A buffer that is outgrown is kept alive:
    captured CUDA graphs still hold its address."""
    cur = st.get(key)
    if cur is None or cur.numel() < need:
        if cur is not None:
            st.setdefault("retired", []).append(cur)
        n = max(int(need), int(minimum))
        st[key] = torch.zeros(n, dtype=dtype, device=device) if zero else torch.empty(n, dtype=dtype, device=device)
    return st[key]


def raise_on_device_error(device=None):
    """Reads the error word that kernels with bounded waits set (this synchronises)."""
    for key, st in _dev_state.items():
        code = int(st["err"].item())
        if code:
            st["err"].zero_()
            raise KernelError(f"a bounded wait ran out inside a kernel on cuda:{key} (where: {code}); "
                              "its results are invalid")


def selftest_wait_runs_out(device, code: int = 99, limit_ns: int = 1_000_000) -> None:
    """Launches a kernel whose bounded wait (about a millisecond) runs out by design and records
    `code` in the device's error word: what raise_on_device_error() and the engine's per-step check
    then report.  For tests of the error path; nothing hangs, the wait ends by itself."""
    lib = _build.load("gemm_tc")
    st = _state(torch.device(device))
    _check(lib.tnx_selftest_wait_runs_out(_p(st["err"]), c_int(code), ctypes.c_longlong(limit_ns), _stream()),
           "selftest_wait_runs_out")


def gemm_tc_supported(a, w, out) -> bool:
    """Size rules of the TMA descriptors: row pitches multiples of 16 bytes, 16-byte aligned bases."""
    if a.dtype not in _H16 or w.dtype != a.dtype or (out.dtype in _H16 and out.dtype != a.dtype):
        return False
    K = a.shape[1]
    if K % 8 or a.stride(0) % 8 or w.stride(0) % 8 or a.data_ptr() % 16 or w.data_ptr() % 16:
        return False
    return out.data_ptr() % 16 == 0


def gemv(a, w, out, bias=None, residual=None, activation=None):
    """out = epilogue(a @ w^T) for one to four tokens, the weights streamed through the multiply-add
    units (16-bit operands, 32-bit sums).  gemm_tc() picks it by itself for one token."""
    lib = _lib("gemv", a, w, out)
    act = activation_code(activation)
    _need(a, "a", _H16, None, contiguous=False)
    _need(w, "w", _H16, None, contiguous=False)
    _need(out, "out", _FLOATS, None, contiguous=False)
    M, K, lda = _rows_2d(a, "a")
    N, Kw, ldw = _rows_2d(w, "w")
    Mo, No, ldc = _rows_2d(out, "out")
    if Kw != K or Mo != M or No != N:
        raise KernelError(f"gemv shapes do not fit: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if not lib.tnx_gemv_supported(c_int(M), c_int(N), c_int(K)) or not gemm_tc_supported(a, w, out):
        raise KernelError("gemv takes one to four tokens, K a multiple of 8 and 16-byte aligned rows")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != N:
            raise KernelError("bias length differs from the output width")
    if residual is not None:
        _need(residual, "residual", torch.float32, None, contiguous=False)
        if tuple(residual.shape) != (M, N) or _rows_2d(residual, "residual")[2] != ldc or out.dtype != torch.float32:
            raise KernelError("residual must be float32 with the shape and row stride of a float32 out")
    _check(lib.tnx_gemv(_p(a), _p(w), _p(bias), _p(residual), _p(out), c_int(M), c_int(N), c_int(K),
                        c_int(lda), c_int(ldw), c_int(ldc), c_int(act), c_int(_is_h16(out)),
                        _stream()), "gemv")


def gemv_layer_norm_supported(x, w, out) -> bool:
    """Whether gemv_layer_norm takes these tensors: one token (measured on the 6.7B sizes: a decode step of one
    request 3.15 -> 3.11 ms; with two requests the tensor-core product after a LayerNorm kernel takes 3.40 ms
    and this kernel 3.90), 32-bit rows of x, a 16-bit matrix, 16-byte aligned rows, the row within shared memory."""
    if x.dim() != 2 or x.dtype != torch.float32 or w.dtype not in _H16 or x.shape[0] != 1:
        return False
    if out.dtype in _H16 and out.dtype != w.dtype:
        return False
    K = x.shape[1]
    return (w.dim() == 2 and w.shape[1] == K and K % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 4 == 0
            and x.data_ptr() % 16 == 0 and w.stride(1) == 1 and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0
            and K * 6 <= 112 * 1024)


def gemv_layer_norm(x, gamma, beta, eps, w, out, bias=None, residual=None, activation=None):
    """out = epilogue(LayerNorm(x) @ w^T) for one to four tokens: x are 32-bit rows (the residual stream),
    normalized in 32-bit by every thread block of the product as it stages its activations, rounded to
    the matrix's 16-bit type as a LayerNorm kernel would round them."""
    lib = _lib("gemv", w, out)
    act = activation_code(activation)
    _need(x, "x", torch.float32, None, contiguous=False)
    _need(w, "w", _H16, None, contiguous=False)
    _need(out, "out", _FLOATS, None, contiguous=False)
    M, K, ldx = _rows_2d(x, "x")
    N, Kw, ldw = _rows_2d(w, "w")
    Mo, No, ldc = _rows_2d(out, "out")
    if Kw != K or Mo != M or No != N:
        raise KernelError(f"gemv shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if not lib.tnx_gemv_supported(c_int(M), c_int(N), c_int(K)):
        raise KernelError("gemv takes one to four tokens and K a multiple of 8")
    for t, nm in ((gamma, "gamma"), (beta, "beta")):
        if t is not None:
            _need(t, nm, torch.float32, 1)
            if t.shape[0] != K:
                raise KernelError(f"{nm} length differs from the row length")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != N:
            raise KernelError("bias length differs from the output width")
    if residual is not None:
        _need(residual, "residual", torch.float32, None, contiguous=False)
        if tuple(residual.shape) != (M, N) or _rows_2d(residual, "residual")[2] != ldc or out.dtype != torch.float32:
            raise KernelError("residual must be float32 with the shape and row stride of a float32 out")
    _check(lib.tnx_gemv_ln(_p(x), c_int(ldx), _p(gamma), _p(beta), c_float(float(eps)), _p(w), _p(bias), _p(residual), _p(out),
                           c_int(M), c_int(N), c_int(K), c_int(ldw), c_int(ldc), c_int(act), c_int(_is_h16(out)),
                           _stream()), "gemv_layer_norm")


def gemm_tc(a, w, out, bias=None, residual=None, activation=None, splits=None, few_tokens_kernel=True, cluster=False):
    """out = epilogue(a @ w^T), 16-bit operands (both bfloat16 or both float16), 32-bit accumulation: on the tcgen05 tensor cores,
    or (one token, unless few_tokens_kernel is False or splits is given) as a stream of the
    weights through the multiply-add units.  `splits` forces a split of K for up to 128 tokens (a test
    hook): partial tiles added by the CTA that finishes last, or (cluster=True, at most 8 splits) by
    the CTAs of a cluster through their shared memory, which is what the kernel's own plan uses."""
    lib = _lib("gemm_tc", a, w, out)
    act = activation_code(activation)
    _need(a, "a", _H16, None, contiguous=False)
    _need(w, "w", _H16, None, contiguous=False)
    _need(out, "out", _FLOATS, None, contiguous=False)
    M, K, lda = _rows_2d(a, "a")
    N, Kw, ldw = _rows_2d(w, "w")
    Mo, No, ldc = _rows_2d(out, "out")
    if Kw != K or Mo != M or No != N:
        raise KernelError(f"gemm shapes do not fit: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if not gemm_tc_supported(a, w, out):
        raise KernelError("the tensor-core product needs K and the row pitches to be multiples of 8 elements "
                          "and 16-byte aligned bases; use gemm_simt for other sizes")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != N:
            raise KernelError("bias length differs from the output width")
    if residual is not None:
        _need(residual, "residual", torch.float32, None, contiguous=False)
        if tuple(residual.shape) != (M, N) or _rows_2d(residual, "residual")[2] != ldc or out.dtype != torch.float32:
            raise KernelError("residual must be float32 with the shape and row stride of a float32 out")
    if few_tokens_kernel and splits is None and M == 1:    # with two tokens and more the tensor-core kernel is as fast (measured)
        gv = _lib("gemv", a, w, out)
        if gv.tnx_gemv_supported(c_int(M), c_int(N), c_int(K)):
            _check(gv.tnx_gemv(_p(a), _p(w), _p(bias), _p(residual), _p(out), c_int(M), c_int(N), c_int(K),
                               c_int(lda), c_int(ldw), c_int(ldc), c_int(act), c_int(_is_h16(out)),
                               _stream()), "gemv")
            return
    st = _state(a.device)
    plan = _gemm_plans.get((M, N, K, st["sms"]))
    if plan is None:
        n_splits, nbytes, ncnt = c_int(1), ctypes.c_longlong(0), c_int(0)
        lib.tnx_gemm_tc_plan(c_int(M), c_int(N), c_int(K), c_int(st["sms"]), ctypes.byref(n_splits),
                             ctypes.byref(nbytes), ctypes.byref(ncnt))
        if len(_gemm_plans) > 4096:
            _gemm_plans.clear()
        plan = _gemm_plans[(M, N, K, st["sms"])] = (n_splits.value, nbytes.value, ncnt.value)
    n_splits, nbytes, ncnt = c_int(plan[0]), ctypes.c_longlong(plan[1]), c_int(plan[2])
    if splits is not None and M <= lib.tnx_gemm_tc_few_tokens():
        kb = -(-K // 64)
        s = max(1, min(int(splits), kb))
        per = -(-kb // s)
        s = -(-kb // per)
        bn = 16 if M <= 16 else (32 if M <= 32 else (64 if M <= 64 else 128))
        tiles = -(-N // 128)
        n_splits, nbytes, ncnt = c_int(s), ctypes.c_longlong(s * tiles * 128 * bn * 4 if s > 1 else 0), c_int(tiles if s > 1 else 0)
        if cluster:
            if s > 8:
                raise KernelError("a cluster holds at most 8 thread blocks")
            nbytes, ncnt = ctypes.c_longlong(0), c_int(0)
    scratch = None
    if nbytes.value:
        need = nbytes.value // 4
        scratch = _grow(st, "scratch", need, torch.float32, a.device, 1 << 22)
        _grow(st, "counters", ncnt.value, torch.int32, a.device, 1024, zero=True)
    _check(lib.tnx_gemm_tc(_p(a), _p(w), _p(bias), _p(residual), _p(out), c_int(M), c_int(N), c_int(K),
                           c_int(lda), c_int(ldw), c_int(ldc), c_int(act), c_int(_is_h16(out)),
                           n_splits, _p(scratch), _p(st["counters"]), _p(st["err"]), _stream()), "gemm_tc")


GEMM_PLANS = {"tiles_128": 0, "pairs": 1, "persistent": 2, "pairs_shared": 4,
              "split_1": 31, "split_2": 32, "split_4": 34, "split_8": 38}


def gemm_tc_force_plan(plan=None, dtype=torch.bfloat16) -> None:
    """Imposes one kernel on every tensor-core product of more than 128 tokens (None: the library's
    own estimates choose again).  A product whose sizes do not allow the plan is refused.  For the
    test that times every candidate against the estimates' choice; not for serving."""
    lib = _build.load("gemm_tc", dtype)
    lib.tnx_gemm_tc_force_plan(c_int(-1 if plan is None else GEMM_PLANS[plan]))
    _gemm_plans.clear()


def decode_attention_plan(pairs: int, sms: int, head_dim: int, max_pages: int):
    """(warps a block, splits of the context) for `pairs` (row, head) pairs of decode attention.

    An SM holds sixteen warps of this kernel: four blocks of four, two of eight or one of sixteen.
    Measured at 1 to 64 rows of 32, 40 and 56 heads of 128 dims over contexts of 2,040 (every plan
    against the one chosen here), the fastest plan keeps all blocks on the GPU at once where it can and
    gives the SMs equal numbers of them:
      * few pairs: blocks of eight warps, as many splits as fill two blocks per SM (1 / 2 rows of 32
        heads: 13 / 18 us);
      * about one pair per SM (0.75 to 1): one block of sixteen warps each and no split (4 rows: 28 us,
        eight warps and two splits 30);
      * up to a third of four blocks per SM: four warps and three splits (6 rows: 39 us; eight warps and
        no split, which leaves the SMs one or two blocks each, 47);
      * up to two pairs per SM: eight warps, no split (8 rows: 49 us);
      * up to 2.7 pairs per SM: four warps and three splits again (12 rows: 73 us; without splits the SMs
        hold two or three blocks each, 80);
      * up to four pairs per SM: four warps, no split (16 rows: 91 us); beyond: four or eight warps, whichever
        an estimate of waves x (streaming + cost of a block) makes the faster (64 rows: eight warps, 321 us;
        256 rows over 256 tokens: four warps, 176 against 208 us).
    (kernels/microbench.py attention-plans repeats the sweep.)  A split keeps at least eight pages, and contexts of fewer than 48 pages are not split in three (at
    500 tokens the plans without splits were 7-12 % faster there, and from a quarter of a pair per SM
    one block of sixteen warps was: 9 against 12 us at 3 rows)."""
    most = max(1, max_pages // 8)
    wide = 16 if head_dim <= 128 else 8
    if pairs * 4 <= sms * 3:
        if most <= 4 and pairs * 4 >= sms:
            return wide, 1
        return 8, max(1, min(most, 32, (2 * sms) // max(1, pairs)))
    if pairs <= sms:
        return wide, 1
    if pairs * 3 <= 4 * sms and most >= 6:
        return 4, 3
    if pairs <= 2 * sms:
        return 8, 1
    if pairs * 10 <= sms * 27 and most >= 6:
        return 4, 3
    if pairs <= 4 * sms:
        return 4, 1
    # More pairs than the GPU holds blocks: blocks of four warps (four an SM) or of eight (two an SM) follow
    # one another.  A block costs 0.6 / 2.2 us beside its pages' streaming (8,192 pairs over 256 tokens: 176
    # against 208 us), and the last wave of blocks is as long as a full one (1,280 pairs over 1,024 tokens:
    # 123 us in three waves of four-warp blocks, 115 us in five of eight-warp ones; over 256 tokens 37 against 41).
    page_us = 16 * head_dim * 4 / 6.5e6                      # one page of keys and values at 6.5 TB/s
    t4 = -(-pairs // (4 * sms)) * (4 * sms * max_pages * page_us + 0.6)
    t8 = -(-pairs // (2 * sms)) * (2 * sms * max_pages * page_us + 2.2)
    return (4, 1) if t4 < t8 else (8, 1)


def attention_decode(q, cache, block_tables, token_request, positions, out, n_heads, scale, window=0, rows=None,
                     n_rows=None, max_kv_len=None, n_splits=None, new_kv=None, warps=None):
    """One query token per row over the paged 16-bit cache.  `rows` (int32) names the rows of q
    that are decode tokens (None: all); max_kv_len bounds their contexts (for the split plan).
    new_kv = (k, v), [rows of q, kv_heads * head_dim] bfloat16: the keys and values of the rows' own
    tokens, which the kernel then writes into their pages itself (no kv_append before it).
    n_splits (with warps, 4 or 8 a block) forces a plan: a test hook."""
    lib = _lib("attention_decode", cache, q, out)
    _need(cache, "cache", _H16, 5)
    N, width, q_stride = _rows_2d(q, "q")
    No, wo, out_stride = _rows_2d(out, "out")
    _, _, n_kv, ps, d = cache.shape
    if width != n_heads * d or (No, wo) != (N, width) or q.dtype != cache.dtype or out.dtype != cache.dtype:
        raise KernelError("q/out do not fit the cache's head size or dtype")
    _need(block_tables, "block_tables", torch.int32, 2)
    _need(token_request, "token_request", torch.int32, 1)
    _need(positions, "positions", torch.int32, 1)
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
    R = int(n_rows) if n_rows is not None else (rows.shape[0] if rows is not None else N)
    st = _state(q.device)
    max_pages = max(1, -(-(int(max_kv_len) if max_kv_len is not None else block_tables.shape[1] * ps) // ps))
    forced_warps, warps = warps, 4
    if n_splits is None:
        warps, n_splits = decode_attention_plan(R * n_heads, st["sms"], d, max_pages)
        pps = -(-max_pages // n_splits)
        pps = -(-pps // warps) * warps
    else:                                                  # a test's own plan (warps: 4, 8 or 16 a block)
        warps = int(forced_warps or 4)
        n_splits = max(1, min(int(n_splits), max_pages))
        pps = -(-max_pages // n_splits)
    n_splits = -(-max_pages // pps)
    scratch = None
    if n_splits > 1:
        need = R * n_heads * n_splits * (d + 2)
        scratch = _grow(st, "att_scratch", need, torch.float32, q.device, 1 << 20)
        _grow(st, "att_counters", R * n_heads, torch.int32, q.device, 8192, zero=True)
    k_new = v_new = None
    kv_stride = 0
    if new_kv is not None:
        k_new, v_new = new_kv
        for t, nm in ((k_new, "k"), (v_new, "v")):
            _need(t, nm, cache.dtype, None, contiguous=False)
            if _rows_2d(t, nm)[:2] != (N, n_kv * d):
                raise KernelError(f"new {nm} must be [{N}, {n_kv * d}]")
        kv_stride = k_new.stride(0)
        if v_new.stride(0) != kv_stride:
            raise KernelError("new k and v must have the same row pitch")
    _check(lib.tnx_attention_decode_append(
        _p(q), c_int(q_stride), _p(cache), _p(block_tables), c_int(block_tables.stride(0)),
        _p(rows), _p(token_request), _p(positions), _p(out), c_int(out_stride), c_int(R),
        c_int(n_heads), c_int(n_kv), c_int(d), c_int(ps), c_int(window or 0), c_float(scale),
        c_int(n_splits), c_int(pps), _p(scratch), _p(st.get("att_counters")), _p(k_new), _p(v_new), c_int(kv_stride),
        c_int(warps), _stream()), "attention_decode")


ATTN_PREFILL_TILE = 128      # query rows of one work item of the prefill attention kernel


def attention_prefill(q, cache, block_tables, tile_req, tile_q0, q_start, q_len, ctx_len, out, n_heads, scale,
                      window=0, n_items=None):
    """Causal attention of prompt portions: work items (request, first row of an ATTN_PREFILL_TILE-row tile)."""
    lib = _lib("attention_prefill", cache, q, out)
    _need(cache, "cache", _H16, 5)
    N, width, q_stride = _rows_2d(q, "q")
    No, wo, out_stride = _rows_2d(out, "out")
    _, _, n_kv, ps, d = cache.shape
    if width != n_heads * d or (No, wo) != (N, width) or q.dtype != cache.dtype or out.dtype != cache.dtype:
        raise KernelError("q/out do not fit the cache's head size or dtype")
    for t, nm in ((block_tables, "block_tables"), (tile_req, "tile_req"), (tile_q0, "tile_q0"), (q_start, "q_start"),
                  (q_len, "q_len"), (ctx_len, "ctx_len")):
        _need(t, nm, torch.int32, 2 if nm == "block_tables" else 1)
    n = int(n_items) if n_items is not None else tile_req.shape[0]
    _check(lib.tnx_attention_prefill(_p(q), c_int(q_stride), _p(cache), _p(block_tables), c_int(block_tables.stride(0)),
                                     _p(tile_req), _p(tile_q0), _p(q_start), _p(q_len), _p(ctx_len), _p(out),
                                     c_int(out_stride), c_int(n), c_int(n_heads), c_int(n_kv), c_int(d), c_int(ps),
                                     c_int(window or 0), c_float(scale), _stream()), "attention_prefill")


def attention_prefill_tc_supported(q, cache, out) -> bool:
    """The tcgen05 prefill kernel takes head sizes 64, 80, 96, 112 and 128, pages of 16 and 16-byte aligned rows."""
    return (cache.dtype in _H16 and q.dtype == cache.dtype and out.dtype == cache.dtype and cache.shape[4] in (64, 80, 96, 112, 128) and cache.shape[3] == 16 and q.stride(0) % 8 == 0 and
            out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0 and
            cache.shape[0] * 2 * cache.shape[2] * 16 < 2 ** 31)


def attention_prefill_tc(q, cache, block_tables, tile_req, tile_q0, q_start, q_len, ctx_len, out, n_heads, scale,
                         window=0, n_items=None):
    """attention_prefill on the tcgen05 tensor cores (head sizes 64 to 128 in steps of 16).  The cache must hold finite
    numbers in every row, written or not (CacheStorage allocates it zeroed)."""
    lib = _lib("attention_prefill_tc", cache, q, out)
    _need(cache, "cache", _H16, 5)
    N, width, q_stride = _rows_2d(q, "q")
    No, wo, out_stride = _rows_2d(out, "out")
    n_pages, _, n_kv, ps, d = cache.shape
    if not attention_prefill_tc_supported(q, cache, out) or width != n_heads * d or (No, wo) != (N, width):
        raise KernelError("attention_prefill_tc takes a 16-bit type, head sizes 64 to 128 in steps of 16, pages of 16, 16-byte aligned rows")
    for t, nm in ((block_tables, "block_tables"), (tile_req, "tile_req"), (tile_q0, "tile_q0"), (q_start, "q_start"),
                  (q_len, "q_len"), (ctx_len, "ctx_len")):
        _need(t, nm, torch.int32, 2 if nm == "block_tables" else 1)
    n = int(n_items) if n_items is not None else tile_req.shape[0]
    st = _state(q.device)
    _check(lib.tnx_attention_prefill_tc(_p(q), c_int(q_stride), c_int(N), _p(cache), ctypes.c_longlong(n_pages * 2 * n_kv * ps),
                                        _p(block_tables), c_int(block_tables.stride(0)), _p(tile_req), _p(tile_q0),
                                        _p(q_start), _p(q_len), _p(ctx_len), _p(out), c_int(out_stride), c_int(n),
                                        c_int(n_heads), c_int(n_kv), c_int(d), c_int(ps), c_int(window or 0),
                                        c_float(scale), _p(st["err"]), _stream()), "attention_prefill_tc")


def _attention_h16(ctx, group, q, cache, out, n_heads, scale, window, new_kv):
    if cache.shape[3] != 16 or q.stride(0) % 8 or q.data_ptr() % 16:
        return False
    bt = ctx.block_tables[group]
    fused = None
    if new_kv is not None:
        k, v, slots = new_kv
        if ctx.decode_only and not ctx.n_prefill_tiles and k.stride(0) % 8 == 0 and k.data_ptr() % 16 == 0 \
                and v.data_ptr() % 16 == 0:
            fused = (k, v)                       # a decode step: the attention kernel appends by itself
        else:
            kv_append(k, v, slots, cache, ctx.page_size)
    if ctx.n_prefill_tiles:
        prefill = attention_prefill_tc if attention_prefill_tc_supported(q, cache, out) else attention_prefill
        prefill(q, cache, bt, ctx.tile_req, ctx.tile_q0, ctx.q_start, ctx.q_len, ctx.ctx_len, out,
                n_heads, scale, window, n_items=ctx.n_prefill_tiles)
    if ctx.n_decode_rows:
        attention_decode(q, cache, bt, ctx.token_request, ctx.positions, out, n_heads, scale, window,
                         rows=None if ctx.decode_only else ctx.decode_rows, n_rows=ctx.n_decode_rows,
                         max_kv_len=ctx.max_decode_ctx, new_kv=fused)
    return True


_attention_impls["h16"] = _attention_h16


def attention(ctx, group, q, cache, out, n_heads, scale, window=0, new_kv=None):
    """Attention of this step's queries over the cache of the running schedule entry.  32-bit
    caches, and head sizes or windows that the 16-bit kernels do not take, run on the CUDA-core
    kernel; a 16-bit cache runs the prefill kernel for requests with several rows and the split
    decode kernel for requests with one.  new_kv = (k, v, slot_mapping): the keys and values of
    this step's tokens, not yet in the cache; they are appended here, by kv_append or (a step of
    decode tokens only, 16-bit) by the decode kernel itself."""
    impl = _attention_impls.get("h16") if cache.dtype in _H16 else None
    if impl is not None and impl(ctx, group, q, cache, out, n_heads, scale, window, new_kv):
        return
    if new_kv is not None:
        kv_append(new_kv[0], new_kv[1], new_kv[2], cache, ctx.page_size)
    attention_simt(q, cache, ctx.block_tables[group], ctx.token_request, ctx.positions, out, n_heads, scale,
                   window)
