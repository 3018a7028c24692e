"""Where a step's time goes, kernel family by kernel family, measured with CUDA events.

    with kernel_profile() as prof:
        runner.step(entries)            # or engine.step(), model.sample(...)
    print(prof.report())

The reference's counterpart runs each compiled kernel under the Neuron profiler
(src/transformers_neuronx/base.py:754-759); here every call of a kernel entry point is bracketed by
two events on the current stream.  Bracketing serialises nothing, but a captured CUDA graph is
replayed as a whole and shows up as nothing: profile with `use_cuda_graphs=False`.
"""
from __future__ import annotations

import contextlib
from collections import OrderedDict

import torch

from . import ops

_NAMES = ("embed", "gather_rows", "patch_tokens", "layer_norm", "pick_rows", "gemm_simt", "gemm_tc", "gemv_layer_norm", "kv_append",
          "attention_simt", "attention_decode", "attention_prefill", "attention_prefill_tc", "sample", "sample_packed")


class KernelProfile:
    def __init__(self):
        self.events = []          # (name, start, end)

    def totals(self):
        torch.cuda.synchronize()
        out = OrderedDict()
        for name, a, b in self.events:
            ms, n = out.get(name, (0.0, 0))
            out[name] = (ms + a.elapsed_time(b), n + 1)
        return out

    def report(self) -> str:
        t = self.totals()
        total = sum(ms for ms, _ in t.values()) or 1.0
        lines = [f"{'kernel':24s} {'calls':>6s} {'ms':>10s} {'share':>7s}"]
        for name, (ms, n) in sorted(t.items(), key=lambda kv: -kv[1][0]):
            lines.append(f"{name:24s} {n:6d} {ms:10.3f} {100 * ms / total:6.1f}%")
        lines.append(f"{'all':24s} {sum(n for _, n in t.values()):6d} {total:10.3f}")
        return "\n".join(lines)


@contextlib.contextmanager
def kernel_profile():
    prof = KernelProfile()
    saved = {}

    def wrap(name, fn):
        def timed(*args, **kwargs):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            try:
                return fn(*args, **kwargs)
            finally:
                b.record()
                prof.events.append((name, a, b))
        return timed

    for name in _NAMES:
        saved[name] = getattr(ops, name)
        setattr(ops, name, wrap(name, saved[name]))
    try:
        yield prof
    finally:
        for name, fn in saved.items():
            setattr(ops, name, fn)
