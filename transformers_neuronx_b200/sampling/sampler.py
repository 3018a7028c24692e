"""Next-token choice on the GPU: greedy, temperature, top-k and top-p, per request.

What the reference samples with: argmax (src/transformers_neuronx/sampling.py:108-128); top-k with
multinomial over softmax and the end-of-sequence score set to -inf (sampling.py:143-156);
temperature, then top-k/top-p filtering, then multinomial (sampling.py:337-345, :199-264); and on
the device (layers/generation.py:147-199) the same with a least number of tokens that top-p keeps
(hlo.py:2349-2361) and, for tests, a draw whose uniform number is fixed at one half
(hlo.py:2452-2463).  All of it is one kernel here (csrc/sampling.cu); a draw depends on (logits,
parameters, seed, counter) only.

Every row's parameters travel packed, ROW_WORDS 32-bit words a row.  The engine packs them on the
host (``pack_rows``) into the step's own staging buffer, so that a sampling call is one kernel launch
and no copy; ``Sampler.sample`` is the stand-alone form that copies the packed rows itself.
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from ..kernels import ops

ROW_WORDS = 16            # csrc/sampling.cu: words of one row's packed parameters
MAX_SUPPRESSED = 4        # ids a row can suppress (a request's end-of-sequence ids)


def pack_rows(temperatures: Sequence[float], top_ks: Sequence[int], top_ps: Sequence[float], seeds: Sequence[int],
              counters: Sequence[int], min_keeps: Optional[Sequence[int]] = None,
              deterministic=False, suppress=None) -> np.ndarray:
    """[rows, ROW_WORDS] int32.  deterministic: one flag or one per row; suppress: None, or per row a
    sequence of at most MAX_SUPPRESSED ids whose scores are set to -inf."""
    R = len(temperatures)
    buf = np.zeros((R, ROW_WORDS), dtype=np.int32)
    buf[:, 0] = np.asarray(temperatures, dtype=np.float32).view(np.int32)
    buf[:, 1] = np.asarray(top_ks, dtype=np.int64).astype(np.int32)
    buf[:, 2] = np.asarray(top_ps, dtype=np.float32).view(np.int32)
    buf[:, 3] = 1 if min_keeps is None else np.asarray(min_keeps, dtype=np.int64).astype(np.int32)
    if R:
        buf[:, 4:6] = np.asarray([int(v) & 0xFFFFFFFFFFFFFFFF for v in seeds], dtype=np.uint64).view(np.int32).reshape(R, 2)
        buf[:, 6:8] = np.asarray([int(v) & 0xFFFFFFFFFFFFFFFF for v in counters], dtype=np.uint64).view(np.int32).reshape(R, 2)
    det = [bool(deterministic)] * R if isinstance(deterministic, (bool, int)) else [bool(d) for d in deterministic]
    buf[:, 8] = np.asarray(det, dtype=np.int32)
    buf[:, 9:9 + MAX_SUPPRESSED] = -1
    if suppress is not None:
        for r, ids in enumerate(suppress):
            ids = list(ids or ())
            if len(ids) > MAX_SUPPRESSED:
                raise ValueError(f"a row can suppress at most {MAX_SUPPRESSED} ids, got {len(ids)}")
            buf[r, 9:9 + len(ids)] = ids
    return buf


def needs_top_p(top_ps: Sequence[float], deterministic) -> bool:
    """Whether any row uses top-p or the fixed draw (the kernel variant with the mass histograms)."""
    det = bool(deterministic) if isinstance(deterministic, (bool, int)) else any(deterministic)
    return det or any(p < 1.0 for p in top_ps)


class Sampler:
    def __init__(self, device):
        self.device = device

    def sample_packed(self, logits: torch.Tensor, packed: torch.Tensor, with_top_p: bool, out: torch.Tensor,
                      err_word: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One kernel: logits [R, V] and packed rows (int32, on the device) -> out[:R]; with err_word,
        out[R] receives that device word."""
        ops.sample_packed(logits, packed, with_top_p, out, err_word)
        return out

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float], top_ks: Sequence[int],
               top_ps: Sequence[float], seeds: Sequence[int], counters: Sequence[int],
               suppress_id: int = -1, out: Optional[torch.Tensor] = None,
               min_keeps: Optional[Sequence[int]] = None, deterministic: bool = False) -> torch.Tensor:
        """logits: 32-bit [R, V] on the device -> int32 [R] on the device (written to `out` when given)."""
        R = logits.shape[0]
        out = torch.empty(R, dtype=torch.int32, device=self.device) if out is None else out[:R]
        if R == 0:
            return out
        if all(t <= 0 for t in temperatures) and suppress_id < 0:
            ops.sample(logits, out)
            return out
        rows = pack_rows(temperatures, top_ks, top_ps, seeds, counters, min_keeps, deterministic,
                         [[suppress_id]] * R if suppress_id >= 0 else None)
        dev = torch.from_numpy(rows).to(self.device)          # one small host-to-device copy
        ops.sample_packed(logits, dev, needs_top_p(top_ps, deterministic), out)
        return out
