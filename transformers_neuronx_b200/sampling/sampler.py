"""Next-token choice on the GPU: greedy, temperature, top-k and top-p, per request.

What the reference samples with: argmax (src/transformers_neuronx/sampling.py:108-128); top-k with
multinomial over softmax and the end-of-sequence score set to -inf (sampling.py:143-156);
temperature, then top-k/top-p filtering, then multinomial (sampling.py:337-345, :199-264); and on
the device (layers/generation.py:147-199) the same with a least number of tokens that top-p keeps
(hlo.py:2349-2361) and, for tests, a draw whose uniform number is fixed at one half
(hlo.py:2452-2463).  All of it is one kernel here (csrc/sampling.cu); a draw depends on (logits,
parameters, seed, counter) only.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from ..kernels import ops


class Sampler:
    def __init__(self, device):
        self.device = device

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
        # one small host-to-device copy: six columns of parameters
        buf = np.zeros((6, R), dtype=np.int64)
        buf[0] = np.asarray(temperatures, dtype=np.float32).view(np.int32).astype(np.int64)
        buf[1] = np.asarray(top_ks, dtype=np.int64)
        buf[2] = np.asarray(top_ps, dtype=np.float32).view(np.int32).astype(np.int64)
        buf[3] = np.asarray(seeds, dtype=np.uint64).view(np.int64)
        buf[4] = np.asarray(counters, dtype=np.int64)
        use_min = min_keeps is not None and any(m > 1 for m in min_keeps)
        if use_min:
            buf[5] = np.asarray(min_keeps, dtype=np.int64)
        dev = torch.from_numpy(buf).to(self.device)
        temp = dev[0].to(torch.int32).view(torch.float32)
        topk = dev[1].to(torch.int32)
        topp = dev[2].to(torch.int32).view(torch.float32)
        # no top-p anywhere in the batch: the kernel variant without the mass histograms
        ops.sample(logits, out, temperature=temp, top_k=topk, top_p=topp if any(p < 1.0 for p in top_ps) else None,
                   seeds=dev[3].contiguous(), counters=dev[4].contiguous(), suppress_id=suppress_id,
                   min_keep=dev[5].to(torch.int32) if use_min else None, deterministic=deterministic)
        return out
