"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives the step
function (engine/step.py) of the model that generation uses.  The nearest thing in the reference is
dumping per-step scores from its demo driver (src/transformers_neuronx/generation_demo.py:694-702).

Input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
Output: for a step in which something is wanted, <out>/<step>.f32 holds the logits at the wanted
places, in the order of the entries and of `want`, as little-endian 32-bit floats [wanted, vocab].
After every step a line `done <step>` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch

from ..config import EngineConfig
from ..kernels import ops
from .loading import load_model
from .step import StepEntry, StepRunner


def replay(model_dir: str, dtype: str, out_dir: str, max_tokens: int, lines=None, out=None) -> int:
    # readline, not iteration: a step must be read as soon as its line is there (the sender waits
    # for `done` before it writes the next one)
    lines = iter(sys.stdin.readline, "") if lines is None else lines
    out = sys.stdout if out is None else out
    os.makedirs(out_dir, exist_ok=True)
    model, cfg = load_model(model_dir, dtype)
    ecfg = EngineConfig(dtype=dtype)
    page = ecfg.page_size
    num_pages = max(1, -(-int(max_tokens) // page))
    runner = StepRunner(model, page_size=page, num_pages=num_pages, max_slots=8,
                        max_model_len=model.spec.max_positions, use_cuda_graphs=True)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            if e["id"] not in runner.cache:
                runner.add_request(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e.get("want", [])))
        if entries:
            logits = runner.step(entries)
            if logits.shape[0] > 0:
                arr = logits.detach().to("cpu", torch.float32).numpy().astype("<f4", copy=False)
                arr.tofile(os.path.join(out_dir, f"{step}.f32"))
            else:
                torch.cuda.synchronize()
            ops.raise_on_device_error()       # a bounded wait that ran out inside a kernel: no `done` for this step
        for rid in rec.get("end", []):
            if rid in runner.cache:
                runner.finish(rid)
        print(f"done {step}", file=out, flush=True)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time (each request rounded up to 64)")
    a = ap.parse_args(argv)
    return replay(a.model, a.dtype, a.out, a.max_tokens)


if __name__ == "__main__":
    sys.exit(main())
