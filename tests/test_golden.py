"""Checks against outputs of the reference's own code (made once by tests/golden/make_reference_goldens.py
on the CPU): the tensor names and shapes of an OPT checkpoint, and which tokens its top-k / top-p filter
keeps."""
import json
import os

import pytest
import torch

from plain import opt_plain as P
from transformers_neuronx_b200.config import OPTConfig
from transformers_neuronx_b200.models import opt as opt_arch
from transformers_neuronx_b200.models.decoder import DecoderModel

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_tensor_names_and_shapes_are_the_references():
    with open(os.path.join(GOLDEN, "opt_tensor_names.json")) as fp:
        g = json.load(fp)
    cfg = OPTConfig.from_dict(g["config"])
    specs = {s.name: list(s.shape) for s in DecoderModel(opt_arch.build_spec(cfg)).tensor_specs()}
    assert specs == g["tensors"]


def _cases():
    with open(os.path.join(GOLDEN, "top_k_top_p.json")) as fp:
        return json.load(fp)


def test_plain_filter_keeps_what_the_reference_keeps():
    for c in _cases():
        scores = torch.tensor(c["scores"])
        kept = P.filter_top_k_top_p(scores, c["top_k"], c["top_p"])
        for b in range(scores.shape[0]):
            mine = sorted(torch.nonzero(kept[b] > -float("inf")).flatten().tolist())
            assert mine == c["kept"][b], (c["top_k"], c["top_p"], b)


@pytest.mark.gpu
def test_sampling_kernel_draws_only_what_the_reference_keeps():
    from transformers_neuronx_b200.kernels import ops
    n = 4000
    for c in _cases():
        scores = torch.tensor(c["scores"])
        for b in range(scores.shape[0]):
            logits = scores[b].cuda()[None].repeat(n, 1).contiguous()
            out = torch.empty(n, dtype=torch.int32, device="cuda")
            ops.sample(logits, out, temperature=torch.ones(n, device="cuda"),
                       top_k=torch.full((n,), c["top_k"] or 0, dtype=torch.int32, device="cuda"),
                       top_p=torch.full((n,), c["top_p"] if c["top_p"] is not None else 1.0, device="cuda"),
                       seeds=torch.full((n,), 1, dtype=torch.int64, device="cuda"),
                       counters=torch.arange(n, dtype=torch.int64, device="cuda"))
            drawn = set(out.cpu().tolist())
            kept = set(c["kept"][b])
            assert drawn <= kept, (c["top_k"], c["top_p"], b, sorted(drawn - kept))
            if len(kept) <= 12:
                assert drawn == kept                      # every kept token is reachable
