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


def test_plain_implementation_computes_what_the_references_own_graph_computes():
    """tests/golden/opt_reference_logits.json holds logits that the reference's OWN layer code
    produced (opt/model.py:272-524 with layers/attention.py, layers/transformer.py and hlo.py, run
    operation by operation on the CPU by tests/golden/reference_graph_eager.py): a left-padded batch of
    two prompts at every position, then three decode steps through its split prior/active softmax and
    its cache update.  The plain implementation, given each row without its padding, must agree at
    every real position: this pins its formulas (LayerNorm, the order of bias and scale, masks, the
    position offset, the head) to the reference's code rather than to a reading of it."""
    import sys
    sys.path.insert(0, GOLDEN)
    from reference_graph_eager import golden_tokens, golden_weights
    with open(os.path.join(GOLDEN, "opt_reference_logits.json")) as fp:
        g = json.load(fp)
    assert g["tokens"] == golden_tokens(g["config"])
    w = golden_weights(g["config"])
    prefill, decode = torch.tensor(g["prefill_logits"]), torch.tensor(g["decode_logits"])
    T0 = prefill.shape[1]
    worst = 0.0
    for b, start in enumerate(g["start_ids"]):
        ids = g["tokens"][b][start:]
        mine = P.forward_logits(ids, w, g["config"])
        theirs = torch.cat([prefill[b, start:], decode[b]])
        assert mine.shape == theirs.shape
        err = float((mine - theirs).abs().max() / theirs.abs().max())
        worst = max(worst, err)
        assert err <= 2e-5, f"row {b}: the plain implementation and the reference's graph differ by {err:.2e}"
    # the golden can fail: the same weights without the position offset of 2 are far off
    w2 = dict(w)
    w2["model.decoder.embed_positions.weight"] = torch.roll(w["model.decoder.embed_positions.weight"], 1, 0)
    off = P.forward_logits(g["tokens"][0], w2, g["config"])
    assert float((off - torch.cat([prefill[0], decode[0]])).abs().max()) > 1e-2
