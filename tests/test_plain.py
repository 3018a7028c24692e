"""The plain implementation checked against itself and against torch's own primitives, so that
the oracle of all other tests is not trusted blindly."""

import pytest
import torch

from helpers import TinyModel
from plain import opt_plain as P


def test_layer_norm_matches_torch():
    x = torch.randn(7, 96)
    w, b = torch.randn(96), torch.randn(96)
    assert torch.allclose(P.layer_norm(x, w, b, 1e-6), torch.nn.functional.layer_norm(x, (96,), w, b, 1e-6), atol=1e-5)
    assert torch.allclose(P.layer_norm(x, None, None, 1e-5), torch.nn.functional.layer_norm(x, (96,), None, None, 1e-5), atol=1e-5)


def test_attention_matches_torch_sdpa():
    T, H, d = 19, 3, 32
    q, k, v = torch.randn(H, T, d), torch.randn(H, T, d), torch.randn(H, T, d)
    s = P.attention_scores(q, k, d)
    c = P.attention_context(P.masked_softmax(s, P.causal_mask(T, T)[None]), v)
    ref = torch.nn.functional.scaled_dot_product_attention(q[None], k[None], v[None], is_causal=True)[0]
    assert torch.allclose(c, ref, atol=1e-5)


def test_causal_mask_and_window():
    m = P.causal_mask(3, 5, first_query_position=2)
    assert m.tolist() == [[True, True, True, False, False], [True, True, True, True, False], [True] * 5]
    m = P.causal_mask(4, 4, window=2)
    assert m.tolist() == [[True, False, False, False], [True, True, False, False], [False, True, True, False], [False, False, True, True]]


def test_position_offset_is_two():
    table = torch.arange(10.0)[:, None].repeat(1, 4)
    assert P.learned_position_embedding(torch.tensor([0, 3]), table)[:, 0].tolist() == [2.0, 5.0]


@pytest.mark.parametrize("name", ["A", "B"])
def test_causality_and_determinism(name):
    m = TinyModel(name, seed=1)
    ids = m.random_ids(24, seed=2)
    full = m.plain_logits(ids)
    part = P.forward_logits(ids[:10], m.tensors, m.cfg.to_dict())
    assert full.shape == (24, m.cfg.vocab_size)
    assert torch.allclose(full[:10], part, atol=1e-5)          # later tokens do not change earlier logits
    f64 = P.forward_logits(ids, m.tensors, m.cfg.to_dict(), dtype=torch.float64)
    assert float((full.double() - f64).abs().max()) < 1e-4 * float(f64.abs().max())


def test_options_matter():
    """Every option of configuration B changes the logits: none is silently ignored."""
    m = TinyModel("B", seed=1)
    ids = m.random_ids(12, seed=3)
    base = m.plain_logits(ids)
    for key, val in (("do_layer_norm_before", True), ("layer_norm_eps", 1e-1), ("num_attention_heads", 6)):
        cfg = dict(m.cfg.to_dict(), **{key: val})
        other = P.forward_logits(ids, m.tensors, cfg)
        assert float((other - base).abs().max()) > 1e-4, key


def test_sampling_filters():
    logits = torch.tensor([[2.0, 1.0, 0.5, 0.0, -1.0]])
    p = P.sampling_distribution(logits, temperature=1.0, top_k=2)
    assert (p[0] > 0).tolist() == [True, True, False, False, False] and abs(float(p.sum()) - 1) < 1e-6
    probs = torch.softmax(logits, -1)[0]
    top_p = float(probs[0] + probs[1] / 2)                      # reached inside the second token
    p = P.sampling_distribution(logits, top_p=top_p)
    assert (p[0] > 0).tolist() == [True, True, False, False, False]
    p = P.sampling_distribution(logits, top_p=float(probs[0]) - 1e-3)
    assert (p[0] > 0).tolist() == [True, False, False, False, False]
    p = P.sampling_distribution(logits, temperature=0.5, suppress=[0])
    assert p[0, 0] == 0 and torch.allclose(p[0, 1:], torch.softmax(logits[0, 1:] / 0.5, -1))
    assert int(P.greedy_token(torch.tensor([1.0, 3.0, 3.0]))) == 1


def test_on_device_sampling_of_the_reference():
    probs = torch.tensor([0.4, 0.3, 0.2, 0.06, 0.04])
    scores = probs.log()
    assert P.top_p_on_device(scores, 0.65).tolist() == [True, True, False, False, False]     # 0.4 < 0.65 <= 0.7
    assert P.top_p_on_device(scores, 0.65, top_p_min_tokens=4).tolist() == [True, True, True, True, False]
    assert P.top_p_on_device(scores, 0.3).tolist() == [True, False, False, False, False]
    assert P.multinomial_on_device(probs, 0.5) == 1 and P.multinomial_on_device(probs, 0.05) == 0
    assert P.multinomial_on_device(probs, 0.95) == 3 and P.multinomial_on_device(probs[:2], 0.5) == 0     # 0.4 / 0.7 > 0.5
    logits = torch.tensor([0.0, 3.0, 1.0, 2.5, -1.0, 2.0])
    tok, _ = P.sample_on_device(logits, top_k=3, top_p=1.0, top_p_min_tokens=1, temperature=1.0)
    assert tok == 1                                       # softmax(3, 2.5, 2) = .51 .31 .19: the first crosses one half
    tok, _ = P.sample_on_device(logits, top_k=3, top_p=1.0, top_p_min_tokens=1, temperature=4.0)
    assert tok == 3                                       # flatter: .38 .33 .29, the second crosses
    tok, _ = P.sample_on_device(logits, top_k=None, top_p=0.3, top_p_min_tokens=1, temperature=4.0)
    assert tok == 1                                       # top-p leaves one token
    tok, _ = P.sample_on_device(logits, top_k=None, top_p=0.3, top_p_min_tokens=3, temperature=4.0)
    assert tok == 3


def test_generation_config():
    from transformers_neuronx_b200 import GenerationConfig, NeuronConfig
    g = GenerationConfig()
    assert g.is_greedy() and g.for_row(0) == (50, 1.0, 1.0, 1) and g.eos_ids() is None
    g = GenerationConfig(do_sample=True, top_k=[5, None], top_p=[0.9, 1.0], temperature=[0.5, 2.0], top_p_min_tokens=[1, 3],
                         per_batch_line=True, dynamic=True, global_top_k=4, eos_token_id=[2, 7])
    assert not g.is_greedy() and g.for_row(0) == (4, 0.9, 0.5, 1) and g.for_row(1) == (4, 1.0, 2.0, 3) and g.eos_ids() == [2, 7]
    assert GenerationConfig(dynamic=True).is_greedy() is False          # a dynamic configuration always samples
    for bad in (dict(top_p=1.5), dict(top_p_min_tokens=0), dict(top_k=0), dict(temperature=0.0), dict(global_top_k=5),
                dict(top_k=[1, 2])):
        try:
            GenerationConfig(**bad)
        except ValueError:
            continue
        raise AssertionError(f"{bad} was accepted")
    import warnings
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        n = NeuronConfig(on_device_generation=g, fuse_qkv=True, quant="int8")
    assert n.on_device_generation is g and list(n.ignored) == ["quant"] and len(w) == 1


def test_greedy_generate():
    m = TinyModel("A", seed=4)
    out = P.greedy_generate(m.random_ids(6, seed=1), 5, m.tensors, m.cfg.to_dict())
    assert len(out) == 5 and all(0 <= t < m.cfg.vocab_size for t in out)


def test_decode_attention_plan_keeps_its_rules():
    """The plan of the decode attention kernel (blocks of 4, 8 or 16 warps, splits of the context) for
    every number of (row, head) pairs, head size and context: a split keeps at least eight pages, sixteen
    warps only serve heads of up to 128 dims, and the whole GPU is used once there is work for it."""
    from transformers_neuronx_b200.kernels.ops import decode_attention_plan
    for sms in (148, 132, 80):
        for head_dim in (64, 128, 256):
            for max_pages in (1, 7, 8, 31, 63, 128, 512):
                for pairs in list(range(1, 700, 7)) + [1024, 4096, 70000]:
                    warps, splits = decode_attention_plan(pairs, sms, head_dim, max_pages)
                    assert warps in (4, 8, 16) and 1 <= splits <= 32
                    assert warps < 16 or head_dim <= 128
                    assert splits == 1 or max_pages // splits >= 8, (pairs, max_pages, splits)
                    assert pairs * splits <= 4 * sms or splits == 1 or pairs * 10 <= sms * 27
                    if pairs > 4 * sms:
                        assert splits == 1, "more pairs than blocks fit at once: no split"
                    if max_pages >= 64 and pairs * 4 <= sms * 3:
                        assert pairs * splits * 2 > sms or splits == min(32, max_pages // 8), \
                            "few pairs and a long context: the splits fill the GPU as far as eight pages each allow"


def test_decode_attention_plan_beyond_the_blocks_the_gpu_holds():
    """More (row, head) pairs than blocks fit at once: many short contexts take blocks of four warps (a block's
    own cost counts), and where four-warp blocks would leave most of their last wave empty, eight-warp blocks
    run (measured: 8,192 pairs over 256 tokens 176 against 208 us; 1,280 pairs over 1,024 tokens 123 against 115 us)."""
    from transformers_neuronx_b200.kernels.ops import decode_attention_plan
    assert decode_attention_plan(8192, 148, 128, 16) == (4, 1)
    assert decode_attention_plan(4096, 148, 128, 8) == (4, 1)
    assert decode_attention_plan(1280, 148, 128, 64) == (8, 1)          # 2.2 waves of 592 blocks against 4.3 of 296
    assert decode_attention_plan(608, 148, 128, 128) == (8, 1)          # one block more than a wave of 592
    assert decode_attention_plan(896, 148, 128, 64) == (4, 1)           # 1.5 waves against 3.03
