"""The kernels at the sizes of real OPT models (6.7B, 13B, 30B layer shapes, one layer each, random
weights): the bfloat16 engine against the 32-bit engine on the same weights, through a long prompt
(the CTA-pair matrix product), portions, and decode steps of a small batch (the swapped product with
split-K, the split decode attention, CUDA graphs); and the 32-bit engine against the plain
implementation at the 6.7B shape."""
import pytest
import torch

from helpers import TOLERANCE
from plain import opt_plain

pytestmark = pytest.mark.gpu
SHAPES = {
    "6.7b": dict(hidden_size=4096, num_attention_heads=32, ffn_dim=16384),
    "13b": dict(hidden_size=5120, num_attention_heads=40, ffn_dim=20480),
    "30b": dict(hidden_size=7168, num_attention_heads=56, ffn_dim=28672),
}


def _build(shape, dtype, tensors=None):
    from transformers_neuronx_b200.config import OPTConfig
    from transformers_neuronx_b200.engine import build_model
    from transformers_neuronx_b200.models import opt as opt_arch
    from transformers_neuronx_b200.models.decoder import DecoderModel
    cfg = OPTConfig.from_dict(dict(SHAPES[shape], vocab_size=50272, num_hidden_layers=1, max_position_embeddings=2048,
                                   init_std=0.02))
    spec = opt_arch.build_spec(cfg)
    if tensors is None:
        g = torch.Generator(device="cuda:0").manual_seed(7)
        tensors = {}
        for s in DecoderModel(spec).tensor_specs():
            if s.tied_to is not None:
                continue
            t = torch.randn(s.shape, generator=g, device="cuda:0", dtype=torch.float32) * cfg.init_std
            tensors[s.name] = (1.0 + t) if s.kind == "norm_weight" else (t if s.kind == "norm_bias" else t.to(torch.bfloat16))
        tensors["lm_head.weight"] = tensors["model.decoder.embed_tokens.weight"]
    return build_model(spec, tensors, dtype, verbose=False), cfg, tensors


def _run(model, cfg, prompts):
    """Prefill in one step (all rows wanted for the first request's tail), then decode three steps."""
    from transformers_neuronx_b200.engine import StepEntry, StepRunner
    runner = StepRunner(model, 16, 64, 4, 2048, use_cuda_graphs=True)
    outs = []
    for i in range(len(prompts)):
        runner.add_request(i)
    entries = [StepEntry(i, p[:-3], [len(p) - 8, len(p) - 4]) for i, p in enumerate(prompts)]
    outs.append(runner.step(entries).float().cpu())
    for k in (3, 2, 1):
        outs.append(runner.step([StepEntry(i, [p[-k]], [0]) for i, p in enumerate(prompts)]).float().cpu())
    return torch.cat(outs)


@pytest.mark.parametrize("shape", list(SHAPES))
def test_bf16_engine_against_32bit_engine(shape):
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(3, 50272, (n,), generator=g).tolist() for n in (300, 41)]
    m16, cfg, tensors = _build(shape, "bfloat16")
    got = _run(m16, cfg, prompts)
    del m16
    m32, _, _ = _build(shape, "float32", tensors)
    want = _run(m32, cfg, prompts)
    err = float((got - want).abs().max()) / float(want.abs().max())
    assert torch.isfinite(got).all() and err <= TOLERANCE["bfloat16"], f"{shape}: {err:.3e}"
    if shape == "6.7b":
        cpu = {k: v.cpu() for k, v in tensors.items()}
        for i, p in enumerate(prompts):
            plain = opt_plain.forward_logits(p, cpu, cfg.to_dict())
            rows = [len(p) - 8, len(p) - 4]                        # the wanted places of the prefill step
            mine = want[2 * i:2 * i + 2]
            e = float((mine - plain[rows]).abs().max()) / float(plain[rows].abs().max())
            assert e <= TOLERANCE["float32"], f"32-bit engine vs plain, request {i}: {e:.3e}"
