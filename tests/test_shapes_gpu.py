"""The kernels at the sizes of the real OPT models (the layer shapes of 6.7B, 13B, 30B and 66B, one layer
each, and of 125M, 350M, 1.3B and 2.7B, two layers each; random weights).  The 32-bit engine against the plain implementation (restated on the GPU, and checked
against the CPU original on a short sequence) at 2e-5: a long portion, a mixed step of a portion
beside decode tokens, and decode steps; then the bfloat16 and float16 engines against the same
32-bit numbers, through the CTA-pair product, the swapped product with split-K, the split decode
attention and captured steps."""
import pytest
import torch

from helpers import TOLERANCE, plain_one_layer_on_gpu, rel_error
from plain import opt_plain

pytestmark = pytest.mark.gpu
SHAPES = {
    "6.7b": dict(hidden_size=4096, num_attention_heads=32, ffn_dim=16384),
    "13b": dict(hidden_size=5120, num_attention_heads=40, ffn_dim=20480),
    "30b": dict(hidden_size=7168, num_attention_heads=56, ffn_dim=28672),
    "66b": dict(hidden_size=9216, num_attention_heads=72, ffn_dim=36864),
}
# The small members of the family, two layers each, against the plain implementation itself on the CPU: head
# sizes 64 and 80, and the one model with post-norm blocks and a projected embedding (350M).
SMALL_SHAPES = {
    "125m": dict(hidden_size=768, num_attention_heads=12, ffn_dim=3072),
    "350m": dict(hidden_size=1024, num_attention_heads=16, ffn_dim=4096, word_embed_proj_dim=512, do_layer_norm_before=False),
    "1.3b": dict(hidden_size=2048, num_attention_heads=32, ffn_dim=8192),
    "2.7b": dict(hidden_size=2560, num_attention_heads=32, ffn_dim=10240),
}


def _build(shape, dtype, tensors=None, stored=torch.bfloat16):
    from transformers_neuronx_b200.config import OPTConfig
    from transformers_neuronx_b200.engine import build_model
    from transformers_neuronx_b200.models import opt as opt_arch
    from transformers_neuronx_b200.models.decoder import DecoderModel
    sizes = SHAPES[shape] if shape in SHAPES else dict(SMALL_SHAPES[shape], num_hidden_layers=2)
    cfg = OPTConfig.from_dict(dict(dict(vocab_size=50272, num_hidden_layers=1, max_position_embeddings=2048, init_std=0.02),
                                   **sizes))
    spec = opt_arch.build_spec(cfg)
    if tensors is None:
        g = torch.Generator(device="cuda:0").manual_seed(7)
        tensors = {}
        for s in DecoderModel(spec).tensor_specs():
            if s.tied_to is not None:
                continue
            t = torch.randn(s.shape, generator=g, device="cuda:0", dtype=torch.float32) * cfg.init_std
            tensors[s.name] = (1.0 + t) if s.kind == "norm_weight" else (t if s.kind == "norm_bias" else t.to(stored))
        tensors["lm_head.weight"] = tensors["model.decoder.embed_tokens.weight"]
    return build_model(spec, tensors, dtype, verbose=False), cfg, tensors


def _run(model, prompts):
    """A long portion of request 0 alone; then the rest of it beside the whole of request 1 and a
    decode token of request 2 (a mixed step); then three decode steps of all.  Returns the logits
    of every wanted row and, for each of them, (request, position)."""
    from transformers_neuronx_b200.engine import StepEntry, StepRunner
    runner = StepRunner(model, 16, 64, 4, 2048, use_cuda_graphs=True)
    for i in range(3):
        runner.add_request(i)
    p0, p1, p2 = prompts
    outs, where = [], []
    n0 = len(p0) - 3
    # (a step's logits are copied at once: a captured step hands out the same buffer at every replay)
    outs.append(runner.step([StepEntry(0, p0[:260], [0, 259]), StepEntry(2, p2[:-4], [])]).clone())
    where += [(0, 0), (0, 259)]
    outs.append(runner.step([StepEntry(0, p0[260:n0], [n0 - 261]), StepEntry(1, p1[:-3], [len(p1) - 4]),
                             StepEntry(2, [p2[-4]], [0])]).clone())
    where += [(0, n0 - 1), (1, len(p1) - 4), (2, len(p2) - 4)]
    for k in (3, 2, 1):
        outs.append(runner.step([StepEntry(i, [p[-k]], [0]) for i, p in enumerate(prompts)]).clone())
        where += [(i, len(p) - k) for i, p in enumerate(prompts)]
    return torch.cat([o.float() for o in outs]), where


@pytest.mark.parametrize("shape", list(SHAPES))
def test_layer_sizes_of_the_large_models(shape):
    tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(3, 50272, (n,), generator=g).tolist() for n in (300, 41, 77)]
        m32, cfg, tensors = _build(shape, "float32")
        w = {k: v.float() for k, v in tensors.items()}
        short = prompts[1][:9]
        cpu = opt_plain.forward_logits(short, {k: v.cpu() for k, v in tensors.items()}, cfg.to_dict())
        assert rel_error(plain_one_layer_on_gpu(short, w, cfg).cpu(), cpu) <= 1e-5, "the restatement is the plain implementation"
        plain = [plain_one_layer_on_gpu(p, w, cfg) for p in prompts]
        got32, where = _run(m32, prompts)
        want = torch.stack([plain[r][pos] for r, pos in where])
        for row, (r, pos) in enumerate(where):
            e = rel_error(got32[row], want[row])
            assert e <= TOLERANCE["float32"], f"{shape} float32: request {r} position {pos}: {e:.3e}"
        del m32, w, plain
        for dtype in ("bfloat16", "float16"):
            # a float16 engine is given the same values stored as float16 (random N(0, 0.02) values lose
            # bits going from bfloat16 storage to float16 only below 2^-14, which they do not reach)
            t16 = tensors if dtype == "bfloat16" else {k: (v.to(torch.float16) if v.dtype == torch.bfloat16 else v)
                                                         for k, v in tensors.items()}
            if dtype == "float16":
                t16["lm_head.weight"] = t16["model.decoder.embed_tokens.weight"]
            m16, _, _ = _build(shape, dtype, t16)
            got16, _ = _run(m16, prompts)
            del m16
            assert torch.isfinite(got16).all()
            for row, (r, pos) in enumerate(where):
                e = rel_error(got16[row], want[row])
                assert e <= TOLERANCE[dtype], f"{shape} {dtype}: request {r} position {pos}: {e:.3e}"
        from transformers_neuronx_b200.kernels import ops
        ops.raise_on_device_error()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = tf32


@pytest.mark.parametrize("shape", list(SMALL_SHAPES))
def test_layer_sizes_of_the_small_models(shape):
    """125M, 350M, 1.3B and 2.7B layer sizes (two layers, the real vocabulary): every wanted row of a long portion, a
    mixed step and three decode steps against the plain implementation on the CPU, in all three types."""
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(3, 50272, (n,), generator=g).tolist() for n in (300, 41, 77)]
    m32, cfg, tensors = _build(shape, "float32")
    cpu = {k: v.cpu() for k, v in tensors.items()}
    plain = [opt_plain.forward_logits(p, cpu, cfg.to_dict()) for p in prompts]
    got32, where = _run(m32, prompts)
    want = torch.stack([plain[r][pos] for r, pos in where])
    del m32
    for dtype in ("float32", "bfloat16", "float16"):
        if dtype == "float32":
            got = got32
        else:
            t16 = tensors if dtype == "bfloat16" else {k: (v.to(torch.float16) if v.dtype == torch.bfloat16 else v)
                                                         for k, v in tensors.items()}
            if dtype == "float16":
                t16["lm_head.weight"] = t16["model.decoder.embed_tokens.weight"]
            m16, _, _ = _build(shape, dtype, t16)
            got, _ = _run(m16, prompts)
            del m16
        for row, (r, pos) in enumerate(where):
            e = rel_error(got[row], want[row])
            assert e <= TOLERANCE[dtype], f"{shape} {dtype}: request {r} position {pos}: {e:.3e}"
    from transformers_neuronx_b200.kernels import ops
    ops.raise_on_device_error()

