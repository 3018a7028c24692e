"""One layer at the sizes of OPT-6.7B (hidden 4096, 32 heads x 128, ffn 16384, vocabulary 50272):
the products, tile plans and attention shapes that the benchmark runs, which the tiny
configurations never reach, compared with a 32-bit computation.

The plain implementation (tests/plain/opt_plain.py) works on the CPU and would take minutes at this
size, so its formulas are restated below with the tensors on the GPU (torch in 32-bit, TF32 off);
the first assertion checks the restatement against the plain implementation on a short sequence.
"""
import pytest
import torch

from helpers import opt_plain, plain_one_layer_on_gpu, rel_error

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

SIZES = dict(vocab_size=50272, hidden_size=4096, num_hidden_layers=1, num_attention_heads=32, ffn_dim=16384,
             max_position_embeddings=2048, word_embed_proj_dim=4096, do_layer_norm_before=True, enable_bias=True,
             layer_norm_elementwise_affine=True, activation_function="relu", init_std=0.02,
             architectures=["OPTForCausalLM"], model_type="opt")
P = "model.decoder."
L0 = P + "layers.0."


def _build():
    from transformers_neuronx_b200.config import OPTConfig
    from transformers_neuronx_b200.engine import build_model
    from transformers_neuronx_b200.models import opt as opt_arch
    from transformers_neuronx_b200.models.decoder import DecoderModel
    cfg = OPTConfig.from_dict(SIZES)
    spec = opt_arch.build_spec(cfg)
    g = torch.Generator(device=DEV).manual_seed(0)
    tensors = {}
    for s in DecoderModel(spec).tensor_specs():
        if s.tied_to is not None:
            continue
        t = torch.randn(s.shape, generator=g, device=DEV, dtype=torch.float32) * cfg.init_std
        tensors[s.name] = 1.0 + t if s.kind == "norm_weight" else (t if s.kind == "norm_bias" else t.to(torch.bfloat16))
    tensors["lm_head.weight"] = tensors[P + "embed_tokens.weight"]
    return build_model(spec, tensors, "bfloat16", verbose=False), cfg, tensors


def test_one_layer_at_the_sizes_of_the_benchmark():
    from transformers_neuronx_b200.engine import StepEntry, StepRunner
    from transformers_neuronx_b200.kernels import ops
    tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        model, cfg, tensors = _build()
        w = {k: v.float() for k, v in tensors.items()}
        gen = torch.Generator().manual_seed(9)
        lens = [2040, 1500, 700, 300, 130, 64, 17, 5]
        seqs = [torch.randint(3, cfg.vocab_size, (n + 6,), generator=gen).tolist() for n in lens]
        plain = lambda ids: plain_one_layer_on_gpu(ids, w, cfg)

        short = seqs[6][:17]
        cpu = opt_plain.forward_logits(short, {k: v.cpu() for k, v in tensors.items()}, cfg.to_dict())
        assert rel_error(plain(short).cpu(), cpu) <= 1e-5, "the restatement on the GPU is the plain implementation"

        tol = 2e-2
        runner = StepRunner(model, 16, sum((n + 6 + 15) // 16 for n in lens) + 4, 8, 2048, use_cuda_graphs=True)
        for i in range(8):
            runner.add_request(i)
        # a whole prompt of 2,040 tokens (CTA-pair products, tcgen05 attention)
        out = runner.step([StepEntry(0, seqs[0][:lens[0]], [lens[0] - 1, 100, 1000])])
        assert rel_error(out, plain(seqs[0][:lens[0]])[[lens[0] - 1, 100, 1000]]) <= tol
        # seven prompts of 5 to 1,500 tokens in one step
        out = runner.step([StepEntry(i, seqs[i][:lens[i]], [lens[i] - 1]) for i in range(1, 8)])
        assert rel_error(out, torch.stack([plain(seqs[i][:lens[i]])[-1] for i in range(1, 8)])) <= tol
        # decode at batch 8 (captured steps: cluster split-K products, attention that appends), then 1, 2 and 4
        for step in range(3):
            out = runner.step([StepEntry(i, [seqs[i][lens[i] + step]], [0]) for i in range(8)])
            assert rel_error(out, torch.stack([plain(seqs[i][:lens[i] + step + 1])[-1] for i in range(8)])) <= tol
        for nb, step in ((1, 3), (2, 4), (4, 5)):
            out = runner.step([StepEntry(i, [seqs[i][lens[i] + step]], [0]) for i in range(nb)])
            assert rel_error(out, torch.stack([plain(seqs[i][:lens[i] + step + 1])[-1] for i in range(nb)])) <= tol, nb
            runner.step([StepEntry(i, [seqs[i][lens[i] + step]], []) for i in range(nb, 8)])
        for i in range(8):
            runner.finish(i)
        # a 512-token portion beside a decode token
        runner.add_request("p"); runner.add_request("q")
        runner.step([StepEntry("q", seqs[1][:900], [])])
        out = runner.step([StepEntry("p", seqs[0][:512], [511]), StepEntry("q", [seqs[1][900]], [0])])
        assert rel_error(out, torch.stack([plain(seqs[0][:512])[-1], plain(seqs[1][:901])[-1]])) <= tol
        for r in ("p", "q"):
            runner.finish(r)
        # short prompts alone: 65..255 tokens take kernels of their own (128 x 256 tiles, K split in clusters)
        for n in (130, 250, 66):
            runner.add_request("s")
            out = runner.step([StepEntry("s", seqs[2][:n], [n - 1, 0])])
            want = plain(seqs[2][:n])
            assert rel_error(out, want[[n - 1, 0]]) <= tol, n
            runner.finish("s")
        ops.raise_on_device_error()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = tf32
