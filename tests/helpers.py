"""Shared by the tests: two tiny OPT configurations that differ in every size and option, model
folders with seeded random weights (made in a temporary folder), the plain implementation's
logits, trace builders and the comparison with its tolerances."""
from __future__ import annotations

import io
import json
import os
import tempfile

import numpy as np
import torch

from plain import opt_plain
from transformers_neuronx_b200.config import OPTConfig
from transformers_neuronx_b200.models import opt as opt_arch
from transformers_neuronx_b200.models.decoder import DecoderModel
from transformers_neuronx_b200.weights import load_tensors, write_model_folder

CONFIG_A = dict(vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, ffn_dim=256,
                max_position_embeddings=128, word_embed_proj_dim=64, do_layer_norm_before=True,
                enable_bias=True, layer_norm_elementwise_affine=True, layer_norm_eps=1e-5,
                activation_function="relu", init_std=0.02, architectures=["OPTForCausalLM"], model_type="opt")
CONFIG_B = dict(vocab_size=1000, hidden_size=96, num_hidden_layers=3, num_attention_heads=3, ffn_dim=320,
                max_position_embeddings=256, word_embed_proj_dim=48, do_layer_norm_before=False,
                enable_bias=False, layer_norm_elementwise_affine=False, layer_norm_eps=1e-6,
                activation_function="relu", init_std=0.05, architectures=["OPTForCausalLM"], model_type="opt")
# Sizes that leave the fast kernels' rules: head size 48 (no power of two), a feed-forward width and
# an embedding width that are no multiples of 8 (the tensor-core product refuses them), an odd vocabulary,
# no final LayerNorm although the layers are pre-norm.
CONFIG_C = dict(vocab_size=333, hidden_size=96, num_hidden_layers=2, num_attention_heads=2, ffn_dim=100,
                max_position_embeddings=80, word_embed_proj_dim=36, do_layer_norm_before=True,
                _remove_final_layer_norm=True, enable_bias=True, layer_norm_elementwise_affine=False,
                layer_norm_eps=1e-4, activation_function="relu", init_std=0.04,
                architectures=["OPTForCausalLM"], model_type="opt")
# Head size 128 (the size of the large OPT models): the tcgen05 attention kernel, longer contexts.
CONFIG_D = dict(vocab_size=2003, hidden_size=256, num_hidden_layers=2, num_attention_heads=2, ffn_dim=520,
                max_position_embeddings=600, word_embed_proj_dim=256, do_layer_norm_before=True, enable_bias=True,
                layer_norm_elementwise_affine=True, layer_norm_eps=1e-5, activation_function="relu", init_std=0.03,
                architectures=["OPTForCausalLM"], model_type="opt")
# Head size 64 (the size of the small OPT models), three heads, post-norm, a projected embedding.
CONFIG_E = dict(vocab_size=1501, hidden_size=192, num_hidden_layers=2, num_attention_heads=3, ffn_dim=264,
                max_position_embeddings=420, word_embed_proj_dim=96, do_layer_norm_before=False, enable_bias=True,
                layer_norm_elementwise_affine=True, layer_norm_eps=1e-5, activation_function="relu", init_std=0.03,
                architectures=["OPTForCausalLM"], model_type="opt")
# Head size 80 (OPT-2.7B's: 2,560 / 32): the tcgen05 attention kernel's layout of 128 with a partly filled
# second slice; the decode kernel's lanes that own no dims.
CONFIG_F = dict(vocab_size=777, hidden_size=240, num_hidden_layers=2, num_attention_heads=3, ffn_dim=328,
                max_position_embeddings=400, word_embed_proj_dim=240, do_layer_norm_before=True, enable_bias=True,
                layer_norm_elementwise_affine=True, layer_norm_eps=1e-5, activation_function="relu", init_std=0.03,
                architectures=["OPTForCausalLM"], model_type="opt")
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C, "D": CONFIG_D, "E": CONFIG_E, "F": CONFIG_F}

# Largest allowed |engine - plain| as a fraction of the largest |plain logit| of the compared rows.
# float32: both sides compute in 32-bit and differ by the order of additions only.
# bfloat16: activations are rounded to 8 bits of mantissa between kernels (relative step 2^-8).
# float16: 11 bits of mantissa (relative step 2^-11), so an eighth of the bfloat16 bound.
TOLERANCE = {"float32": 2e-5, "bfloat16": 2e-2, "float16": 2.5e-3}
TORCH_DTYPE = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def storage_for(dtype: str) -> torch.dtype:
    """The type a test model's matrices are stored in for an engine of `dtype`: the engine's own 16-bit
    type (no rounding at load), bfloat16 for the 32-bit engine."""
    return torch.float16 if dtype == "float16" else torch.bfloat16


def rel_error(got, want) -> float:
    """Largest |got - want| as a fraction of the largest |want| (both moved to the CPU in 32-bit)."""
    got, want = got.detach().float().cpu(), want.detach().float().cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


class TinyModel:
    """A model folder with random weights plus what the tests need to know about it."""

    def __init__(self, name: str, seed: int = 0, root: str = None, matrix_dtype=torch.bfloat16, overrides=None):
        self.name = name
        self.cfg_dict = dict(CONFIGS[name], **(overrides or {}))
        self.cfg = OPTConfig.from_dict(self.cfg_dict)
        self._tmp = tempfile.TemporaryDirectory(prefix=f"tnx_tiny_{name}_", dir=root)
        self.folder = self._tmp.name
        specs = DecoderModel(opt_arch.build_spec(self.cfg)).tensor_specs()
        write_model_folder(self.folder, self.cfg, specs, seed, matrix_dtype=matrix_dtype)
        # The plain implementation gets the file's tensors through the `safetensors` package, not
        # through the engine's own reader: a fault that the engine's writer and reader share would
        # otherwise be invisible.  (The engine's writer still made the file; tests/test_config_weights.py
        # checks it against the package in both directions.)
        from safetensors.torch import load_file
        self.plain_tensors = load_file(os.path.join(self.folder, "model.safetensors"))
        self.tensors = load_tensors(self.folder, specs)        # as the engine reads them (ties resolved)
        self._plain_cache = {}

    def plain_logits(self, ids) -> torch.Tensor:
        key = tuple(int(i) for i in ids)
        if key not in self._plain_cache:
            self._plain_cache[key] = opt_plain.forward_logits(list(key), self.plain_tensors, self.cfg.to_dict())
        return self._plain_cache[key]

    def random_ids(self, n: int, seed: int):
        g = torch.Generator().manual_seed(seed)
        ids = torch.randint(3, self.cfg.vocab_size, (n,), generator=g).tolist()
        ids[0] = self.cfg.bos_token_id
        return ids


def trace_lines(steps) -> list:
    return [json.dumps(s) for s in steps]


def run_trace_inprocess(folder: str, dtype: str, steps, max_tokens: int):
    """Runs the replay program's own function in this process; returns {step: array [wanted, vocab]}."""
    from transformers_neuronx_b200.engine.replay import replay
    out_dir = tempfile.mkdtemp(prefix="tnx_trace_out_")
    sink = io.StringIO()
    rc = replay(folder, dtype, out_dir, max_tokens, lines=trace_lines(steps), out=sink)
    assert rc == 0
    done = [l for l in sink.getvalue().splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in steps]
    res = {}
    for s in steps:
        p = os.path.join(out_dir, f"{s['step']}.f32")
        n_want = sum(len(e.get("want", [])) for e in s["entries"])
        if n_want:
            arr = np.fromfile(p, dtype="<f4")
            res[s["step"]] = arr.reshape(n_want, -1)
        else:
            assert not os.path.exists(p)
    return res


def live_tokens_rounded(counts, unit=64):
    return sum(-(-c // unit) * unit for c in counts)


def compare_trace(model: TinyModel, requests: dict, steps, results, dtype: str):
    """requests: {id: full token list}.  Checks every wanted row against the plain logits of its
    request at its position; returns the largest relative error seen."""
    pos = {rid: 0 for rid in requests}
    worst = 0.0
    for s in steps:
        row = 0
        for e in s["entries"]:
            rid, n = e["id"], len(e["tokens"])
            assert list(e["tokens"]) == list(requests[rid][pos[rid]:pos[rid] + n]), "trace builder bug"
            plain = model.plain_logits(requests[rid]) if e.get("want") else None
            for w in e.get("want", []):
                got = torch.from_numpy(results[s["step"]][row].copy())
                want = plain[pos[rid] + w]
                scale = float(want.abs().max())
                err = float((got - want).abs().max()) / scale
                worst = max(worst, err)
                assert err <= TOLERANCE[dtype], (
                    f"{dtype} step {s['step']} request {rid} position {pos[rid] + w}: "
                    f"relative error {err:.3e} > {TOLERANCE[dtype]:.1e} "
                    f"(first wrong place: argmax got {int(got.argmax())}, plain {int(want.argmax())})")
                row += 1
            pos[rid] += n
    return worst


def check_greedy(model: TinyModel, dtype: str, prompt, out, suppress=()) -> int:
    """Every token of a greedy continuation against the plain implementation, teacher-forced on the
    engine's own tokens (one plain pass over prompt + out gives the logits before each of them): a
    token must be the plain argmax, or lose to it by no more than twice the tolerance of `dtype` (a
    tie that rounding may decide either way).  Returns how many tokens were such ties; all
    len(out) tokens are compared."""
    seq = list(prompt) + list(out)
    logits = model.plain_logits(seq)
    ties = 0
    for i, tok in enumerate(out):
        lg = logits[len(prompt) - 1 + i].clone()
        for s_ in suppress:
            lg[s_] = -float("inf")
        best = int(lg.argmax())
        if tok != best:
            gap = float(lg[best] - lg[tok]) / float(lg[lg > -1e30].abs().max())
            assert gap <= 2 * TOLERANCE[dtype], f"{dtype}: token {i} is {tok}, plain {best}, gap {gap:.2e}"
            ties += 1
    return ties


def check_sampled(model: TinyModel, dtype: str, prompt, out, temperature, seed, top_k=None, top_p=None,
                  suppress=()) -> int:
    """Every token of a sampled continuation against a draw from the plain logits with the same
    uniform number (a function of the request's seed and the token's index), teacher-forced on the
    engine's tokens.  A token may differ only where the number lies so close to a summed
    probability that the rounding of `dtype` can move the boundary across it.  Returns the number
    of such tokens."""
    seq = list(prompt) + list(out)
    logits = model.plain_logits(seq)
    close = 0
    for i, tok in enumerate(out):
        lg = logits[len(prompt) - 1 + i]
        probs = opt_plain.sampling_distribution(lg, temperature, top_k, top_p, list(suppress) or None)
        u = opt_plain.philox_uniform(seed, i)
        want, dist = opt_plain.draw_in_index_order(probs, u)
        if tok != want:
            # a change of every score by at most d moves a summed probability by at most about 2 d
            slack = 1e-4 + 4 * TOLERANCE[dtype] * float(lg.abs().max()) / temperature
            assert dist <= slack, f"{dtype}: token {i} is {tok}, plain draws {want} (u={u:.6f}, {dist:.2e} from a boundary)"
            close += 1
    return close


def plain_one_layer_on_gpu(ids, w, cfg, dev="cuda:0"):
    """opt_plain.forward_logits for a model of ONE pre-norm layer with biases, affine norms and no
    projections, restated with the tensors on the GPU (torch in 32-bit; the caller switches TF32 off):
    the plain implementation runs on the CPU and would take minutes at the sizes of the large models.
    A test that uses this checks it against the plain implementation on a short sequence first."""
    import math
    P_, L0 = "model.decoder.", "model.decoder.layers.0."
    H, heads = cfg.hidden_size, cfg.num_attention_heads
    d, T = H // heads, len(ids)
    ln = lambda x, a, b: torch.nn.functional.layer_norm(x, (H,), w[a], w[b], cfg.layer_norm_eps)
    x = w[P_ + "embed_tokens.weight"][torch.tensor(ids, device=dev)] + \
        w[P_ + "embed_positions.weight"][torch.arange(T, device=dev) + 2]
    h = ln(x, L0 + "self_attn_layer_norm.weight", L0 + "self_attn_layer_norm.bias")
    q, k, v = ((h @ w[L0 + f"self_attn.{n}_proj.weight"].t() + w[L0 + f"self_attn.{n}_proj.bias"])
               .view(T, heads, d).transpose(0, 1) for n in "qkv")
    s_ = (q @ k.transpose(1, 2)) / math.sqrt(d)
    s_ = s_.masked_fill(torch.ones(T, T, device=dev, dtype=torch.bool).triu(1), float("-inf"))
    a = (torch.softmax(s_, -1) @ v).transpose(0, 1).reshape(T, H)
    x = x + a @ w[L0 + "self_attn.out_proj.weight"].t() + w[L0 + "self_attn.out_proj.bias"]
    h = ln(x, L0 + "final_layer_norm.weight", L0 + "final_layer_norm.bias")
    x = x + torch.relu(h @ w[L0 + "fc1.weight"].t() + w[L0 + "fc1.bias"]) @ w[L0 + "fc2.weight"].t() + w[L0 + "fc2.bias"]
    return ln(x, P_ + "final_layer_norm.weight", P_ + "final_layer_norm.bias") @ w[P_ + "embed_tokens.weight"].t()
