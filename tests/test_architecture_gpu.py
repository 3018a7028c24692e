"""Another architecture through the front door, without a change to the package: a typed
configuration class and a spec builder are registered under a new name; a model folder with that
name in config.json is written by the random-weights mode, loaded by ``load_model``, generated from
by ``LLMEngine`` and replayed by the trace program's own function.  The toy architecture has a
recurrent mixer with state of its own in one layer, attention in the other, a feed-forward with
another activation, and a mixer whose cache is a kind of need that the package does not know (one
compressed vector per position, in pages of its own shape)."""
import dataclasses
import json
import math
import os
import tempfile

import pytest
import torch

from helpers import run_trace_inprocess
from plain import opt_plain as P

pytestmark = pytest.mark.gpu


@dataclasses.dataclass(frozen=True)
class ToyConfig:
    vocab_size: int = 131
    width: int = 48
    inner: int = 72
    heads: int = 3
    latent: int = 10
    decay: float = 0.85
    max_len: int = 160
    init_std: float = 0.3
    eos_token_id: int = 1
    architectures: tuple = ("ToyDecayForCausalLM",)
    model_type: str = "toy_decay"

    @classmethod
    def from_dict(cls, d):
        names = {f.name for f in dataclasses.fields(cls)}
        kw = {k: v for k, v in d.items() if k in names}
        kw["architectures"] = tuple(kw.get("architectures", ()))
        return cls(**kw)

    def to_dict(self):
        return dict(dataclasses.asdict(self), architectures=list(self.architectures))

    def save(self, folder):
        with open(os.path.join(folder, "config.json"), "w") as fp:
            json.dump(self.to_dict(), fp)


@dataclasses.dataclass(frozen=True)
class LatentNeed:
    """A paged cache of another shape than keys and values: one vector of `dim` numbers per position,
    always 32-bit.  It shares pages' bookkeeping with every other paged need that has no window."""
    dim: int
    window = None
    clear_on_admission = False

    @property
    def group_key(self):
        return ("paged", None)

    def make_storage(self, page_size, num_pages, max_slots, act_dtype, device):
        return torch.full((num_pages, page_size, self.dim), float("nan"), dtype=torch.float32, device=device)

    def bytes_per_page(self, page_size, act_dtype):
        return page_size * self.dim * 4


class _Spec:
    def __init__(self, kind, **kw):
        self.kind = kind
        self.__dict__.update(kw)


def _register():
    from transformers_neuronx_b200.cache import FixedStateNeed
    from transformers_neuronx_b200.config import Architecture, register_architecture
    from transformers_neuronx_b200.parts import Mixer, register_mixer, to_device
    from transformers_neuronx_b200.parts.spec import (AttentionSpec, DenseFeedForwardSpec, EmbeddingSpec, HeadSpec,
                                                      LayerSpec, LinearSpec, ModelSpec, NormSpec, PositionSpec,
                                                      ScheduleEntry)
    from transformers_neuronx_b200.weights import TensorSpec

    class DecayMixer(Mixer):
        """state_t = decay * state_{t-1} + h_t W;  residual += state_t."""
        def __init__(self, spec):
            self.spec = spec

        def tensor_specs(self):
            return [TensorSpec(self.spec.weight, (self.spec.hidden, self.spec.hidden), "matrix")]

        def load(self, tensors, device, act_dtype):
            self.w = to_device(tensors[self.spec.weight], device, torch.float32)

        def cache_need(self):
            return FixedStateNeed((self.spec.hidden,), "float32")

        def forward(self, ctx, h, residual):
            state, hb = ctx.cache(), ctx.host
            u = h.float() @ self.w.t()
            for r in range(ctx.n_requests):
                s = state[hb.slots[r]]
                for i in range(hb.q_start[r], hb.q_start[r] + hb.q_len[r]):
                    s = self.spec.decay * s + u[i]
                    residual[i] += s
                state[hb.slots[r]] = s

    class LatentMeanMixer(Mixer):
        """c_t = h_t Wc is kept per position (in pages); residual_t += mean_{j <= t}(c_j) Wu."""
        def __init__(self, spec):
            self.spec = spec

        def tensor_specs(self):
            s = self.spec
            return [TensorSpec(s.down, (s.latent, s.hidden), "matrix"), TensorSpec(s.up, (s.hidden, s.latent), "matrix")]

        def load(self, tensors, device, act_dtype):
            self.wc = to_device(tensors[self.spec.down], device, torch.float32)
            self.wu = to_device(tensors[self.spec.up], device, torch.float32)

        def cache_need(self):
            return LatentNeed(self.spec.latent)

        def forward(self, ctx, h, residual):
            cache, g, hb, ps = ctx.cache(), ctx.cache_group(), ctx.host, ctx.page_size
            flat = cache.view(-1, cache.shape[-1])
            flat[ctx.slot_mapping[g].long()] = h.float() @ self.wc.t()
            for r in range(ctx.n_requests):
                n_all = hb.ctx_len[r] + hb.q_len[r]
                pages = ctx.block_tables[g][r, :-(-n_all // ps)].long()
                c = cache[pages].reshape(-1, cache.shape[-1])[:n_all]
                mean = c.cumsum(0) / torch.arange(1, n_all + 1, device=c.device)[:, None]
                rows = slice(hb.q_start[r], hb.q_start[r] + hb.q_len[r])
                residual[rows] += mean[hb.ctx_len[r]:] @ self.wu.t()

    register_mixer("toy_decay_arch", DecayMixer)
    register_mixer("toy_latent_mean", LatentMeanMixer)

    def build_spec(cfg: ToyConfig):
        H, F, V = cfg.width, cfg.inner, cfg.vocab_size
        d = H // cfg.heads
        norm = lambda: NormSpec("layer_norm", H, 1e-5)
        lin = lambda name, i, o: LinearSpec(i, o, name + ".w", name + ".b")
        ff = lambda i, act: DenseFeedForwardSpec("dense", lin(f"l{i}.up", H, F), lin(f"l{i}.down", F, H), act)
        att = AttentionSpec("attention", H, cfg.heads, cfg.heads, d, 1 / math.sqrt(d), q=lin("l1.q", H, H),
                            k=lin("l1.k", H, H), v=lin("l1.v", H, H), out=lin("l1.o", H, H))
        layers = (LayerSpec("pre_norm", norm(), _Spec("toy_decay_arch", hidden=H, weight="l0.mix", decay=cfg.decay), norm(), ff(0, "silu")),
                  LayerSpec("pre_norm", norm(), att, norm(), ff(1, "gelu_new")),
                  LayerSpec("pre_norm", norm(), _Spec("toy_latent_mean", hidden=H, latent=cfg.latent, down="l2.c", up="l2.u"),
                            norm(), ff(2, "relu")))
        return ModelSpec(H, V, cfg.max_len, EmbeddingSpec("emb", V, H, None, PositionSpec("none")), layers,
                         tuple(ScheduleEntry(i, i) for i in range(3)),
                         HeadSpec("head", V, H, tied_to="emb", final_norm=norm()), eos_token_id=cfg.eos_token_id)

    register_architecture(Architecture(name="ToyDecayForCausalLM", model_type="toy_decay", config_class=ToyConfig,
                                       build_spec=build_spec))


def _plain(ids, w, cfg: ToyConfig):
    w = {k: v.float() for k, v in w.items()}
    x = w["emb"][torch.tensor(ids)]
    T, H = x.shape
    ln = lambda t: P.layer_norm(t, None, None)
    lin = lambda t, n: t @ w[n + ".w"].t() + w[n + ".b"]
    ff = lambda t, i, act: lin(P.activation(act, lin(t, f"l{i}.up")), f"l{i}.down")
    u = ln(x) @ w["l0.mix"].t()
    s, outs = torch.zeros(H), []
    for i in range(T):
        s = cfg.decay * s + u[i]; outs.append(s)
    x = x + torch.stack(outs)
    x = x + ff(ln(x), 0, "silu")
    h, d = ln(x), H // cfg.heads
    q, k, v = (lin(h, f"l1.{n}").view(T, cfg.heads, d).transpose(0, 1) for n in "qkv")
    p = P.masked_softmax(P.attention_scores(q, k, d), P.causal_mask(T, T, 0, None)[None])
    x = x + lin(P.attention_context(p, v).transpose(0, 1).reshape(T, H), "l1.o")
    x = x + ff(ln(x), 1, "gelu_new")
    c = ln(x) @ w["l2.c"].t()
    x = x + (c.cumsum(0) / torch.arange(1, T + 1)[:, None]) @ w["l2.u"].t()
    x = x + ff(ln(x), 2, "relu")
    return ln(x) @ w["emb"].t()


def test_a_registered_architecture_goes_through_the_front_door():
    from safetensors.torch import load_file
    from transformers_neuronx_b200.config import EngineConfig, load_config
    from transformers_neuronx_b200.engine import LLMEngine, load_model
    from transformers_neuronx_b200.models.decoder import DecoderModel
    from transformers_neuronx_b200.weights import write_model_folder
    _register()
    cfg = ToyConfig()
    with tempfile.TemporaryDirectory(prefix="tnx_toy_arch_") as folder:
        # the random-weights mode writes the folder: config.json with the new name, model.safetensors
        arch, _ = None, None
        from transformers_neuronx_b200.config import config_from_dict
        arch, typed = config_from_dict(cfg.to_dict())
        assert arch.name == "ToyDecayForCausalLM" and typed == cfg
        write_model_folder(folder, typed, DecoderModel(arch.build_spec(typed)).tensor_specs(), seed=3,
                           matrix_dtype=torch.float32)
        assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
        assert json.load(open(os.path.join(folder, "config.json")))["architectures"] == ["ToyDecayForCausalLM"]
        arch2, cfg2 = load_config(folder)
        assert arch2 is arch and cfg2 == cfg
        w = load_file(os.path.join(folder, "model.safetensors"))
        g = torch.Generator().manual_seed(9)
        seqs = {f"t{i}": torch.randint(2, cfg.vocab_size, (n,), generator=g).tolist() for i, n in enumerate((70, 33, 121))}
        want = {r: _plain(ids, w, cfg) for r, ids in seqs.items()}

        # trace replay: portions of changing size and single tokens, requests mixed, pages used again
        steps, pos, k = [], {r: 0 for r in seqs}, 0
        sizes = [9, 2, 1, 30, 1, 17, 5, 1, 40]
        live = ["t0", "t1"]
        waiting = ["t2"]
        while live:
            entries, end = [], []
            for r in list(live):
                n = min(sizes[k % len(sizes)], len(seqs[r]) - pos[r]); k += 1
                entries.append({"id": r, "tokens": seqs[r][pos[r]:pos[r] + n], "want": [0, n - 1] if n > 1 else [0]})
                pos[r] += n
                if pos[r] == len(seqs[r]):
                    end.append(r); live.remove(r)
                    if waiting:
                        live.append(waiting.pop())
            steps.append({"step": len(steps), "entries": entries, "end": end})
        res = run_trace_inprocess(folder, "float32", steps, 64 * 2 + 128)
        at = {r: 0 for r in seqs}
        worst = 0.0
        for s in steps:
            row = 0
            for e in s["entries"]:
                for wpos in e["want"]:
                    got = torch.from_numpy(res[s["step"]][row].copy()); row += 1
                    ref = want[e["id"]][at[e["id"]] + wpos]
                    worst = max(worst, float((got - ref).abs().max() / ref.abs().max()))
                at[e["id"]] += len(e["tokens"])
        assert worst <= 5e-5, worst

        # the engine: scheduler, step function and sampler above the same model
        model, typed = load_model(folder, "float32", verbose=False)
        eng = LLMEngine(model, EngineConfig(dtype="float32", max_num_seqs=2, max_batch_tokens=24, max_portion=11,
                                            max_tokens=256), eos_token_id=typed.eos_token_id)
        prompts = [seqs["t0"][:25], seqs["t1"][:7], seqs["t2"][:40]]
        outs = eng.generate(prompts, 10, stop_on_eos=False)
        for prompt, out in zip(prompts, outs):
            seq = list(prompt)
            for tok in out:
                lg = _plain(seq, w, cfg)[-1]
                top = torch.topk(lg, 2).values
                if tok != int(lg.argmax()):
                    assert float(top[0] - top[1]) / float(lg.abs().max()) < 1e-4
                    break
                seq.append(tok)
        eng.runner.cache.check()
        assert eng.runner.cache.slots.num_free == 2


def test_an_unknown_architecture_names_the_known_ones():
    from transformers_neuronx_b200.config import resolve_architecture
    with pytest.raises(KeyError, match="OPTForCausalLM"):
        resolve_architecture({"architectures": ["NoSuchModel"], "model_type": "none"})
