"""Each part alone against the plain implementation, and a model put together from toy parts that
are defined here: a mixer with state of its own (fixed size per request), a gated feed-forward, a
position encoding applied inside the mixer, a schedule that runs a layer twice and lets a layer read
another layer's cache.  None of it changes a file of the package."""
import math

import pytest
import torch

from helpers import TinyModel
from plain import opt_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ctx(n_tokens, dtype):
    from transformers_neuronx_b200.parts import StepContext
    ctx = StepContext(torch.device(DEV), dtype)
    ctx.n_tokens = n_tokens
    return ctx


def rel_err(got, want):
    return float((got.float() - want.float()).abs().max()) / max(float(want.float().abs().max()), 1e-30)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1e-2)])
def test_linear_norm_feed_forward_alone(dtype, tol):
    from transformers_neuronx_b200.parts import build_part
    from transformers_neuronx_b200.parts.spec import DenseFeedForwardSpec, LinearSpec, NormSpec
    H, F, N = 96, 328, 21
    g = torch.Generator().manual_seed(0)
    t = {"n.weight": 1 + 0.1 * torch.randn(H, generator=g), "n.bias": 0.1 * torch.randn(H, generator=g),
         "fc1.weight": (torch.randn(F, H, generator=g) / 10).bfloat16(), "fc1.bias": torch.randn(F, generator=g).bfloat16(),
         "fc2.weight": (torch.randn(H, F, generator=g) / 18).bfloat16(), "fc2.bias": torch.randn(H, generator=g).bfloat16()}
    norm = build_part("norm", NormSpec("layer_norm", H, 1e-3, "n.weight", "n.bias"))
    ff = build_part("feed_forward", DenseFeedForwardSpec("dense", LinearSpec(H, F, "fc1.weight", "fc1.bias"),
                                                         LinearSpec(F, H, "fc2.weight", "fc2.bias"), "relu"))
    for p in (norm, ff):
        p.load(t, torch.device(DEV), dtype)
    x = torch.randn(N, H, generator=g).to(DEV)
    ctx = _ctx(N, dtype)
    h = ctx.empty(N, H)
    norm.forward(ctx, x, out_act=h)
    tf = {k: v.float() for k, v in t.items()}
    want_h = P.layer_norm(x.cpu(), tf["n.weight"], tf["n.bias"], 1e-3)
    assert rel_err(h, want_h.to(DEV)) <= tol
    res = x.clone()
    ff.forward(ctx, h, res)
    want = x.cpu() + P.feed_forward(h.float().cpu(), tf, "", "relu")
    assert rel_err(res, want.to(DEV)) <= tol
    from transformers_neuronx_b200.kernels.ops import KernelError
    with pytest.raises(KernelError, match="not built"):
        build_part("feed_forward", DenseFeedForwardSpec("dense", LinearSpec(H, F, "a", None), LinearSpec(F, H, "b", None), "solu"))
    with pytest.raises(KeyError, match="registered"):
        build_part("norm", NormSpec("rms_norm_of_tomorrow", H, 1e-5))


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 2e-2)])
def test_attention_part_alone(name, dtype, tol):
    """The attention mixer with its cache, fed a sequence in two portions, against the plain
    attention of the whole sequence."""
    from transformers_neuronx_b200.engine import StepEntry, StepRunner, build_model
    from transformers_neuronx_b200.parts.spec import (EmbeddingSpec, HeadSpec, LayerSpec, ModelSpec, ScheduleEntry)
    from transformers_neuronx_b200.models import opt as opt_arch
    tiny = TinyModel(name, seed=31)
    spec = opt_arch.build_spec(tiny.cfg)
    model = build_model(spec, tiny.tensors, dtype, verbose=False)
    mixer = model.blocks[0].mixer
    runner = StepRunner(model, 16, 8, 2, 128)
    runner.add_request("a")
    H = tiny.cfg.hidden_size
    T = 50
    hs = torch.randn(T, H, generator=torch.Generator().manual_seed(1))
    outs = []
    for lo, hi in ((0, 33), (33, 50)):
        ctx = runner.prepare([StepEntry("a", [3] * (hi - lo), [])])
        ctx.cache_id = 0
        h = hs[lo:hi].to(DEV).to(model.act_dtype)
        res = torch.zeros(hi - lo, H, device=DEV)
        mixer.forward(ctx, h, res)
        outs.append(res)
    got = torch.cat(outs)
    w = {k: v.float() for k, v in tiny.plain_tensors.items()}
    hin = hs.to(model.act_dtype).float()
    want = P.multi_head_attention(hin, w, "model.decoder.layers.0.self_attn.", tiny.cfg.num_attention_heads)
    assert rel_err(got, want.to(DEV)) <= tol


# ---- toy parts, defined here --------------------------------------------------------------------------
def _register_toys():
    from transformers_neuronx_b200.cache import FixedStateNeed
    from transformers_neuronx_b200.parts import (FeedForward, Mixer, PositionEncoding, register_feed_forward,
                                                 register_mixer, register_position, to_device)
    from transformers_neuronx_b200.weights import TensorSpec

    class DecayMixer(Mixer):
        """state_t = decay * state_{t-1} + h_t W;  residual += state_t.  State of fixed size per request."""
        def __init__(self, spec):
            self.spec = spec

        def tensor_specs(self):
            return [TensorSpec(self.spec.weight, (self.spec.hidden, self.spec.hidden), "matrix")]

        def load(self, tensors, device, act_dtype):
            self.w = to_device(tensors[self.spec.weight], device, torch.float32)

        def cache_need(self):
            return FixedStateNeed((self.spec.hidden,), "float32")

        def forward(self, ctx, h, residual):
            state = ctx.cache()                                  # [slots, hidden]
            u = h.float() @ self.w.t()
            hb = ctx.host
            for r in range(ctx.n_requests):                     # a portion is run in order, from the state before it;
                s = state[hb.slots[r]]                          # a new request finds its slot's state zeroed
                for i in range(hb.q_start[r], hb.q_start[r] + hb.q_len[r]):
                    s = self.spec.decay * s + u[i]
                    residual[i] += s
                state[hb.slots[r]] = s

    class GatedFeedForward(FeedForward):
        """residual += (sigmoid(h Wg) * (h Wu)) Wd: a feed-forward whose inner values route themselves."""
        def __init__(self, spec):
            self.spec = spec

        def tensor_specs(self):
            s = self.spec
            return [TensorSpec(s.prefix + "gate", (s.inner, s.hidden)), TensorSpec(s.prefix + "up", (s.inner, s.hidden)),
                    TensorSpec(s.prefix + "down", (s.hidden, s.inner))]

        def load(self, tensors, device, act_dtype):
            s = self.spec
            self.g, self.u, self.d = (to_device(tensors[s.prefix + n], device, torch.float32) for n in ("gate", "up", "down"))

        def forward(self, ctx, h, residual):
            x = h.float()
            residual += (torch.sigmoid(x @ self.g.t()) * (x @ self.u.t())) @ self.d.t()

    class SignFlipPositions(PositionEncoding):
        """A stand-in for an encoding applied to queries and keys: odd positions change sign."""
        def __init__(self, spec):
            self.spec = spec

        def rotate(self, ctx, q, k):
            sign = (1 - 2 * (ctx.positions % 2)).to(q.dtype)[:, None]
            q.mul_(sign); k.mul_(sign)

    register_mixer("toy_decay", DecayMixer)
    register_feed_forward("toy_gated", GatedFeedForward)
    register_position("toy_signflip", SignFlipPositions)


class DecaySpec:
    kind = "toy_decay"

    def __init__(self, hidden, weight, decay):
        self.hidden, self.weight, self.decay = hidden, weight, decay


class GatedSpec:
    kind = "toy_gated"

    def __init__(self, hidden, inner, prefix):
        self.hidden, self.inner, self.prefix = hidden, inner, prefix


def _toy_model(dtype):
    from transformers_neuronx_b200.engine import build_model
    from transformers_neuronx_b200.parts.spec import (AttentionSpec, EmbeddingSpec, HeadSpec, LayerSpec, LinearSpec,
                                                      ModelSpec, NormSpec, PositionSpec, ScheduleEntry)
    _register_toys()
    H, V, F, heads = 64, 97, 80, 2
    g = torch.Generator().manual_seed(5)
    rn = lambda *s: (torch.randn(*s, generator=g) / math.sqrt(s[-1])).bfloat16()
    t = {"emb": torch.randn(V, H, generator=g).bfloat16(), "mix.w": rn(H, H) * 0.5,
         "ff0.gate": rn(F, H), "ff0.up": rn(F, H), "ff0.down": rn(H, F),
         "ff1.gate": rn(F, H), "ff1.up": rn(F, H), "ff1.down": rn(H, F)}
    for n in "qkvo":
        t[f"att.{n}"] = rn(H, H)
    norm = lambda: NormSpec("layer_norm", H, 1e-5)
    att = AttentionSpec("attention", H, heads, heads, H // heads, 1 / math.sqrt(H // heads),
                        q=LinearSpec(H, H, "att.q"), k=LinearSpec(H, H, "att.k"), v=LinearSpec(H, H, "att.v"),
                        out=LinearSpec(H, H, "att.o"), window=24, position=PositionSpec("toy_signflip"))
    layers = (LayerSpec("pre_norm", norm(), DecaySpec(H, "mix.w", 0.9), norm(), GatedSpec(H, F, "ff0.")),
              LayerSpec("pre_norm", norm(), att, norm(), GatedSpec(H, F, "ff1.")))
    # the recurrent layer runs twice (with two states of its own); the attention layer runs twice
    # and its second run reads and extends the cache of its first
    schedule = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2), ScheduleEntry(1, 3))
    spec = ModelSpec(H, V, 256, EmbeddingSpec("emb", V, H, None, PositionSpec("none")), layers, schedule,
                     HeadSpec("head", V, H, tied_to="emb", final_norm=norm()))
    t["head"] = t["emb"]
    return build_model(spec, t, dtype, verbose=False), t, spec


def _toy_plain(ids, t, heads=2, window=24):
    """The toy model over a whole sequence in plain torch."""
    w = {k: v.float() for k, v in t.items()}
    x = w["emb"][torch.tensor(ids)]
    T, H = x.shape

    def decay_layer(x, ff):
        u = P.layer_norm(x, None, None) @ w["mix.w"].t()
        s, outs = torch.zeros(H), []
        for i in range(T):
            s = 0.9 * s + u[i]; outs.append(s)
        x = x + torch.stack(outs)
        h = P.layer_norm(x, None, None)
        return x + (torch.sigmoid(h @ w[ff + "gate"].t()) * (h @ w[ff + "up"].t())) @ w[ff + "down"].t()

    def att_layer(x, ff):
        h = P.layer_norm(x, None, None)
        d = H // heads
        sign = (1 - 2 * (torch.arange(T) % 2)).float()[:, None]
        q = ((h @ w["att.q"].t()) * sign).view(T, heads, d).transpose(0, 1)
        k = ((h @ w["att.k"].t()) * sign).view(T, heads, d).transpose(0, 1)
        v = (h @ w["att.v"].t()).view(T, heads, d).transpose(0, 1)
        p = P.masked_softmax(P.attention_scores(q, k, d), P.causal_mask(T, T, 0, window)[None])
        x = x + P.attention_context(p, v).transpose(0, 1).reshape(T, H) @ w["att.o"].t()
        h = P.layer_norm(x, None, None)
        return x + (torch.sigmoid(h @ w[ff + "gate"].t()) * (h @ w[ff + "up"].t())) @ w[ff + "down"].t()

    x = decay_layer(x, "ff0."); x = att_layer(x, "ff1."); x = decay_layer(x, "ff0."); x = att_layer(x, "ff1.")
    return P.layer_norm(x, None, None) @ w["emb"].t()


def test_toy_parts_are_registered_built_and_stepped():
    from transformers_neuronx_b200.cache import FixedStateNeed, PagedKVNeed
    from transformers_neuronx_b200.engine import StepEntry, StepRunner
    model, t, spec = _toy_model("float32")
    needs = model.cache_needs()
    assert isinstance(needs[0], FixedStateNeed) and isinstance(needs[1], PagedKVNeed) and needs[1].window == 24
    runner = StepRunner(model, 16, 12, 3, 256)
    assert [g.key for g in runner.cache.groups] == [("state",), ("paged", 24)]
    g = torch.Generator().manual_seed(6)
    seqs = {r: torch.randint(0, 97, (n,), generator=g).tolist() for r, n in (("a", 90), ("b", 41))}
    got = {r: [] for r in seqs}
    pos = {r: 0 for r in seqs}
    for r in seqs:
        runner.add_request(r)
    sizes = [5, 2, 17, 1, 1, 30, 3, 16, 1, 9]
    i = 0
    while any(pos[r] < len(seqs[r]) for r in seqs):               # portions and single tokens of both, mixed
        entries = []
        for r in seqs:
            if pos[r] < len(seqs[r]):
                n = min(sizes[i % len(sizes)], len(seqs[r]) - pos[r]); i += 1
                entries.append(StepEntry(r, seqs[r][pos[r]:pos[r] + n], list(range(n))))
                pos[r] += n
        logits = runner.step(entries)
        row = 0
        for e in entries:
            got[e.rid].append(logits[row:row + len(e.tokens)].cpu()); row += len(e.tokens)
    # the window gave pages back while the requests ran: 90 tokens would need 6 pages, a window of 24 at most 3
    assert len([p for p in runner.cache.block_table("a") if p >= 0]) <= 3
    for r in seqs:
        want = _toy_plain(seqs[r], t)
        assert rel_err(torch.cat(got[r]), want) <= 5e-5, r
    slots = {r: runner.cache.slot(r) for r in seqs}
    for r in seqs:
        runner.finish(r)
    runner.cache.check()
    assert runner.cache.free_pages() == [12] and runner.cache.slots.num_free == 3
    # A request that takes a slot another one has used finds clean state there: the mixer above
    # never looks at the context length, the cache manager zeroes the slot's row at admission.
    assert float(runner.storage.tensor(0)[slots["b"]].abs().max()) > 0, "the last owner left its state behind"
    ids = torch.randint(0, 97, (37,), generator=g).tolist()
    assert runner.add_request("c") in slots.values()
    lg = torch.cat([runner.step([StepEntry("c", ids[:20], list(range(20)))]).cpu(),
                    runner.step([StepEntry("c", ids[20:], list(range(17)))]).cpu()])
    assert rel_err(lg, _toy_plain(ids, t)) <= 5e-5
    runner.finish("c")


def test_toy_feed_forward_with_routing():
    """A feed-forward that routes each token to one of three experts (router logits in 32-bit, top-1),
    defined here, registered and stepped in portions beside the framework's attention."""
    from transformers_neuronx_b200.engine import StepEntry, StepRunner, build_model
    from transformers_neuronx_b200.parts import FeedForward, register_feed_forward, to_device
    from transformers_neuronx_b200.parts.spec import (AttentionSpec, EmbeddingSpec, HeadSpec, LayerSpec, LinearSpec,
                                                      ModelSpec, NormSpec, PositionSpec, ScheduleEntry)
    from transformers_neuronx_b200.weights import TensorSpec
    H, V, F, E, heads = 48, 61, 40, 3, 3

    class RoutedFeedForward(FeedForward):
        def __init__(self, spec):
            self.spec = spec

        def tensor_specs(self):
            return [TensorSpec("moe.router", (E, H)), TensorSpec("moe.up", (E * F, H)), TensorSpec("moe.down", (E * H, F))]

        def load(self, tensors, device, act_dtype):
            self.router = to_device(tensors["moe.router"], device, torch.float32)
            self.up = to_device(tensors["moe.up"], device, torch.float32).view(E, F, H)
            self.down = to_device(tensors["moe.down"], device, torch.float32).view(E, H, F)

        def forward(self, ctx, h, residual):
            x = h.float()
            expert = (x @ self.router.t()).argmax(dim=-1)                  # one expert per token
            for e in range(E):
                rows = (expert == e).nonzero().flatten()
                if rows.numel():
                    residual[rows] += torch.relu(x[rows] @ self.up[e].t()) @ self.down[e].t()

    class RoutedSpec:
        kind = "toy_routed"

    register_feed_forward("toy_routed", RoutedFeedForward)
    g = torch.Generator().manual_seed(11)
    rn = lambda *s: (torch.randn(*s, generator=g) / math.sqrt(s[-1])).bfloat16()
    t = {"emb": torch.randn(V, H, generator=g).bfloat16(), "moe.router": rn(E, H) * 4, "moe.up": rn(E * F, H),
         "moe.down": rn(E * H, F)}
    for n in "qkvo":
        t[f"att.{n}"] = rn(H, H)
    t["head"] = t["emb"]
    norm = lambda: NormSpec("layer_norm", H, 1e-5)
    att = AttentionSpec("attention", H, heads, heads, H // heads, 1 / math.sqrt(H // heads),
                        q=LinearSpec(H, H, "att.q"), k=LinearSpec(H, H, "att.k"), v=LinearSpec(H, H, "att.v"),
                        out=LinearSpec(H, H, "att.o"))
    spec = ModelSpec(H, V, 128, EmbeddingSpec("emb", V, H, None, PositionSpec("none")),
                     (LayerSpec("pre_norm", norm(), att, norm(), RoutedSpec()),), (ScheduleEntry(0, 0),),
                     HeadSpec("head", V, H, tied_to="emb", final_norm=norm()))
    model = build_model(spec, t, "float32", verbose=False)
    ids = torch.randint(0, V, (70,), generator=g).tolist()

    w = {k: v.float() for k, v in t.items()}
    x = w["emb"][torch.tensor(ids)]
    T, d = len(ids), H // heads
    hh = P.layer_norm(x, None, None)
    q, k, v = ((hh @ w[f"att.{n}"].t()).view(T, heads, d).transpose(0, 1) for n in "qkv")
    p = P.masked_softmax(P.attention_scores(q, k, d), P.causal_mask(T, T, 0, None)[None])
    x = x + P.attention_context(p, v).transpose(0, 1).reshape(T, H) @ w["att.o"].t()
    hh = P.layer_norm(x, None, None)
    expert = (hh @ w["moe.router"].t()).argmax(dim=-1)
    up, down = w["moe.up"].view(E, F, H), w["moe.down"].view(E, H, F)
    x = x + torch.stack([torch.relu(hh[i] @ up[e].t()) @ down[e].t() for i, e in enumerate(expert.tolist())])
    want = P.layer_norm(x, None, None) @ w["emb"].t()
    assert len(set(expert.tolist())) == E, "the test's weights should use every expert"

    runner = StepRunner(model, 16, 8, 1, 128)
    runner.add_request("r")
    got, pos = [], 0
    for n in (33, 2, 1, 1, 20, 13):
        got.append(runner.step([StepEntry("r", ids[pos:pos + n], list(range(n)))]).cpu()); pos += n
    assert rel_err(torch.cat(got), want) <= 5e-5


def test_schedule_may_share_a_cache():
    """Two schedule entries with one cache id: the second reads what the first wrote (and writes the
    same rows again); entries with different needs must not share."""
    from transformers_neuronx_b200.models.decoder import DecoderModel
    from transformers_neuronx_b200.parts.spec import ModelSpec, ScheduleEntry
    import dataclasses
    model, t, spec = _toy_model("float32")
    shared = dataclasses.replace(spec, schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(1, 1)))
    assert sorted(DecoderModel(shared).cache_needs()) == [0, 1]
    bad = dataclasses.replace(spec, schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 0)))
    with pytest.raises(ValueError, match="different needs"):
        DecoderModel(bad).cache_needs()
