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
TOL16 = {"bfloat16": 2e-2, "float16": 2.5e-3}
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


def test_reorder_carries_state_of_fixed_size_and_windowed_pages():
    """StepRunner.reorder on the toy model: a request goes on from another one's recurrent state (slots'
    rows, which may be read and written by the same reorder: a swap) and from its attention pages behind a
    window (some of them released already)."""
    from transformers_neuronx_b200.engine import StepEntry, StepRunner
    model, t, spec = _toy_model("float32")
    runner = StepRunner(model, 16, 24, 4, 256)
    g = torch.Generator().manual_seed(9)
    rids = ["a", "b", "c", "d"]
    hist = {r: torch.randint(0, 97, (45,), generator=g).tolist() for r in rids}
    for r in rids:
        runner.add_request(r)
    runner.step([StepEntry(r, hist[r], []) for r in rids])
    for sources in ([1, 0, 0, 3], [2, 2, 2, 2], [3, 0, 1, 2]):
        runner.reorder(rids, sources)
        runner.cache.check()
        hist = {r: list(hist[rids[s]]) for r, s in zip(rids, sources)}
        nxt = torch.randint(0, 97, (4,), generator=g).tolist()
        logits = runner.step([StepEntry(r, [nxt[i]], [0]) for i, r in enumerate(rids)]).cpu()
        for i, r in enumerate(rids):
            hist[r].append(nxt[i])
            assert rel_err(logits[i], _toy_plain(hist[r], t)[-1]) <= 5e-5, (sources, r)
    for r in rids:
        runner.finish(r)
    runner.cache.check()
    assert runner.cache.free_pages() == [24]


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


@pytest.mark.parametrize("dtype,d", [("bfloat16", 64), ("float16", 128), ("bfloat16", 48)])
def test_windowed_attention_in_16_bit_with_portions_after_a_release(dtype, d):
    """A sliding window in the 16-bit engine: head sizes 64 and 128 take the tcgen05 prefill kernel,
    48 the mma.sync one.  The request is fed in portions, so later portions start after the cache
    manager has given back the pages behind the window (their block-table entries are -1, and the
    pages are filled with another request's numbers meanwhile)."""
    from transformers_neuronx_b200.engine import StepEntry, StepRunner, build_model
    from transformers_neuronx_b200.parts.spec import (AttentionSpec, DenseFeedForwardSpec, EmbeddingSpec, HeadSpec, LayerSpec,
                                                      LinearSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry)
    heads, window, V = 2, 40, 211
    H, F = heads * d, 96
    g = torch.Generator().manual_seed(17)
    tdt = torch.bfloat16 if dtype == "bfloat16" else torch.float16
    rn = lambda *s: (torch.randn(*s, generator=g) / math.sqrt(s[-1])).to(tdt)
    t = {"emb": torch.randn(V, H, generator=g).to(tdt), "fc1.w": rn(F, H), "fc2.w": rn(H, F)}
    for n in "qkvo":
        t[f"att.{n}"] = rn(H, H)
    t["head"] = t["emb"]
    norm = lambda: NormSpec("layer_norm", H, 1e-5)
    att = AttentionSpec("attention", H, heads, heads, d, 1 / math.sqrt(d), q=LinearSpec(H, H, "att.q"), k=LinearSpec(H, H, "att.k"),
                        v=LinearSpec(H, H, "att.v"), out=LinearSpec(H, H, "att.o"), window=window)
    ff = DenseFeedForwardSpec("dense", LinearSpec(H, F, "fc1.w"), LinearSpec(F, H, "fc2.w"), "relu")
    spec = ModelSpec(H, V, 512, EmbeddingSpec("emb", V, H, None, PositionSpec("none")),
                     (LayerSpec("pre_norm", norm(), att, norm(), ff),), (ScheduleEntry(0, 0),),
                     HeadSpec("head", V, H, tied_to="emb", final_norm=norm()))
    model = build_model(spec, t, dtype, verbose=False)

    def plain(ids):
        w = {k: v.float() for k, v in t.items()}
        x = w["emb"][torch.tensor(ids)]
        T = len(ids)
        h = P.layer_norm(x, None, None)
        q, k, v = ((h @ w[f"att.{n}"].t()).view(T, heads, d).transpose(0, 1) for n in "qkv")
        p = P.masked_softmax(P.attention_scores(q, k, d), P.causal_mask(T, T, 0, window)[None])
        x = x + P.attention_context(p, v).transpose(0, 1).reshape(T, H) @ w["att.o"].t()
        x = x + torch.relu(P.layer_norm(x, None, None) @ w["fc1.w"].t()) @ w["fc2.w"].t()
        return P.layer_norm(x, None, None) @ w["emb"].t()

    runner = StepRunner(model, 16, 9, 2, 512, use_cuda_graphs=True)      # nine pages: far fewer than the 300 tokens need
    ids = torch.randint(0, V, (300,), generator=g).tolist()
    other = torch.randint(0, V, (60,), generator=g).tolist()
    want, want_other = plain(ids), plain(other)
    runner.add_request("w")
    got, pos = [], 0
    for step, n in enumerate([70, 50, 33, 2, 1, 1, 47, 1, 64, 17, 1, 1, 12]):
        entries = [StepEntry("w", ids[pos:pos + n], list(range(n)))]
        if step == 3:                                          # another request takes (and dirties) the pages given back
            runner.add_request("x")
            entries.append(StepEntry("x", other, [len(other) - 1]))
        lg = runner.step(entries).float().cpu()
        got.append(lg[:n]); pos += n
        if step == 3:
            assert rel_err(lg[n], want_other[-1]) <= TOL16[dtype]
            runner.finish("x")
        assert -1 in runner.cache.block_table("w") or pos < 2 * window
    assert pos == 300
    assert rel_err(torch.cat(got), want) <= TOL16[dtype]
    runner.finish("w")
    runner.cache.check()
    from transformers_neuronx_b200.kernels import ops
    ops.raise_on_device_error()


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("where", [15, 16, 127, 255, 256])
def test_a_planted_key_is_found_through_portions_and_captured_decode_steps(dtype, where):
    """With random weights attention is close to uniform over hundreds of keys, and a key dropped at
    the edge of a page, a tile, a split or a context bucket moves the logits far less than the
    16-bit tolerance.  Here the weights are made so that one query token (Q) puts nearly all its
    weight on one key token (M): M sits at `where` (the last row of a page, the first of the next, a
    tile's edge, the edge of the 256-token context bucket), the prompt goes in as two portions, and
    the decode steps that follow (eager, captured, replayed, across the bucket change) feed Q again
    and again.  Every logit is compared with the plain implementation, which would be far off if the
    key were lost: that is asserted too."""
    from transformers_neuronx_b200.engine import StepEntry, StepRunner, build_model
    from transformers_neuronx_b200.parts.spec import (AttentionSpec, DenseFeedForwardSpec, EmbeddingSpec, HeadSpec, LayerSpec,
                                                      LinearSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry)
    heads, d, V, F = 2, 64, 157, 96
    H = heads * d
    M, Q = 5, 6
    g = torch.Generator().manual_seed(23)
    tdt = torch.bfloat16 if dtype == "bfloat16" else torch.float16
    emb = torch.randn(V, H, generator=g) * 0.3
    emb[M, 0] += 5.0
    emb[Q, 1] += 5.0
    wq, wk = torch.randn(H, H, generator=g) / math.sqrt(H), torch.randn(H, H, generator=g) / math.sqrt(H)
    wq[0, 1] += 4.0                      # head 0, dim 0 of the query reads the Q direction ...
    wk[0, 0] += 4.0                      # ... and of the key the M direction
    rn = lambda *s_: (torch.randn(*s_, generator=g) / math.sqrt(s_[-1]))
    t = {"emb": emb, "att.q": wq, "att.k": wk, "att.v": rn(H, H), "att.o": rn(H, H), "fc1.w": rn(F, H), "fc2.w": rn(H, F)}
    t = {k: v.to(tdt) for k, v in t.items()}
    t["head"] = t["emb"]
    norm = lambda: NormSpec("layer_norm", H, 1e-5)
    att = AttentionSpec("attention", H, heads, heads, d, 1 / math.sqrt(d), q=LinearSpec(H, H, "att.q"), k=LinearSpec(H, H, "att.k"),
                        v=LinearSpec(H, H, "att.v"), out=LinearSpec(H, H, "att.o"))
    ff = DenseFeedForwardSpec("dense", LinearSpec(H, F, "fc1.w"), LinearSpec(F, H, "fc2.w"), "relu")
    spec = ModelSpec(H, V, 512, EmbeddingSpec("emb", V, H, None, PositionSpec("none")),
                     (LayerSpec("pre_norm", norm(), att, norm(), ff),), (ScheduleEntry(0, 0),),
                     HeadSpec("head", V, H, tied_to="emb", final_norm=norm()))
    model = build_model(spec, t, dtype, verbose=False)

    def plain(ids):
        w = {k: v.float() for k, v in t.items()}
        x = w["emb"][torch.tensor(ids)]
        T = len(ids)
        h = P.layer_norm(x, None, None)
        q, k, v = ((h @ w[f"att.{n}"].t()).view(T, heads, d).transpose(0, 1) for n in "qkv")
        p = P.masked_softmax(P.attention_scores(q, k, d), P.causal_mask(T, T, 0, None)[None])
        x = x + P.attention_context(p, v).transpose(0, 1).reshape(T, H) @ w["att.o"].t()
        x = x + torch.relu(P.layer_norm(x, None, None) @ w["fc1.w"].t()) @ w["fc2.w"].t()
        return P.layer_norm(x, None, None) @ w["emb"].t(), p

    ids = torch.randint(7, V, (275,), generator=g).tolist()
    ids[where] = M
    q_places = [249] + list(range(251, 275, 3))                  # the last prompt token and every third decode token
    for i in q_places:
        ids[i] = Q
    want, probs = plain(ids)
    assert all(float(probs[0, i, where]) > 0.9 for i in q_places if i > where), "the plant must dominate head 0"
    lost = list(ids); lost[where] = 9
    gone, _ = plain(lost)
    assert min(rel_err(gone[i], want[i]) for i in q_places if i > where) > 0.1, "losing the key must show"

    runner = StepRunner(model, 16, 20, 1, 512, use_cuda_graphs=True)
    runner.add_request("r")
    got = [runner.step([StepEntry("r", ids[:100], [99])]).float().cpu(),
           runner.step([StepEntry("r", ids[100:250], [149])]).float().cpu()]
    for i in range(250, 275):
        got.append(runner.step([StepEntry("r", [ids[i]], [0])]).float().cpu())
    got = torch.cat(got)
    places = [99, 249] + list(range(250, 275))
    assert len(runner.captured_steps()) >= 2, "decode steps below and beyond 256 tokens of context are graphs of their own"
    for row, i in enumerate(places):
        assert rel_err(got[row], want[i]) <= TOL16[dtype], (i, rel_err(got[row], want[i]))
        if i in q_places:
            assert int(got[row].argmax()) == int(want[i].argmax()), i
    from transformers_neuronx_b200.kernels import ops
    ops.raise_on_device_error()
