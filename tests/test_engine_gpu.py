"""The engine above the step function: greedy generation through the Python entry point, long
decoding, the first tokens of a sequence, the scheduler with real pages (preemption), temperature
sampling, the static-batch forward, and the command line."""
import os
import subprocess
import sys

import pytest
import torch

from helpers import TOLERANCE, TinyModel, check_greedy
from plain import opt_plain as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module", params=["A", "B"])
def tiny(request):
    return TinyModel(request.param, seed=21)


def _engine(tiny, dtype, **kw):
    from transformers_neuronx_b200.config import EngineConfig
    from transformers_neuronx_b200.engine import LLMEngine, load_model
    model, cfg = load_model(tiny.folder, dtype, verbose=False)
    return LLMEngine(model, EngineConfig(dtype=dtype, **kw), eos_token_id=cfg.eos_token_id)


def _plain_greedy_with_margin(tiny, prompt, n_new):
    """Greedy continuation by the plain implementation, with the gap between the two best logits at
    every step (a gap below the bf16 tolerance makes the token a legitimate tie)."""
    ids, toks, gaps = list(prompt), [], []
    for _ in range(n_new):
        lg = tiny.plain_logits(ids)[-1]
        top = torch.topk(lg, 2).values
        toks.append(int(lg.argmax())); gaps.append(float(top[0] - top[1]) / float(lg.abs().max()))
        ids.append(toks[-1])
    return toks, gaps


def _assert_greedy_equal(tiny, dtype, prompt, got, n_new, suppress=()):
    """All n_new tokens against the plain implementation (teacher-forced, so a tie does not end the
    comparison); returns how many of them were ties."""
    assert len(got) == n_new
    return check_greedy(tiny, dtype, prompt, got, suppress)


@pytest.mark.parametrize("amp", ["f32", "bf16"])
def test_greedy_through_the_entry_point(tiny, amp):
    from transformers_neuronx_b200.opt.model import OPTForSampling
    n_pos = 64
    model = OPTForSampling.from_pretrained(tiny.folder, batch_size=3, amp=amp, n_positions=n_pos)
    model.to_neuron()
    prompts = [tiny.random_ids(12, seed=s) for s in (1, 2, 3)]
    out = model.sample(torch.tensor(prompts), sequence_length=40, top_k=1)
    assert out.shape == (3, 40) and out[:, :12].tolist() == prompts
    dtype = "float32" if amp == "f32" else "bfloat16"
    eos = tiny.cfg.eos_token_id
    for row, prompt in zip(out.tolist(), prompts):
        assert eos not in row[12:]                          # sample() never draws the end-of-sequence token
        _assert_greedy_equal(tiny, dtype, prompt, row[12:], 28, suppress=(eos,))
    # left padding through start_ids: row 1 starts two places later
    padded = [prompts[0], [tiny.cfg.pad_token_id] * 2 + prompts[1][:10]]
    out2 = model.sample(torch.tensor(padded), sequence_length=20, start_ids=torch.tensor([0, 2]), top_k=1)
    _assert_greedy_equal(tiny, dtype, prompts[1][:10], out2[1, 12:].tolist(), 8, suppress=(eos,))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(tiny, dtype):
    """One token of prompt, then decoding to the model's full length: every page edge is crossed."""
    eng = _engine(tiny, dtype, max_num_seqs=2)
    n_new = tiny.cfg.max_position_embeddings - 1
    prompt = [tiny.cfg.bos_token_id]
    got = eng.generate([prompt], n_new, stop_on_eos=False)[0]
    ties = _assert_greedy_equal(tiny, dtype, prompt, got, n_new)
    print(f"long decoding {tiny.name} {dtype}: {n_new} tokens compared, {ties} ties")
    assert eng.runner.cache.free_pages() == [eng.runner.cache.pools[0].num_pages]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(tiny, dtype):
    """Logits at positions 0, 1, 2 (one key, two keys, ...) through forward(), fed one by one."""
    from transformers_neuronx_b200.opt.model import OPTForSampling
    amp = "f32" if dtype == "float32" else "bf16"
    model = OPTForSampling.from_pretrained(tiny.folder, batch_size=2, amp=amp, n_positions=32).to_neuron()
    ids = [tiny.random_ids(5, seed=8), tiny.random_ids(5, seed=9)]
    t = torch.tensor(ids)
    logits = [model.forward(t[:, :1])]
    for p in range(1, 5):
        logits.append(model(t[:, p:p + 1], torch.tensor([p]), None))
    for b in range(2):
        plain = tiny.plain_logits(ids[b])
        for p in range(5):
            err = float((logits[p][b] - plain[p]).abs().max()) / float(plain[p].abs().max())
            assert err <= TOLERANCE[dtype], f"position {p}: {err:.2e}"
    whole = model.forward(t)                                 # a new batch of whole prompts
    for b in range(2):
        plain = tiny.plain_logits(ids[b])[-1]
        assert float((whole[b] - plain).abs().max()) / float(plain.abs().max()) <= TOLERANCE[dtype]
    model.reset()
    assert model.engine.runner.cache.live_requests() == []


def test_scheduler_on_the_gpu_with_preemption(tiny):
    """So few pages that running requests are preempted and computed again: the tokens that come
    out are those of an engine with room for everything."""
    prompts = [tiny.random_ids(n, seed=40 + i) for i, n in enumerate([30, 9, 25, 14, 40, 5])]
    n_new = 40
    roomy = _engine(tiny, "float32", max_num_seqs=8, max_batch_tokens=64)
    want = roomy.generate(prompts, n_new, stop_on_eos=False)
    tight = _engine(tiny, "float32", max_num_seqs=4, max_batch_tokens=24, num_pages=12)
    got = tight.generate(prompts, n_new, stop_on_eos=False)
    assert tight.stats["preemptions"] > 0, "the pool was meant to be too small"
    assert got == want
    assert tight.runner.cache.free_pages() == [12] and tight.runner.cache.pools[0].reuse_count > 0
    tight.runner.cache.check()


def test_launching_ahead_changes_no_token(tiny):
    """The engine launches a step before the ids of the step before it are read back (the next
    input is taken from the device).  With that switched off the same tokens must come out, under
    preemption and with requests that end on the end-of-sequence token at different times."""
    from transformers_neuronx_b200.engine import SamplingParams
    prompts = [tiny.random_ids(n, seed=60 + i) for i, n in enumerate([22, 7, 31, 12, 18])]
    params = [SamplingParams(temperature=0.9, top_k=40, seed=3 + i) for i in range(len(prompts))]
    outs = {}
    for ahead in (True, False):
        eng = _engine(tiny, "float32", max_num_seqs=3, max_batch_tokens=24, num_pages=10, async_scheduling=ahead)
        first = eng.generate(prompts, 30, params, stop_on_eos=False)
        eng.eos_token_id = first[0][9]                      # some requests now end early, at different steps
        outs[ahead] = (first, eng.generate(prompts, 30, params, stop_on_eos=True), eng.stats["preemptions"])
        assert eng.runner.cache.free_pages() == [10] and eng.runner.cache.slots.num_free == 3
    assert outs[True][0] == outs[False][0] and outs[True][1] == outs[False][1]
    assert outs[True][2] > 0
    eos = outs[True][0][0][9]
    for full, cut in zip(*outs[True][:2]):
        want = full[:full.index(eos) + 1] if eos in full else full
        assert cut == want and -1 not in cut


@pytest.mark.parametrize("seed", range(4))
def test_a_tight_engine_generates_what_a_roomy_one_does(seed):
    """Random requests through two engines in 32-bit: one with room for everything, whole prompts and no
    graphs; one with few pages and slots, a small token budget, CUDA graphs and steps launched ahead, so that
    prompts are cut, requests wait and some are preempted and computed again.  The tokens are the same
    (greedy, and sampled with temperature, top-k and top-p: a draw depends on seed and counter alone)."""
    import random
    from transformers_neuronx_b200.config import EngineConfig
    from transformers_neuronx_b200.engine import LLMEngine, SamplingParams, load_model
    rng = random.Random(500 + seed)
    tiny = TinyModel("ABDF"[seed], seed=rng.randrange(50))
    maxlen = tiny.cfg.max_position_embeddings
    n = rng.randint(3, 8)
    prompts = [tiny.random_ids(rng.randint(1, maxlen // 2), seed=rng.randrange(10 ** 6)) for _ in range(n)]
    news = [rng.randint(1, min(40, maxlen - len(p))) for p in prompts]
    sample = seed % 2 == 1
    params = [SamplingParams(temperature=0.8, top_k=rng.choice([0, 20]), top_p=rng.choice([1.0, 0.9]), seed=i) if sample else None
              for i in range(n)]
    model, cfg = load_model(tiny.folder, "float32", verbose=False)
    roomy = LLMEngine(model, EngineConfig(dtype="float32", max_num_seqs=16, max_batch_tokens=4096, async_scheduling=False,
                                          use_cuda_graphs=False), eos_token_id=cfg.eos_token_id)
    want = roomy.generate(prompts, news, params, stop_on_eos=True)
    most = max(-(-(len(p) + m) // 16) for p, m in zip(prompts, news))
    pages = most + rng.randint(0, most)
    tight = LLMEngine(model, EngineConfig(dtype="float32", max_num_seqs=rng.randint(1, 4), max_batch_tokens=rng.choice([8, 24, 100]),
                                          num_pages=pages, async_scheduling=True, use_cuda_graphs=True),
                      eos_token_id=cfg.eos_token_id)
    got = tight.generate(prompts, news, params, stop_on_eos=True)
    assert got == want
    assert tight.runner.cache.free_pages() == [pages]
    tight.runner.cache.check()


def test_temperature_sampling_is_seeded(tiny):
    from transformers_neuronx_b200.engine import SamplingParams
    eng = _engine(tiny, "bfloat16", max_num_seqs=4)
    prompts = [tiny.random_ids(10, seed=s) for s in (1, 2)]
    ps = [SamplingParams(temperature=0.8, top_k=50, seed=7), SamplingParams(temperature=0.8, top_p=0.9, seed=8)]
    a = eng.generate(prompts, 32, ps, stop_on_eos=False)
    b = eng.generate(prompts, 32, ps, stop_on_eos=False)
    c = eng.generate(prompts, 32, [SamplingParams(temperature=0.8, top_k=50, seed=9)] * 2, stop_on_eos=False)
    assert a == b and a != c
    greedy = eng.generate(prompts, 32, None, stop_on_eos=False)
    assert greedy != a


def test_eos_stops_a_request(tiny):
    eng = _engine(tiny, "float32", max_num_seqs=2)
    prompt = tiny.random_ids(8, seed=3)
    first = eng.generate([prompt], 5, stop_on_eos=False)[0]
    eng.eos_token_id = first[2]                               # pretend the third new token ends the sequence
    out = eng.generate([prompt], 5, stop_on_eos=True)[0]
    assert out == first[:first.index(first[2]) + 1]


def test_on_device_generation_config_through_the_entry_point(tiny):
    """neuron_config=NeuronConfig(on_device_generation=...): greedy by default; with do_sample the
    reference's fixed draw (deterministic) is followed token by token against the plain choice; with
    eos_token_id finished rows are filled with it and the result ends where the last row finished."""
    from transformers_neuronx_b200 import GenerationConfig, NeuronConfig
    from transformers_neuronx_b200.opt.model import OPTForSampling
    prompts = [tiny.random_ids(9, seed=s) for s in (4, 5)]
    ids = torch.tensor(prompts)

    def model(gen):
        m = OPTForSampling.from_pretrained(tiny.folder, batch_size=2, amp="f32", n_positions=48,
                                           neuron_config=NeuronConfig(on_device_generation=gen))
        return m.to_neuron()

    greedy = model(GenerationConfig()).sample(ids, sequence_length=30)
    assert greedy.shape == (2, 30)
    for b in range(2):
        _assert_greedy_equal(tiny, "float32", prompts[b], greedy[b, 9:].tolist(), 21)

    gen = GenerationConfig(do_sample=True, top_k=[12, 40], top_p=[0.9, 0.7], temperature=[1.5, 3.0], top_p_min_tokens=[1, 5],
                           per_batch_line=True, deterministic=True)
    out = model(gen).sample(ids, sequence_length=30)
    for b in range(2):
        k, p, t, n_min = gen.for_row(b)
        seq = list(prompts[b])
        for i in range(21):
            want, margin = P.sample_on_device(tiny.plain_logits(seq)[-1], k, p, n_min, t)
            got = int(out[b, 9 + i])
            if got != want:
                assert margin <= 1e-3, f"row {b} token {i}: {got}, plain {want}, margin {margin:.2e}"
                break                                # one half lay on a summed probability: the sequences part
            seq.append(got)

    # the id that row 0 produces greedily as its 6th new token ends that row; row 1 runs on
    eos = int(greedy[0, 9 + 5])
    first = [t == eos for t in greedy[0, 9:].tolist()].index(True)
    stop = model(GenerationConfig(eos_token_id=eos)).sample(ids, sequence_length=30)
    hits1 = [i for i, t in enumerate(greedy[1, 9:].tolist()) if t == eos]
    end = max(first, hits1[0] if hits1 else 20) + 1
    assert stop.shape == (2, 9 + end), (stop.shape, first, hits1)
    assert stop[0, 9:9 + first + 1].tolist() == greedy[0, 9:9 + first + 1].tolist()
    assert all(t == eos for t in stop[0, 9 + first:].tolist())
    n1 = (hits1[0] + 1) if hits1 else end
    assert stop[1, 9:9 + n1].tolist() == greedy[1, 9:9 + n1].tolist()


def test_streamer_gets_tokens_while_they_are_generated(tiny):
    from transformers_neuronx_b200 import GenerationConfig, NeuronConfig
    from transformers_neuronx_b200.opt.model import OPTForSampling
    model = OPTForSampling.from_pretrained(tiny.folder, batch_size=2, amp="f32", n_positions=40).to_neuron()

    class Recorder:
        def __init__(self):
            self.cols, self.at_step, self.ended = [], [], False

        def put(self, t):
            assert not self.ended and tuple(t.shape) == (2, 1)
            self.cols.append(t.clone()); self.at_step.append(model.engine.stats["steps"])

        def end(self):
            self.ended = True

    ids = torch.tensor([tiny.random_ids(7, seed=s) for s in (8, 9)])
    rec = Recorder()
    out = model.sample(ids, sequence_length=25, top_k=1, streamer=rec)
    assert rec.ended and torch.equal(torch.cat(rec.cols, dim=1), out[:, 7:])
    assert rec.at_step[-1] - rec.at_step[0] >= 15, "the tokens came while the engine was stepping, not at the end"
    assert torch.equal(out, model.sample(ids, sequence_length=25, top_k=1))
    # with early stop: the streamed columns are the returned ones, finished rows filled with the id
    eos = int(out[0, 7 + 4])
    stopping = OPTForSampling.from_pretrained(tiny.folder, batch_size=2, amp="f32", n_positions=40, neuron_config=NeuronConfig(
        on_device_generation=GenerationConfig(eos_token_id=eos))).to_neuron()
    rec2 = Recorder()
    model = stopping
    out2 = stopping.sample(ids, sequence_length=25, streamer=rec2)
    assert rec2.ended and torch.equal(torch.cat(rec2.cols, dim=1), out2[:, 7:])
    assert torch.equal(out2, stopping.sample(ids, sequence_length=25))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_tapped_hidden_states_match_the_plain_layers(tiny, dtype):
    """model.tap_hidden_states(): the residual stream after the embedding and after every layer, for
    a prompt run in two portions, against the plain implementation layer by layer (a fault shows at
    the first layer that has it); captured graphs are not used while tapping and are used after."""
    from transformers_neuronx_b200.engine import StepEntry, StepRunner, load_model
    model, _ = load_model(tiny.folder, dtype, verbose=False)
    runner = StepRunner(model, 16, 8, 2, 128, use_cuda_graphs=True)
    ids = tiny.random_ids(45, seed=31)
    cfg = tiny.cfg.to_dict()
    w = {k: v.float() for k, v in tiny.plain_tensors.items()}
    want = [P.embed(torch.tensor(ids), w)]
    for i in range(cfg["num_hidden_layers"]):
        want.append(P.decoder_layer(want[-1], w, i, cfg))
    runner.add_request("t")
    with model.tap_hidden_states() as taps:
        runner.step([StepEntry("t", ids[:29], [])])
        first = {k: v.cpu() for k, v in taps.items()}
        lg = runner.step([StepEntry("t", ids[29:], [15])])
        second = {k: v.cpu() for k, v in taps.items()}
    assert not runner.captured_steps() and "logits" not in first and torch.equal(second["logits"], lg.cpu())
    tol = TOLERANCE[dtype]
    for name, i in [("embedding", 0)] + [(f"entry{j}", j + 1) for j in range(cfg["num_hidden_layers"])]:
        got = torch.cat([first[name], second[name]])
        err = float((got - want[i]).abs().max()) / float(want[i].abs().max())
        assert err <= tol, f"{dtype} {name}: {err:.2e}"
    for t in range(3):                                        # afterwards single tokens are captured again
        runner.step([StepEntry("t", [ids[t]], [0])])
    assert runner.captured_steps()


def test_generate_adapter_with_left_padded_rows(tiny):
    from transformers_neuronx_b200.generation_utils import HuggingFaceGenerationModelAdapter
    from transformers_neuronx_b200.opt.model import OPTForSampling
    model = OPTForSampling.from_pretrained(tiny.folder, batch_size=3, amp="f32", n_positions=48).to_neuron()
    adapter = HuggingFaceGenerationModelAdapter(model.config, model)
    prompts = [tiny.random_ids(n, seed=40 + n) for n in (5, 9, 12)]
    pad = tiny.cfg.pad_token_id
    ids = torch.tensor([[pad] * (12 - len(p)) + p for p in prompts])
    mask = torch.tensor([[0] * (12 - len(p)) + [1] * len(p) for p in prompts])
    assert adapter.start_ids_of(mask).tolist() == [7, 3, 0]
    out = adapter.generate(ids, attention_mask=mask, max_new_tokens=10)
    assert out.shape == (3, 22) and torch.equal(out[:, :12], ids)
    for b in range(3):
        _assert_greedy_equal(tiny, "float32", prompts[b], out[b, 12:].tolist(), 10)
    assert torch.equal(adapter.generate(ids, attention_mask=mask, max_length=22), out)
    # forward, as a generation loop of the caller's would use it
    adapter.reset_generation()
    lg = adapter(ids, None, attention_mask=mask)[0]
    assert lg.shape == (3, 1, tiny.cfg.vocab_size) and adapter.cur_len == 12
    for b in range(3):
        want = tiny.plain_logits(prompts[b])[-1]
        assert float((lg[b, 0] - want).abs().max()) / float(want.abs().max()) <= TOLERANCE["float32"]
    # eos ends a row; the pad id follows it
    eos = int(out[0, 12 + 3])
    first = out[0, 12:].tolist().index(eos)
    stopped = adapter.generate(ids, attention_mask=mask, max_new_tokens=10, eos_token_id=eos, pad_token_id=pad)
    assert stopped[0, 12:12 + first + 1].tolist() == out[0, 12:12 + first + 1].tolist()
    assert all(t == pad for t in stopped[0, 12 + first + 1:].tolist())
    sampled = adapter.generate(ids, attention_mask=mask, max_new_tokens=6, do_sample=True, top_k=5, temperature=0.8, seed=3)
    assert torch.equal(sampled, adapter.generate(ids, attention_mask=mask, max_new_tokens=6, do_sample=True, top_k=5,
                                                 temperature=0.8, seed=3))
    with pytest.raises(NotImplementedError):
        adapter.generate(ids, num_beams=4, do_sample=True)
    with pytest.raises(TypeError):
        adapter.generate(ids, logits_processor=[])


def test_reorder_cache_lets_a_row_go_on_from_another(tiny):
    """The cache side of beam search: after reorder_cache(ids) row i holds what row ids[i] held; a row that
    two rows go on from is copied, the others' pages only change hands.  The next token's logits are those
    of the source's prompt, whatever is done twice in a row."""
    from transformers_neuronx_b200.opt.model import OPTForSampling
    model = OPTForSampling.from_pretrained(tiny.folder, batch_size=5, amp="f32", n_positions=64).to_neuron()
    prompts = [tiny.random_ids(21, seed=70 + i) for i in range(5)]
    model(torch.tensor(prompts), None, None)
    cache = model.engine.runner.cache
    held = [list(cache.block_table(f"row{i}")) for i in range(5)]
    history = [list(p) for p in prompts]
    for step, ids in enumerate(([2, 2, 0, 4, 2], [1, 0, 3, 3, 3], [0, 1, 2, 3, 4])):
        model.reorder_cache(ids)
        cache.check()
        history = [list(history[i]) for i in ids]
        nxt = [7 + step, 8, 9, 10, 11 + step]
        lg = model(torch.tensor(nxt)[:, None], torch.tensor([21 + step]), None)
        for i in range(5):
            history[i].append(nxt[i])
            want = tiny.plain_logits(history[i])[-1]
            assert float((lg[i] - want).abs().max()) / float(want.abs().max()) <= TOLERANCE["float32"], (step, i)
    assert sorted(p for t in held for p in t) == sorted(p for i in range(5) for p in cache.block_table(f"row{i}")[:len(held[0])])
    with pytest.raises(ValueError):
        model.reorder_cache([0, 1])


def _plain_beam_search(tiny, prompt, nb, n_new, eos, length_penalty=1.0, early_stopping=False):
    """Beam search restated over whole sequences: every step the plain implementation reads each running
    sequence from its first token (no cache, nothing reordered)."""
    running = [(0.0, [])]
    ended = []
    for step in range(n_new):
        cands = []
        for score, toks in running:
            logp = torch.log_softmax(tiny.plain_logits(list(prompt) + toks)[-1].float(), -1)
            top = torch.topk(logp, min(2 * nb, logp.numel()))
            cands += [(score + float(v), toks, int(t)) for v, t in zip(top.values, top.indices)]
        cands.sort(key=lambda c: -c[0])
        cands = cands[:2 * nb]
        nxt = []
        for rank, (v, toks, t) in enumerate(cands):
            if t in eos:
                if rank < nb:
                    ended.append((v / (len(toks) + 1) ** length_penalty, toks + [t]))
                continue
            nxt.append((v, toks + [t]))
            if len(nxt) == nb:
                break
        running = nxt
        if len(ended) >= nb:
            ended = sorted(ended, key=lambda h: -h[0])[:nb]
            best = max((r[0] for r in running), default=float("-inf")) / (step + 1) ** length_penalty
            if early_stopping or not running or best <= ended[-1][0]:
                return max(ended, key=lambda h: h[0])[1]
        if not running:
            break
    cands = ended + [(v / len(t) ** length_penalty, t) for v, t in running if t]
    return max(cands, key=lambda h: h[0])[1]


@pytest.mark.parametrize("nb,lp,early", [(3, 1.0, False), (4, 0.6, True), (2, 1.5, False)])
def test_beam_search_through_the_adapter(tiny, nb, lp, early):
    """generate(num_beams=...) against a beam search over the plain implementation's logits: left-padded
    prompts of different lengths, an eos id that ends some beams early, length penalty and early stopping."""
    from transformers_neuronx_b200.generation_utils import HuggingFaceGenerationModelAdapter
    from transformers_neuronx_b200.opt.model import OPTForSampling
    model = OPTForSampling.from_pretrained(tiny.folder, batch_size=2 * nb, amp="f32", n_positions=40).to_neuron()
    adapter = HuggingFaceGenerationModelAdapter(model.config, model)
    prompts = [tiny.random_ids(n, seed=90 + n) for n in (6, 11)]
    pad = tiny.cfg.pad_token_id
    ids = torch.tensor([[pad] * (11 - len(p)) + p for p in prompts])
    mask = torch.tensor([[0] * (11 - len(p)) + [1] * len(p) for p in prompts])
    n_new = 9
    free = _plain_beam_search(tiny, prompts[0], nb, n_new, set(), lp, early)
    eos = free[4]                                            # a token that the best beam of prompt 0 reaches
    out = adapter.generate(ids, attention_mask=mask, num_beams=nb, max_new_tokens=n_new, eos_token_id=eos,
                           pad_token_id=pad, length_penalty=lp, early_stopping=early)
    assert torch.equal(out[:, :11], ids)
    longest = 0
    for b in range(2):
        want = _plain_beam_search(tiny, prompts[b], nb, n_new, {eos}, lp, early)
        got = out[b, 11:].tolist()
        assert got[:len(want)] == want, (b, got, want)
        assert all(t == pad for t in got[len(want):])
        longest = max(longest, len(want))
    assert out.shape[1] == 11 + longest
    model.engine.runner.cache.check()
    assert model.engine.runner.cache.live_requests() == []
    # without an eos id every beam runs to the limit and the most likely one is returned
    out2 = adapter.generate(ids, attention_mask=mask, num_beams=nb, max_new_tokens=n_new, length_penalty=lp)
    assert out2[0, 11:].tolist() == _plain_beam_search(tiny, prompts[0], nb, n_new, set(), lp, False)
    with pytest.raises(ValueError, match="batch_size"):
        adapter.generate(ids, num_beams=nb + 1, max_new_tokens=2)


def test_forward_with_sequence_ids_as_a_serving_loop_drives_it(tiny):
    """NeuronConfig(continuous_batching=...): forward(input_ids, cache_ids, seq_ids) as the reference takes it from
    a serving loop outside the model (base.py:492-587): prompts for some cache lines (right-padded rows, 2-D
    positions), single tokens for any lines in any order, a line begun anew, a further portion of a prompt."""
    from transformers_neuronx_b200 import ContinuousBatchingConfig, NeuronConfig
    from transformers_neuronx_b200.opt.model import OPTForSampling
    nc = NeuronConfig(continuous_batching=ContinuousBatchingConfig(batch_size_for_shared_caches=3))
    model = OPTForSampling.from_pretrained(tiny.folder, batch_size=1, amp="f32", n_positions=64, neuron_config=nc).to_neuron()
    tol = TOLERANCE["float32"]

    def close(got, ids):
        want = tiny.plain_logits(ids)[-1]
        assert float((got - want).abs().max()) / float(want.abs().max()) <= tol

    seqs = {2: tiny.random_ids(9, seed=1)}
    lg = model(torch.tensor([seqs[2]]), torch.arange(9)[None], torch.tensor([2]))
    close(lg[0], seqs[2])
    seqs[0], seqs[1] = tiny.random_ids(12, seed=2), tiny.random_ids(5, seed=3)
    ids = torch.tensor([seqs[0], seqs[1] + [0] * 7])
    pos = torch.tensor([list(range(12)), list(range(5)) + [0] * 7])
    lg = model(ids, pos, torch.tensor([0, 1]))
    close(lg[0], seqs[0]); close(lg[1], seqs[1])
    for step in range(3):                                    # single tokens, the lines in another order every time
        order = [[1, 2, 0], [2, 0, 1], [0, 1, 2]][step]
        toks = [7 + step + s for s in order]
        lg = model(torch.tensor(toks)[:, None], torch.tensor([[len(seqs[s])] for s in order]), torch.tensor(order))
        for i, s in enumerate(order):
            seqs[s] = seqs[s] + [toks[i]]
            close(lg[i], seqs[s])
    seqs[1] = tiny.random_ids(6, seed=4)                     # line 1 begins anew; what it held is given back
    lg = model(torch.tensor([seqs[1]]), torch.arange(6)[None], torch.tensor([1]))
    close(lg[0], seqs[1])
    more = tiny.random_ids(4, seed=5)                        # a further portion of line 2, beside nothing else
    lg = model(torch.tensor([more]), torch.arange(len(seqs[2]), len(seqs[2]) + 4)[None], torch.tensor([2]))
    seqs[2] = seqs[2] + more
    close(lg[0], seqs[2])
    lg = model(torch.tensor([[9], [10]]), torch.tensor([[len(seqs[1])], [len(seqs[2])]]), torch.tensor([1, 2]))
    close(lg[0], seqs[1] + [9]); close(lg[1], seqs[2] + [10])
    with pytest.raises(ValueError, match="holds"):
        model(torch.tensor([[3]]), torch.tensor([[40]]), torch.tensor([0]))
    with pytest.raises(ValueError, match="sequence id"):
        model(torch.tensor([[3]]), torch.tensor([[0]]), torch.tensor([3]))
    model.engine.runner.cache.check()
    model.reset()
    assert model.engine.runner.cache.live_requests() == []
    # cast_logits_dtype (base.py:641-647): the type the logits are handed out in
    nc16 = NeuronConfig(cast_logits_dtype="bfloat16")
    m16 = OPTForSampling.from_pretrained(tiny.folder, batch_size=1, amp="f32", n_positions=32, neuron_config=nc16).to_neuron()
    lg = m16(torch.tensor([seqs[0][:8]]))
    assert lg.dtype == torch.bfloat16
    want = tiny.plain_logits(seqs[0][:8])[-1]
    assert float((lg[0].float() - want).abs().max()) / float(want.abs().max()) <= 1e-2


def test_validate_against_a_reference_model(tiny):
    """testing.validate (the reference's testing/validation.py:23-101) with the plain implementation standing in
    for the CPU model, on the left-padded batches of testing.data."""
    from transformers_neuronx_b200.opt.model import OPTForSampling
    from transformers_neuronx_b200.testing import batch_all_lengths, batch_full_lengths, batch_varying_lengths, validate

    class PlainModel:
        def generate(self, input_ids, attention_mask, max_new_tokens, **_):
            rows = []
            for ids, mask in zip(input_ids.tolist(), attention_mask.tolist()):
                start = mask.index(1)
                toks, _ = _plain_greedy_with_margin(tiny, ids[start:], max_new_tokens)
                rows.append(ids + toks)
            return torch.tensor(rows)

    V = tiny.cfg.vocab_size
    ids, mask, starts = batch_all_lengths(V, 6, seed=1)
    assert mask.tolist()[2] == [0, 0, 1, 1, 1, 1] and starts.tolist() == list(range(6)) and int(ids[3, 2]) == 0
    for inputs in (batch_varying_lengths(V, 4, 9, seed=2), batch_full_lengths(V, 3, 5, seed=3), (ids, mask, starts)):
        rows = inputs[0].shape[0]
        model = OPTForSampling.from_pretrained(tiny.folder, batch_size=rows, amp="f32", n_positions=32)
        validate(PlainModel(), model, tiny.cfg, inputs, sequence_length=inputs[0].shape[1] + 6, verbose=False)
    wrong = PlainModel()
    wrong.generate = lambda **kw: PlainModel().generate(**kw) + 1
    with pytest.raises(AssertionError, match="differs"):
        validate(wrong, model, tiny.cfg, inputs, sequence_length=inputs[0].shape[1] + 6, verbose=False)


@pytest.mark.parametrize("amp", ["f32", "bf16"])
def test_sliding_window_through_neuron_config(tiny, amp):
    """NeuronConfig(sparse_attn=SparseAttnConfig('window', causal=True, SlidingWindowAttnConfig(W))): every layer
    attends to the token itself and the W before it (sparse_attn_utils.py:140-150), in prompts, in portions and when
    decoding; pages behind the window go back to the pool while the sequence runs."""
    from transformers_neuronx_b200 import NeuronConfig, SlidingWindowAttnConfig, SparseAttnConfig
    from transformers_neuronx_b200.opt.model import OPTForSampling
    W = 19
    nc = NeuronConfig(sparse_attn=SparseAttnConfig("window", causal=True, sparse_attn_config=SlidingWindowAttnConfig(W)))
    n_pos = min(100, tiny.cfg.max_position_embeddings)
    model = OPTForSampling.from_pretrained(tiny.folder, batch_size=2, amp=amp, n_positions=n_pos, neuron_config=nc).to_neuron()
    cfg = dict(tiny.cfg.to_dict(), sliding_window_size=W)
    dtype = {"f32": "float32", "bf16": "bfloat16"}[amp]
    prompts = [tiny.random_ids(60, seed=5), tiny.random_ids(60, seed=6)]
    lg = model(torch.tensor(prompts))
    seqs = [list(p) for p in prompts]
    for step in range(12):
        for b in range(2):
            want = P.forward_logits(seqs[b], tiny.plain_tensors, cfg)[-1]
            assert float((lg[b] - want).abs().max()) / float(want.abs().max()) <= TOLERANCE[dtype], (step, b)
            full = tiny.plain_logits(seqs[b])[-1]
            if step == 0:
                assert float((want - full).abs().max()) / float(full.abs().max()) > 1e-3, \
                    "the window must matter for this check to mean anything"
        nxt = [int(lg[b].argmax()) for b in range(2)]
        for b in range(2):
            seqs[b].append(nxt[b])
        lg = model(torch.tensor(nxt)[:, None], torch.tensor([60 + step]))
    held = [p for p in model.engine.runner.cache.block_table("row0") if p >= 0]
    assert len(held) <= -(-(W + 1) // 16) + 1 < -(-72 // 16), "pages behind the window were given back"
    with pytest.raises(NotImplementedError):
        SparseAttnConfig("blk_sparse")
    with pytest.raises(NotImplementedError):
        SparseAttnConfig("window", causal=False, sparse_attn_config=SlidingWindowAttnConfig(8))


def test_all_logits_of_a_prompt_and_kept_kernels(tiny, tmp_path):
    from transformers_neuronx_b200 import NeuronConfig
    from transformers_neuronx_b200.opt.model import OPTForSampling
    model = OPTForSampling.from_pretrained(tiny.folder, batch_size=2, amp="f32", n_positions=32,
                                           neuron_config=NeuronConfig(output_all_logits=True))
    model.to_neuron()
    prompts = [tiny.random_ids(n, seed=60 + n) for n in (6, 11)]
    pad = tiny.cfg.pad_token_id
    ids = torch.tensor([[pad] * (11 - len(p)) + p for p in prompts])
    lg = model(ids, None, torch.tensor([5, 0]))
    assert lg.shape == (2, 11, tiny.cfg.vocab_size) and float(lg[0, :5].abs().max()) == 0.0
    for b, p in enumerate(prompts):
        want = tiny.plain_logits(p)
        got = lg[b, 11 - len(p):]
        assert float((got - want).abs().max()) / float(want.abs().max()) <= TOLERANCE["float32"]
    nxt = model(torch.tensor([[7], [9]]), torch.tensor([11]), torch.tensor([5, 0]))       # a decode call: last token only
    assert nxt.shape == (2, tiny.cfg.vocab_size)
    model.save(str(tmp_path / "kernels"))
    kept = os.listdir(tmp_path / "kernels")
    assert kept and all(f.endswith(".so") for f in kept)
    other = OPTForSampling.from_pretrained(tiny.folder, batch_size=1, amp="f32", n_positions=32)
    other.load(str(tmp_path / "kernels"))
    assert other.to_neuron().sample(ids[1:], sequence_length=14, top_k=1).shape == (1, 14)


def test_kernel_profile(tiny):
    """The profiling helper brackets every kernel call with events and names the families."""
    from transformers_neuronx_b200.kernels import kernel_profile
    eng = _engine(tiny, "bfloat16", max_num_seqs=2, use_cuda_graphs=False)
    with kernel_profile() as prof:
        eng.generate([tiny.random_ids(20, seed=1)], 4, stop_on_eos=False)
    t = prof.totals()
    assert {"embed", "layer_norm", "kv_append", "sample_packed"} <= set(t)
    assert ("gemm_tc" in t) or ("gemm_simt" in t)
    assert all(ms >= 0 and n > 0 for ms, n in t.values()) and "share" in prof.report()
    from transformers_neuronx_b200.kernels import ops
    assert ops.embed.__name__ == "embed"                      # the wrappers are gone


def test_profile_of_the_entry_point(tiny, tmp_path):
    """model.profile(dir), under the reference's name: a report per kernel family, written to the folder."""
    from transformers_neuronx_b200.opt.model import OPTForSampling
    model = OPTForSampling.from_pretrained(tiny.folder, batch_size=2, amp="bf16", n_positions=48).to_neuron()
    assert model.is_compiled()
    report = model.profile(str(tmp_path / "prof"))
    assert open(tmp_path / "prof" / "kernel_profile.txt").read() == report
    for word in ("layer_norm", "embed", "share", "decode steps"):
        assert word in report
    assert model.engine.runner.cache.live_requests() == []
    out = model.sample(torch.tensor([tiny.random_ids(5, seed=3)] * 2), sequence_length=12, top_k=1)      # still usable
    assert out.shape == (2, 12)


def test_command_line_save_and_run(tmp_path):
    cfg = tmp_path / "cfg.json"
    import json
    from helpers import CONFIG_A
    cfg.write_text(json.dumps(CONFIG_A))
    folder = tmp_path / "model"
    demo = os.path.join(ROOT, "bin", "opt_demo")
    r = subprocess.run([sys.executable, demo, "--amp", "bf16", "save", str(folder), "--random", "--config", str(cfg)],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-1500:]
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    r = subprocess.run([sys.executable, demo, "--amp", "bf16", "run", str(folder), "--batch_size", "2", "--n_positions", "24",
                        "--print_latency"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-1500:]
    assert "generated_sequence=" in r.stdout and "Latency:" in r.stdout
    # the reference's sliding-window options (gpt_demo.py:57-65, :107-123): tokens differ from the full attention's
    # once the window is shorter than the sequence
    full = r.stdout[r.stdout.index("generated_sequence="):]
    r = subprocess.run([sys.executable, demo, "--amp", "bf16", "run", str(folder), "--batch_size", "2", "--n_positions", "24",
                        "--sparse_attn", "window", "--window_size", "3"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-1500:]
    assert "generated_sequence=" in r.stdout and r.stdout[r.stdout.index("generated_sequence="):] != full
    r = subprocess.run([sys.executable, demo, "run", str(folder), "--sparse_attn", "blk_sparse"], capture_output=True, text=True,
                       timeout=600)
    assert r.returncode != 0 and "not implemented" in r.stderr.lower()
