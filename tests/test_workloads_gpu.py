"""The two tiny workloads of the build's baseline, through the engine (scheduler, step function,
sampler) against the plain implementation, in 32-bit, bfloat16 and float16:

A: four prompts of 5, 17, 33 and 64 tokens (BOS first, the rest uniform in [3, vocab)), 32 new tokens
   greedy and 32 at temperature 0.8 with seed 0;
B: three prompts of 1, 40 and 120 tokens, prompts cut into 16-token portions that run beside the
   other requests' decode tokens, 48 new tokens each;
and the scheduler under pressure (preemption, late end-of-sequence) in the 16-bit types as well."""
import pytest
import torch

from helpers import TinyModel, check_greedy, check_sampled, storage_for

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16", "float16"]
_models = {}


def _model(name, dtype, seed=51):
    key = (name, storage_for(dtype))
    if key not in _models:
        _models[key] = TinyModel(name, seed=seed, matrix_dtype=storage_for(dtype))
    return _models[key]


def _engine(tiny, dtype, **kw):
    from transformers_neuronx_b200.config import EngineConfig
    from transformers_neuronx_b200.engine import LLMEngine, load_model
    model, cfg = load_model(tiny.folder, dtype, verbose=False)
    return LLMEngine(model, EngineConfig(dtype=dtype, **kw), eos_token_id=cfg.eos_token_id)


def _prompts(tiny, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    out = []
    for n in lengths:
        ids = [tiny.cfg.bos_token_id] + torch.randint(3, tiny.cfg.vocab_size, (n - 1,), generator=g).tolist()
        out.append(ids)
    return out


@pytest.mark.parametrize("dtype", DTYPES)
def test_workload_a_greedy_and_temperature(dtype):
    from transformers_neuronx_b200.engine import SamplingParams
    tiny = _model("A", dtype)
    prompts = _prompts(tiny, [5, 17, 33, 64], seed=0)
    eng = _engine(tiny, dtype, max_num_seqs=4, max_batch_tokens=128)
    greedy = eng.generate(prompts, 32, stop_on_eos=False)
    ties = [check_greedy(tiny, dtype, p, o) for p, o in zip(prompts, greedy)]
    assert all(len(o) == 32 for o in greedy)
    print(f"workload A {dtype}: 4 x 32 greedy tokens compared, ties {ties}")
    params = [SamplingParams(temperature=0.8, seed=0) for _ in prompts]
    drawn = eng.generate(prompts, 32, params, stop_on_eos=False)
    close = [check_sampled(tiny, dtype, p, o, 0.8, 0) for p, o in zip(prompts, drawn)]
    print(f"workload A {dtype}: 4 x 32 tokens at temperature 0.8 compared, near a boundary {close}")
    assert drawn != greedy and sum(close) <= 8
    # greedy and sampled rows in one batch, each with its own parameters (top-k, top-p, suppressed ids, the fixed draw)
    mixed = [SamplingParams(), SamplingParams(temperature=0.8, seed=0), SamplingParams(temperature=1.3, top_k=20, seed=5),
             SamplingParams(temperature=0.0, suppress_eos=True)]
    eos = greedy[3][4]                                           # an id that row 3 would produce greedily
    rids = [eng.add_request(p, 32, q, stop_on_eos=False, eos_token_id=[eos, 7] if i == 3 else None)
            for i, (p, q) in enumerate(zip(prompts, mixed))]
    while eng.has_work():
        eng.step()
    outs = [eng.requests.pop(r).output for r in rids]
    assert check_greedy(tiny, dtype, prompts[0], outs[0]) >= 0
    check_sampled(tiny, dtype, prompts[1], outs[1], 0.8, 0)
    check_sampled(tiny, dtype, prompts[2], outs[2], 1.3, 5, top_k=20)
    assert eos not in outs[3] and 7 not in outs[3]
    check_greedy(tiny, dtype, prompts[3], outs[3], suppress=(eos, 7))


@pytest.mark.parametrize("dtype", DTYPES)
def test_workload_b_sixteen_token_portions_beside_decode(dtype):
    tiny = _model("B", dtype)
    prompts = _prompts(tiny, [1, 40, 120], seed=1)
    eng = _engine(tiny, dtype, max_num_seqs=3, max_batch_tokens=24, max_portion=16)
    seen = {"mixed": 0, "longest_portion": 0}
    inner = eng.runner.step

    def watching(entries, *a, **kw):
        sizes = [len(e.tokens) for e in entries]
        seen["longest_portion"] = max(seen["longest_portion"], max(sizes))
        if any(n > 1 for n in sizes) and any(n == 1 for n in sizes):
            seen["mixed"] += 1
        return inner(entries, *a, **kw)
    eng.runner.step = watching
    outs = eng.generate(prompts, 48, stop_on_eos=False)
    assert seen["longest_portion"] == 16 and seen["mixed"] >= 5, seen
    ties = [check_greedy(tiny, dtype, p, o) for p, o in zip(prompts, outs)]
    assert all(len(o) == 48 for o in outs)
    print(f"workload B {dtype}: 3 x 48 greedy tokens compared, ties {ties}; steps with portions beside decode: {seen['mixed']}")


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_preemption_and_late_end_of_sequence_in_16_bit(dtype):
    """So few pages that running requests are preempted and computed again, sampling ahead of the
    ids' arrival, requests that end on an end-of-sequence id at different steps: every token that
    comes out is checked against the plain implementation."""
    from transformers_neuronx_b200.engine import SamplingParams
    tiny = _model("A", dtype)
    prompts = [tiny.random_ids(n, seed=60 + i) for i, n in enumerate([22, 7, 31, 12, 18])]
    eng = _engine(tiny, dtype, max_num_seqs=3, max_batch_tokens=24, num_pages=10)
    first = eng.generate(prompts, 30, stop_on_eos=False)
    assert eng.stats["preemptions"] > 0, "the pool was meant to be too small"
    for p, o in zip(prompts, first):
        assert len(o) == 30
        check_greedy(tiny, dtype, p, o)
    eos = first[0][9]
    cut = eng.generate(prompts, 30, stop_on_eos=True, eos_token_id=eos)
    for p, o in zip(prompts, cut):
        assert -1 not in o and (eos not in o[:-1]) and (o[-1] == eos or len(o) == 30)
        check_greedy(tiny, dtype, p, o)
    assert any(len(o) < 30 for o in cut)
    params = [SamplingParams(temperature=0.9, top_k=40, seed=3 + i) for i in range(len(prompts))]
    drawn = eng.generate(prompts, 30, params, stop_on_eos=False)
    for i, (p, o) in enumerate(zip(prompts, drawn)):
        check_sampled(tiny, dtype, p, o, 0.9, 3 + i, top_k=40)
    assert eng.runner.cache.free_pages() == [10] and eng.runner.cache.slots.num_free == 3
    eng.runner.cache.check()


def test_a_request_that_cannot_be_sampled_is_refused_when_it_is_submitted():
    from transformers_neuronx_b200.engine import SamplingParams
    tiny = _model("A", "float32")
    eng = _engine(tiny, "float32", max_num_seqs=2)
    with pytest.raises(ValueError, match="at most 4"):
        eng.add_request([2, 5], 4, SamplingParams(suppress_eos=True), eos_token_id=[1, 2, 3, 4, 5])
    with pytest.raises(ValueError, match="at least 1"):
        eng.add_request([2, 5], 0)
    assert not eng.has_work()
