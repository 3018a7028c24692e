"""The three element types of the reference (f32, f16, bf16; src/transformers_neuronx/dtypes.py:18-35)
as stored types and as engine types, and the activations that config.json may name: a float16
checkpoint read without loss by the 32-bit path, matrices stored in 32-bit through the engine, the
float16 serving path through the entry point, the warning when a 16-bit engine has to round the
other 16-bit type, and each activation through replay."""
import warnings

import pytest
import torch

from helpers import TOLERANCE, TinyModel, check_greedy, compare_trace, run_trace_inprocess, storage_for

pytestmark = pytest.mark.gpu


def _whole_steps(reqs):
    return [{"step": i, "entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], "end": [rid]}
            for i, (rid, ids) in enumerate(reqs.items())]


def test_float16_checkpoint_is_read_without_loss_by_the_32_bit_path():
    """Matrices stored in float16 hold values that bfloat16 cannot represent; the 32-bit engine must
    compute with exactly those values (2e-5 against the plain implementation fed the float16 values),
    which rounding them to bfloat16 on the way would miss by three orders of magnitude."""
    tiny = TinyModel("A", seed=31, matrix_dtype=torch.float16)
    w = tiny.plain_tensors["model.decoder.layers.0.fc1.weight"]
    assert w.dtype == torch.float16
    lost = (w.to(torch.bfloat16).to(torch.float16) != w).float().mean()
    assert lost > 0.5, "most float16 values must not be bfloat16 values for this test to mean anything"
    reqs = {f"h{i}": tiny.random_ids(n, seed=700 + i) for i, n in enumerate([64, 17, 120])}
    steps = _whole_steps(reqs)
    res = run_trace_inprocess(tiny.folder, "float32", steps, 128)
    worst = compare_trace(tiny, reqs, steps, res, "float32")
    # and the same values rounded to bfloat16 would not have passed: the test can fail
    rounded = {k: (v.to(torch.bfloat16).to(torch.float16) if v.dtype == torch.float16 else v) for k, v in tiny.plain_tensors.items()}
    from plain import opt_plain
    ids = reqs["h0"]
    a = opt_plain.forward_logits(ids, tiny.plain_tensors, tiny.cfg.to_dict())
    b = opt_plain.forward_logits(ids, rounded, tiny.cfg.to_dict())
    assert float((a - b).abs().max() / a.abs().max()) > 20 * TOLERANCE["float32"] > worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float16"])
def test_matrices_stored_in_32_bit(dtype):
    """A folder as `opt_demo --amp f32 save` writes it: every matrix in 32-bit.  The 32-bit engine
    reads it as it is; in a 16-bit engine such a matrix still runs on the 32-bit product kernel, so
    only the activations between the kernels are rounded."""
    from transformers_neuronx_b200.config import EngineConfig
    from transformers_neuronx_b200.engine import LLMEngine, load_model
    tiny = TinyModel("B", seed=37, matrix_dtype=torch.float32)
    assert all(t.dtype == torch.float32 for t in tiny.plain_tensors.values())
    reqs = {f"w{i}": tiny.random_ids(n, seed=800 + i) for i, n in enumerate([40, 121, 9])}
    steps = _whole_steps(reqs)
    res = run_trace_inprocess(tiny.folder, dtype, steps, 128)
    compare_trace(tiny, reqs, steps, res, dtype)
    # through the engine: greedy tokens against the plain implementation's
    model, cfg = load_model(tiny.folder, dtype, verbose=False)
    eng = LLMEngine(model, EngineConfig(dtype=dtype, max_num_seqs=2, max_batch_tokens=16), eos_token_id=cfg.eos_token_id)
    prompt = tiny.random_ids(21, seed=5)
    got = eng.generate([prompt], 12, stop_on_eos=False)[0]
    seq, compared = list(prompt), 0
    for t in got:
        lg = tiny.plain_logits(seq)[-1]
        top = torch.topk(lg, 2).values
        if t != int(lg.argmax()):
            assert float(top[0] - top[1]) / float(lg.abs().max()) <= 2 * TOLERANCE[dtype]
            break
        seq.append(t); compared += 1
    assert compared >= (12 if dtype == "float32" else 1)


def test_a_16_bit_engine_says_when_it_rounds_the_other_16_bit_type():
    from transformers_neuronx_b200.engine import load_model
    tiny = TinyModel("A", seed=41, matrix_dtype=torch.float16)
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        model, _ = load_model(tiny.folder, "bfloat16", verbose=False)
    assert any("rounded to bfloat16" in str(w.message) for w in caught)
    assert model.embedding.table.dtype == torch.bfloat16
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        model, _ = load_model(tiny.folder, "float16", verbose=False)
        model32, _ = load_model(tiny.folder, "float32", verbose=False)
    assert not [w for w in caught if "rounded" in str(w.message)]
    assert model.embedding.table.dtype == torch.float16 and model32.embedding.table.dtype == torch.float16


def test_float16_through_the_entry_point():
    """amp='f16' (the type OPT checkpoints are stored in) is a serving path of its own: the same
    kernels compiled with float16 as their 16-bit type."""
    from transformers_neuronx_b200.opt.model import OPTForSampling
    tiny = TinyModel("D", seed=43, matrix_dtype=torch.float16, overrides={"torch_dtype": "float16"})
    model = OPTForSampling.from_pretrained(tiny.folder, batch_size=2, n_positions=200)     # amp from torch_dtype
    assert model.amp == "f16" and model.dtype == "float16"
    model.to_neuron()
    assert model.model.act_dtype == torch.float16
    prompts = [tiny.random_ids(150, seed=s) for s in (1, 2)]
    out = model.sample(torch.tensor(prompts), sequence_length=170, top_k=1)
    for row, prompt in zip(out.tolist(), prompts):
        check_greedy(tiny, "float16", prompt, row[150:], suppress=(tiny.cfg.eos_token_id,))   # sample() never draws that id
    lg = model.forward(torch.tensor(prompts))
    for b in range(2):
        want = tiny.plain_logits(prompts[b])[-1]
        assert float((lg[b] - want).abs().max()) / float(want.abs().max()) <= TOLERANCE["float16"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float16"])
@pytest.mark.parametrize("name", ["gelu", "gelu_new", "silu", "sigmoid"])
def test_activation_named_by_the_configuration(name, dtype):
    """config.json's activation_function is looked up by name, as the reference does
    (hlo.py:485-501): configuration A with another activation through chunked replay."""
    tiny = TinyModel("A", seed=47, matrix_dtype=storage_for(dtype), overrides={"activation_function": name})
    reqs = {f"a{i}": tiny.random_ids(n, seed=900 + i) for i, n in enumerate([50, 100])}
    steps, k = [], 0
    for rid, ids in reqs.items():
        for p0, p1 in ((0, 33), (33, len(ids) - 3)):
            steps.append({"step": k, "entries": [{"id": rid, "tokens": ids[p0:p1], "want": [0, p1 - p0 - 1]}], "end": []}); k += 1
        for j in range(len(ids) - 3, len(ids)):
            steps.append({"step": k, "entries": [{"id": rid, "tokens": [ids[j]], "want": [0]}],
                          "end": [rid] if j == len(ids) - 1 else []}); k += 1
    res = run_trace_inprocess(tiny.folder, dtype, steps, 128)
    compare_trace(tiny, reqs, steps, res, dtype)


def test_an_activation_that_is_not_built_is_refused_by_name():
    from transformers_neuronx_b200.engine import load_model
    from transformers_neuronx_b200.kernels.ops import KernelError
    tiny = TinyModel("A", seed=47)
    import json, os
    path = os.path.join(tiny.folder, "config.json")
    cfg = json.load(open(path)); cfg["activation_function"] = "solu"
    json.dump(cfg, open(path, "w"))
    with pytest.raises(KernelError, match="solu.*available.*gelu_new"):
        load_model(tiny.folder, "float32", verbose=False)
