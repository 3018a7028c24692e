"""What the engine does when something is wrong: a step that names a bad token, a request twice, or
more tokens than a request may hold is refused before anything runs; a bounded wait that runs out
inside a kernel is reported at the step whose results it spoiled, not sampled from."""
import pytest
import torch

from helpers import TinyModel

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tiny():
    return TinyModel("A", seed=61)


def _runner(tiny, dtype="float32", **kw):
    from transformers_neuronx_b200.engine import StepRunner, load_model
    model, _ = load_model(tiny.folder, dtype, verbose=False)
    return StepRunner(model, 16, kw.pop("num_pages", 8), 2, kw.pop("max_model_len", 40), **kw)


def test_a_bad_step_is_refused_and_leaves_the_cache_as_it_was(tiny):
    from transformers_neuronx_b200.cache import OutOfPages
    from transformers_neuronx_b200.engine import StepEntry
    runner = _runner(tiny, num_pages=3)
    runner.add_request("a"); runner.add_request("b")
    ids = tiny.random_ids(20, seed=1)
    runner.step([StepEntry("a", ids[:10], [9])])
    before = (runner.cache.length("a"), runner.cache.length("b"), runner.cache.free_pages())
    V = tiny.cfg.vocab_size
    for entries, exc, text in [
        ([StepEntry("a", [5, V], [0])], ValueError, "out of range"),
        ([StepEntry("a", [-1], [0])], ValueError, "out of range"),
        ([StepEntry("a", [5], [0]), StepEntry("a", [6], [0])], ValueError, "twice"),
        ([StepEntry("a", ids[:10] * 4, [])], ValueError, "limit is 40"),
        ([StepEntry("zz", [5], [0])], KeyError, "not live"),
        ([StepEntry("a", [], [])], ValueError, "at least one token"),
        ([StepEntry("a", [5, 6], [2])], ValueError, "wanted place"),
        ([StepEntry("a", [5, 6], [], from_device=0)], ValueError, "only token"),
        ([StepEntry("b", ids[:10] * 4, [])], OutOfPages, "free"),        # 40 tokens need 3 pages, 2 are free
        ([], ValueError, "at least one entry"),
    ]:
        with pytest.raises(exc, match=text):
            runner.step(entries)
        assert (runner.cache.length("a"), runner.cache.length("b"), runner.cache.free_pages()) == before
        runner.cache.check()
    # and the runner still works: the next token's logits are those of the plain implementation
    lg = runner.step([StepEntry("a", ids[10:], [9])]).cpu()
    want = tiny.plain_logits(ids)[-1]
    assert float((lg[0] - want).abs().max() / want.abs().max()) <= 2e-5


def test_a_wait_that_runs_out_is_reported(tiny):
    """A kernel's bounded wait gives up after about a millisecond (nothing ever arrives at its
    barrier), sets the device's error word and returns; the context stays usable."""
    from transformers_neuronx_b200.kernels import ops
    dev = torch.device("cuda:0")
    ops.raise_on_device_error()
    ops.selftest_wait_runs_out(dev, code=77)
    torch.cuda.synchronize()
    with pytest.raises(ops.KernelError, match="77"):
        ops.raise_on_device_error()
    ops.raise_on_device_error()                               # the word was cleared by the report
    a = torch.ones(4, device=dev)
    assert float((a + a).sum()) == 8.0                        # the GPU still answers


def test_the_engine_reads_the_error_word_with_every_steps_ids(tiny):
    """The error word travels to the host with the sampled ids, in the same copy: a step that ran
    after a wait gave up raises instead of handing out tokens."""
    from transformers_neuronx_b200.config import EngineConfig
    from transformers_neuronx_b200.engine import LLMEngine, load_model
    from transformers_neuronx_b200.kernels import ops
    model, cfg = load_model(tiny.folder, "bfloat16", verbose=False)
    eng = LLMEngine(model, EngineConfig(dtype="bfloat16", max_num_seqs=2), eos_token_id=cfg.eos_token_id)
    eng.add_request(tiny.random_ids(9, seed=2), 6, stop_on_eos=False)
    eng.step(); eng.step()
    ops.selftest_wait_runs_out(model.device, code=55)
    with pytest.raises(ops.KernelError, match="55.*invalid"):
        for _ in range(4):
            eng.step()
    ops.raise_on_device_error()                               # cleared
    # the entry point's forward checks it too, before logits go to the host
    from transformers_neuronx_b200.opt.model import OPTForSampling
    m = OPTForSampling.from_pretrained(tiny.folder, batch_size=1, amp="bf16", n_positions=32).to_neuron()
    ops.selftest_wait_runs_out(model.device, code=56)
    with pytest.raises(ops.KernelError, match="56"):
        m.forward(torch.tensor([tiny.random_ids(6, seed=3)]))
    ops.raise_on_device_error()
