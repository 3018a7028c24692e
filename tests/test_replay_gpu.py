"""Trace replay against the plain implementation, in 32-bit and in bfloat16: each request alone and
whole; most of it in one step and the last 32 tokens one by one; in portions of changing size down
to two tokens; and mixed, up to four live requests with so few pages that they are used again."""
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

from helpers import (TOLERANCE, TinyModel, compare_trace, live_tokens_rounded, run_trace_inprocess,
                     storage_for, trace_lines)

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16", "float16"]
LENGTHS = {"A": [5, 17, 33, 64, 120], "B": [1, 40, 120, 250]}
_models = {}


def _model(name, dtype, seed):
    """One model folder per (configuration, storage type): a 16-bit engine reads matrices stored in its own type."""
    key = (name, storage_for(dtype), seed)
    if key not in _models:
        _models[key] = TinyModel(name, seed=seed, matrix_dtype=storage_for(dtype))
    return _models[key]


@pytest.fixture(scope="module", params=["A", "B"])
def tiny_name(request):
    return request.param


@pytest.fixture
def tiny(tiny_name, dtype):
    return _model(tiny_name, dtype, 11)


def _requests(tiny, lengths=None):
    lengths = lengths or LENGTHS[tiny.name]
    return {f"r{i}": tiny.random_ids(n, seed=100 + i) for i, n in enumerate(lengths)}


@pytest.mark.parametrize("dtype", DTYPES)
def test_whole(tiny, dtype):
    reqs = _requests(tiny)
    steps = [{"step": i, "entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], "end": [rid]}
             for i, (rid, ids) in enumerate(reqs.items())]
    res = run_trace_inprocess(tiny.folder, dtype, steps, live_tokens_rounded([max(len(v) for v in reqs.values())]))
    compare_trace(tiny, reqs, steps, res, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prefix_then_one_by_one(tiny, dtype):
    reqs = _requests(tiny, [n for n in LENGTHS[tiny.name] if n > 33])
    steps, k = [], 0
    for rid, ids in reqs.items():
        cut = len(ids) - 32
        steps.append({"step": k, "entries": [{"id": rid, "tokens": ids[:cut], "want": [cut - 1]}], "end": []})
        k += 1
        for j in range(cut, len(ids)):
            steps.append({"step": k, "entries": [{"id": rid, "tokens": [ids[j]], "want": [0]}],
                          "end": [rid] if j == len(ids) - 1 else []})
            k += 1
    res = run_trace_inprocess(tiny.folder, dtype, steps, live_tokens_rounded([max(len(v) for v in reqs.values())]))
    compare_trace(tiny, reqs, steps, res, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_portions_of_changing_size(tiny, dtype):
    reqs = _requests(tiny, [n for n in LENGTHS[tiny.name] if n >= 17])
    sizes = [2, 3, 16, 2, 7, 17, 5, 2, 31, 4, 15, 33]
    steps, k = [], 0
    for rid, ids in reqs.items():
        p, j = 0, 0
        while p < len(ids):
            n = min(sizes[j % len(sizes)], len(ids) - p)
            if len(ids) - p - n == 1:      # never leave a single token: portions go down to two
                n += 1
            steps.append({"step": k, "entries": [{"id": rid, "tokens": ids[p:p + n], "want": [0, n - 1]}],
                          "end": [rid] if p + n == len(ids) else []})
            p += n; j += 1; k += 1
    res = run_trace_inprocess(tiny.folder, dtype, steps, live_tokens_rounded([max(len(v) for v in reqs.values())]))
    compare_trace(tiny, reqs, steps, res, dtype)


def mixed_steps(reqs, chunk_sizes=(7, 16, 2, 21, 5), decode_tail=12, max_live=4):
    """Up to `max_live` requests live: portions of some prompts beside single decoded tokens of others;
    a request ends, its pages go back, and the next waiting request takes them."""
    waiting = list(reqs.items())
    live = {}          # rid -> position reached
    steps, k, j = [], 0, 0
    peak = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, ids = waiting.pop(0)
            live[rid] = 0
        entries, end = [], []
        for rid in list(live):
            ids, p = reqs[rid], live[rid]
            prompt_end = max(1, len(ids) - decode_tail)
            if p < prompt_end:
                n = min(chunk_sizes[j % len(chunk_sizes)], prompt_end - p)
                j += 1
                if k % 3 == 2 and len(entries) >= 2:
                    continue                 # a request may be left out of a step and go on later
                want = [n - 1]
            else:
                n, want = 1, [0]
            entries.append({"id": rid, "tokens": ids[p:p + n], "want": want})
            live[rid] = p + n
            if live[rid] == len(ids):
                end.append(rid)
        peak = max(peak, live_tokens_rounded([live[r] for r in live]))
        steps.append({"step": k, "entries": entries, "end": end})
        for rid in end:
            del live[rid]
        k += 1
    return steps, peak


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixed_with_page_reuse(tiny, dtype):
    lens = {"A": [40, 90, 17, 64, 120, 33, 75, 50], "B": [120, 30, 200, 64, 250, 90, 45, 160]}[tiny.name]
    reqs = _requests(tiny, lens)
    steps, peak = mixed_steps(reqs)
    assert sum(-(-n // 64) * 64 for n in lens) > peak, "the pool must be too small for all requests at once"
    res = run_trace_inprocess(tiny.folder, dtype, steps, peak)
    compare_trace(tiny, reqs, steps, res, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_sizes_outside_the_fast_kernels_rules(dtype):
    """Configuration C: head size 48, widths that are no multiples of 8, an odd vocabulary: the engine
    takes the slower kernels where the fast ones refuse, and the logits are still right."""
    tiny = _model("C", dtype, 13)
    reqs = {f"c{i}": tiny.random_ids(n, seed=300 + i) for i, n in enumerate([70, 33, 9, 78, 50, 21])}
    steps, peak = mixed_steps(reqs, chunk_sizes=(5, 16, 2, 19), decode_tail=10, max_live=3)
    res = run_trace_inprocess(tiny.folder, dtype, steps, peak)
    compare_trace(tiny, reqs, steps, res, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_head_size_128_long_contexts(dtype):
    """Configuration D: head size 128 (the tcgen05 attention kernel in bfloat16), prompts of several
    hundred tokens in portions that start inside a page and cross 128-row tiles, beside decode tokens."""
    tiny = _model("D", dtype, 19)
    reqs = {f"l{i}": tiny.random_ids(n, seed=500 + i) for i, n in enumerate([590, 133, 300, 64, 411, 257])}
    steps, peak = mixed_steps(reqs, chunk_sizes=(129, 16, 2, 200, 75, 128), decode_tail=9, max_live=3)
    res = run_trace_inprocess(tiny.folder, dtype, steps, peak)
    compare_trace(tiny, reqs, steps, res, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_head_size_64(dtype):
    """Configuration E: head size 64 (the tcgen05 attention kernel's other size), post-norm blocks."""
    tiny = _model("E", dtype, 23)
    reqs = {f"e{i}": tiny.random_ids(n, seed=600 + i) for i, n in enumerate([410, 130, 257, 66, 300])}
    steps, peak = mixed_steps(reqs, chunk_sizes=(130, 2, 64, 17, 150), decode_tail=9, max_live=3)
    res = run_trace_inprocess(tiny.folder, dtype, steps, peak)
    compare_trace(tiny, reqs, steps, res, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_head_size_80(dtype):
    """Configuration F: head size 80, which is neither of the tcgen05 attention kernel's native sizes
    (it runs in the layout of 128 with the columns beyond 80 left out of the products)."""
    tiny = _model("F", dtype, 29)
    reqs = {f"f{i}": tiny.random_ids(n, seed=700 + i) for i, n in enumerate([390, 130, 257, 66, 200])}
    steps, peak = mixed_steps(reqs, chunk_sizes=(130, 2, 64, 17, 150), decode_tail=9, max_live=3)
    res = run_trace_inprocess(tiny.folder, dtype, steps, peak)
    compare_trace(tiny, reqs, steps, res, dtype)


def _random_trace(rng, tiny, n_req, max_live):
    """Requests of random lengths cut at random: single tokens, portions of 2 to 200 tokens, requests left out
    of a step, random wanted rows, at most max_live alive; the pool is sized for the peak, so pages come back."""
    maxlen = tiny.cfg.max_position_embeddings
    reqs = {f"q{i}": tiny.random_ids(rng.randint(1, maxlen), seed=rng.randrange(10 ** 6)) for i in range(n_req)}
    waiting, live, steps, peak = list(reqs), {}, [], 0
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.7):
            live[waiting.pop(0)] = 0
        entries, end = [], []
        for rid in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue
            ids, p = reqs[rid], live[rid]
            n = 1 if rng.random() < 0.45 else rng.choice([1, 2, 3, 5, 15, 16, 17, 31, 33, 64, 65, 127, 129, 200])
            n = min(n, len(ids) - p)
            want = sorted(set(rng.sample(range(n), min(n, rng.choice([0, 1, 1, 2, 3])))) | ({n - 1} if rng.random() < 0.7 else set()))
            entries.append({"id": rid, "tokens": ids[p:p + n], "want": want})
            live[rid] = p + n
            if live[rid] == len(ids):
                end.append(rid)
        if not entries:
            continue
        peak = max(peak, live_tokens_rounded([live[r] for r in live]))
        steps.append({"step": len(steps), "entries": entries, "end": end})
        for rid in end:
            del live[rid]
    return reqs, steps, peak


@pytest.mark.parametrize("seed", range(6))
def test_random_traces(seed):
    """Random cuts and interleavings of random requests, one configuration per seed, in all three types."""
    import random
    rng = random.Random(1000 + seed)
    name = "ABCDEF"[seed]
    models = {dt: _model(name, dt, 31 + seed) for dt in DTYPES}
    reqs, steps, peak = _random_trace(rng, models["float32"], rng.randint(3, 6), rng.randint(1, 4))
    for dt in DTYPES:
        res = run_trace_inprocess(models[dt].folder, dt, steps, peak)
        compare_trace(models[dt], reqs, steps, res, dt)


@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_steps_where_not_every_request_wants_logits(dtype):
    """Single-token steps (replayed as CUDA graphs) in which some entries ask for nothing."""
    tiny = _model("A", dtype, 17)
    reqs = {f"d{i}": tiny.random_ids(n, seed=400 + i) for i, n in enumerate([30, 26, 22])}
    steps = [{"step": 0, "entries": [{"id": r, "tokens": ids[:20], "want": []} for r, ids in reqs.items()], "end": []}]
    for t in range(20, 30):
        entries = []
        for i, (r, ids) in enumerate(reqs.items()):
            if t < len(ids):
                entries.append({"id": r, "tokens": [ids[t]], "want": [0] if (t + i) % 3 else []})
        steps.append({"step": len(steps), "entries": entries, "end": []})
    res = run_trace_inprocess(tiny.folder, dtype, steps, 192)
    assert 0 not in res, "a step in which nothing is wanted writes no file (run_trace_inprocess checks there is none)"
    assert any(s["step"] not in res for s in steps[1:]), "the trace was meant to hold decode steps without a wanted row"
    compare_trace(tiny, reqs, steps, res, dtype)


def test_32_bit_logits_do_not_depend_on_the_cut_bit_for_bit(tiny_name):
    """The 32-bit path adds every sum in an order that the row alone decides (products in ascending
    k with one accumulator, attention key by key, norms per row): the logits of a position are the
    same bits whether its request ran whole, token by token, in portions, or beside other requests
    on other pages."""
    tiny = _model(tiny_name, "float32", 11)
    ids = tiny.random_ids(LENGTHS[tiny.name][-1], seed=100)
    other = {f"o{i}": tiny.random_ids(n, seed=140 + i) for i, n in enumerate([50, 23, 64])}
    n = len(ids)
    want_all = list(range(n))
    whole = [{"step": 0, "entries": [{"id": "x", "tokens": ids, "want": want_all}], "end": ["x"]}]
    cut = n - 32
    tail = [{"step": 0, "entries": [{"id": "x", "tokens": ids[:cut], "want": list(range(cut))}], "end": []}]
    tail += [{"step": 1 + j, "entries": [{"id": "x", "tokens": [ids[cut + j]], "want": [0]}], "end": []} for j in range(32)]
    sizes, portions, p, j = [2, 3, 16, 2, 7, 17, 5, 2, 31, 4, 15, 33], [], 0, 0
    while p < n:
        m = min(sizes[j % len(sizes)], n - p)
        portions.append({"step": len(portions), "entries": [{"id": "x", "tokens": ids[p:p + m], "want": list(range(m))}], "end": []})
        p += m; j += 1
    # mixed: other requests come first and take the low pages, end, and x goes on over their pages
    mixed, p, k = [], 0, 0
    opos = {r: 0 for r in other}
    mixed.append({"step": 0, "entries": [{"id": r, "tokens": t[:20], "want": []} for r, t in other.items()], "end": []})
    for r in other:
        opos[r] = 20
    while p < n:
        m = min(sizes[(k + 5) % len(sizes)], n - p)
        entries = [{"id": "x", "tokens": ids[p:p + m], "want": list(range(m))}]
        end = []
        for r, t in other.items():
            if r in opos and opos[r] < len(t):
                entries.insert(0, {"id": r, "tokens": [t[opos[r]]], "want": [0] if k % 2 else []})
                opos[r] += 1
                if opos[r] == len(t):
                    end.append(r)
        mixed.append({"step": len(mixed), "entries": entries, "end": end})
        p += m; k += 1

    def rows_of_x(steps, max_tokens):
        res = run_trace_inprocess(tiny.folder, "float32", steps, max_tokens)
        rows = []
        for s_ in steps:
            row = 0
            for e in s_["entries"]:
                nw = len(e.get("want", []))
                if e["id"] == "x" and nw:
                    rows.append(torch.from_numpy(res[s_["step"]][row:row + nw].copy()))
                row += nw
        return torch.cat(rows)
    a = rows_of_x(whole, 256)
    assert a.shape[0] == n
    for name, steps, room in (("one by one", tail, 256), ("portions", portions, 256), ("mixed", mixed, 256 + 3 * 64)):
        b = rows_of_x(steps, room)
        assert torch.equal(a, b), f"{tiny.name}: {name} differs from whole by {float((a - b).abs().max()):.3e}"


def test_program_in_a_subprocess():
    """bin/trace_run itself, as a user calls it: steps on stdin, `done` lines, files, exit code 0."""
    tiny = TinyModel("A", seed=3)
    ids = tiny.random_ids(40, seed=5)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": ids[:30], "want": [29]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": ids[30:], "want": [0, 9]}], "end": ["x"]},
             {"step": 2, "entries": [{"id": "y", "tokens": ids[:8], "want": []}], "end": ["y"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tempfile.mkdtemp(prefix="tnx_trace_sub_")
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", tiny.folder,
                           "--dtype", "float32", "--out", out, "--max-tokens", "64"],
                          input="\n".join(trace_lines(steps)) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not os.path.exists(os.path.join(out, "2.f32"))
    plain = tiny.plain_logits(ids)
    got0 = np.fromfile(os.path.join(out, "0.f32"), dtype="<f4").reshape(1, -1)
    got1 = np.fromfile(os.path.join(out, "1.f32"), dtype="<f4").reshape(2, -1)
    for got, p in ((got0[0], 29), (got1[0], 30), (got1[1], 39)):
        err = float(np.abs(got - plain[p].numpy()).max()) / float(plain[p].abs().max())
        assert err <= TOLERANCE["float32"]


@pytest.mark.parametrize("dtype", DTYPES)
def test_small_steps_with_portions_are_captured_and_replayed(tiny, dtype):
    """Steps of a few tokens with prompt portions run as CUDA graphs padded to a few sizes: the
    same shapes come again and again here (first use eager, second captured, then replayed), with
    portions beside decoded tokens, none, few and all logits wanted, and pages used again."""
    from transformers_neuronx_b200.engine import StepEntry, StepRunner, load_model
    model, _ = load_model(tiny.folder, dtype, verbose=False)
    runner = StepRunner(model, 16, 20, 4, 256, use_cuda_graphs=True)
    worst = 0.0
    for rnd in range(6):
        reqs = {f"s{rnd}_{i}": tiny.random_ids(n, seed=900 + 10 * rnd + i) for i, n in enumerate([70, 45, 61])}
        plain = {r: tiny.plain_logits(ids) for r, ids in reqs.items()}
        pos = {r: 0 for r in reqs}
        for r in reqs:
            runner.add_request(r)
        sizes = {0: [9, 1, 1, 14, 2, 1], 1: [5, 30, 1, 3, 1, 1], 2: [17, 2, 1, 1, 8, 1]}
        k = 0
        while any(pos[r] < len(reqs[r]) for r in reqs):
            entries, checks = [], []
            for i, r in enumerate(reqs):
                left = len(reqs[r]) - pos[r]
                if left == 0 or (k + i) % 4 == 3:                    # a request may sit a step out
                    continue
                n = min(sizes[i][k % 6], left)
                want = [] if (k + i) % 3 == 0 else ([n - 1] if (k + i) % 3 == 1 else list(range(n)))
                entries.append(StepEntry(r, reqs[r][pos[r]:pos[r] + n], want))
                checks += [(r, pos[r] + w) for w in want]
                pos[r] += n
            k += 1
            if not entries:
                continue
            logits = runner.step(entries).cpu()
            assert logits.shape[0] == len(checks)
            for row, (r, p) in enumerate(checks):
                err = float((logits[row] - plain[r][p]).abs().max()) / float(plain[r][p].abs().max())
                worst = max(worst, err)
                assert err <= TOLERANCE[dtype], f"{dtype} round {rnd} step {k} request {r} position {p}: {err:.3e}"
        for r in reqs:
            runner.finish(r)
        runner.cache.check()
    replayed = {key: runs for key, runs in runner.captured_steps().items() if isinstance(key[0], tuple) and key[0][0] == "portions"}
    assert replayed and max(replayed.values()) >= 4, runner.captured_steps()


def test_shapes_beyond_the_graph_limit_run_eagerly():
    from transformers_neuronx_b200.engine import StepEntry, StepRunner, load_model
    tiny = TinyModel("A", seed=29)
    model, _ = load_model(tiny.folder, "bfloat16", verbose=False)
    runner = StepRunner(model, 16, 16, 2, 128, use_cuda_graphs=True, max_graphs=2)
    ids = tiny.random_ids(120, seed=77)
    plain = tiny.plain_logits(ids)
    runner.add_request("g")
    pos = 0
    for n in [3, 3, 3, 20, 20, 20, 1, 1, 1, 35, 1, 1, 5]:        # four shapes; only the first two are kept
        lg = runner.step([StepEntry("g", ids[pos:pos + n], [n - 1])]).cpu()
        err = float((lg[0] - plain[pos + n - 1]).abs().max()) / float(plain[pos + n - 1].abs().max())
        assert err <= TOLERANCE["bfloat16"], (pos, n, err)
        pos += n
    assert len(runner.captured_steps()) == 2
