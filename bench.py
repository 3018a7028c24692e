#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, on the layer sizes of OPT-6.7B with
random weights (the reference publishes no number for them, so vs_baseline is null).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  `value` is decoded tokens per second at batch 8 with the context ending at
2,048, timed on the device over exactly K decode steps; `e2e` is the same through the Python entry
point's engine loop (host token ids in through pinned memory, sampled ids out, every step);
`prefill` is one 2,048-token prompt; `roofline` is the decode step's bytes (every weight once plus
the live requests' cache) over its time.  `points` holds decode at batch 1 and 64 with their
roofline fractions, decode at batch 8 with the context ending at 1,024, 1,536 and 2,048 (the metric
is "1,024-token prompts decoded to 2,048"), the percentiles of the step time over 256 consecutive
decode steps (the reference reports p0/50/90/95/99/100 of its latencies,
src/transformers_neuronx/generation_demo.py:157-163), and the two further workloads of the baseline:
OPT-30B sizes decoding at batch 16, and OPT-13B sizes serving 32 requests with a 512-token budget.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

OPT_6_7B = dict(vocab_size=50272, hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, ffn_dim=16384,
                max_position_embeddings=2048, word_embed_proj_dim=4096, do_layer_norm_before=True, enable_bias=True,
                layer_norm_elementwise_affine=True, activation_function="relu", init_std=0.02,
                architectures=["OPTForCausalLM"], model_type="opt", torch_dtype="float16")
OPT_13B = dict(OPT_6_7B, hidden_size=5120, num_hidden_layers=40, num_attention_heads=40, ffn_dim=20480, word_embed_proj_dim=5120)
OPT_30B = dict(OPT_6_7B, hidden_size=7168, num_hidden_layers=48, num_attention_heads=56, ffn_dim=28672, word_embed_proj_dim=7168)
# the other published sizes of the family (facebook/opt-* config.json values): layers, width, heads, ffn, embedding width
OPT_FAMILY = {
    "125m": dict(OPT_6_7B, hidden_size=768, num_hidden_layers=12, num_attention_heads=12, ffn_dim=3072, word_embed_proj_dim=768),
    "350m": dict(OPT_6_7B, hidden_size=1024, num_hidden_layers=24, num_attention_heads=16, ffn_dim=4096, word_embed_proj_dim=512,
                 do_layer_norm_before=False),
    "1.3b": dict(OPT_6_7B, hidden_size=2048, num_hidden_layers=24, num_attention_heads=32, ffn_dim=8192, word_embed_proj_dim=2048),
    "2.7b": dict(OPT_6_7B, hidden_size=2560, num_hidden_layers=32, num_attention_heads=32, ffn_dim=10240, word_embed_proj_dim=2560),
    "6.7b": OPT_6_7B, "13b": OPT_13B, "30b": OPT_30B,
    "66b": dict(OPT_6_7B, hidden_size=9216, num_hidden_layers=64, num_attention_heads=72, ffn_dim=36864, word_embed_proj_dim=9216),
}
CONTEXT = 2048
PREFILL_TOKENS = 2048


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm, tf, src = 6650.0, 1590.0, "fallback"
    if os.path.isfile(path):
        try:
            with open(path) as fp:
                d = json.load(fp)
            hbm = float(d.get("hbm_gbs", hbm))
            tf = float(d.get("bf16_tflops", tf))
            src = "measured"
        except Exception:
            pass
    return hbm, tf, src


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


DTYPE = "float16"        # OPT's own 16-bit type (the baseline's configurations say fp16); --dtype changes it
SHORT = {"float16": "fp16", "bfloat16": "bf16"}


def build(n_layers, dtype=None, base=None):
    import torch
    dtype = dtype or DTYPE
    from transformers_neuronx_b200.config import OPTConfig
    from transformers_neuronx_b200.engine import build_model
    from transformers_neuronx_b200.models import opt as opt_arch
    from transformers_neuronx_b200.models.decoder import DecoderModel
    cfg = OPTConfig.from_dict(dict(base or OPT_6_7B, num_hidden_layers=n_layers))
    spec = opt_arch.build_spec(cfg)
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(0)
    tensors = {}
    for s in DecoderModel(spec).tensor_specs():            # random weights made on the device
        if s.tied_to is not None:
            continue
        t = torch.randn(s.shape, generator=g, device=dev, dtype=torch.float32) * cfg.init_std
        if s.kind == "norm_weight":
            tensors[s.name] = 1.0 + t
        elif s.kind == "norm_bias":
            tensors[s.name] = t
        else:
            tensors[s.name] = t.to(getattr(torch, dtype))
    tensors["lm_head.weight"] = tensors["model.decoder.embed_tokens.weight"]
    model = build_model(spec, tensors, dtype, verbose=False)
    return model, cfg


def decode_bytes(model, cfg, batch, ctx):
    """Bytes one decode step has to read: every weight it uses once (the embedding table as the
    output matrix; of the token and position tables only the batch's rows) and the live cache."""
    H, L = cfg.hidden_size, cfg.num_hidden_layers
    w = model.parameter_bytes()
    pos_table = (cfg.max_position_embeddings + 2) * H * 2
    w = w - pos_table + batch * (H + cfg.word_embed_proj_dim) * 2
    kv = batch * ctx * 2 * H * 2 * L
    return w + kv


def prefill_flops(cfg, T):
    H, F, L, V = cfg.hidden_size, cfg.ffn_dim, cfg.num_hidden_layers, cfg.vocab_size
    per_layer = 2 * T * (4 * H * H + 2 * H * F) + 2 * T * T * H      # products + causal attention
    return L * per_layer + 2 * V * H


def time_decode(model, cfg, batch, steps, warmup, use_engine=False, end=None, per_step=None, tight_pool=False):
    """K decode steps at `batch`, the context ending at `end` (default CONTEXT).  Returns
    (ms_per_step, launches, h2d, d2h); per_step (a list) receives every timed step's own time in ms.
    tight_pool: pages for contexts of `end` only (large batches of short contexts), not of CONTEXT."""
    import torch
    from transformers_neuronx_b200.engine import StepEntry, StepRunner
    from transformers_neuronx_b200.kernels import ops
    total = steps + warmup
    end = end or CONTEXT
    ctx0 = end - total
    pages = batch * ((end + 15) // 16 + 1 if tight_pool else CONTEXT // 16)
    runner = StepRunner(model, 16, pages, max(batch, 1), CONTEXT, use_cuda_graphs=True)
    g = torch.Generator().manual_seed(1)
    for b in range(batch):                                  # the cache as 2,048 - (W + K) earlier tokens left it:
        runner.add_request(b)                               # synthetic keys and values, real bookkeeping
        runner.cache.append(b, ctx0)
    for cid in model.cache_needs():
        runner.storage.tensor(cid).normal_(0, 0.5)
    toks = torch.randint(3, cfg.vocab_size, (total, batch), generator=g).tolist()
    from transformers_neuronx_b200.sampling import Sampler
    sampler = Sampler(model.device)
    pinned = torch.empty(batch, dtype=torch.int32).pin_memory()

    def one(i):
        entries = [StepEntry(b, [toks[i][b]], [0]) for b in range(batch)]
        logits = runner.step(entries)
        if use_engine:
            ids = sampler.sample(logits, [0.0] * batch, [0] * batch, [1.0] * batch, [0] * batch, [i] * batch)
            pinned.copy_(ids, non_blocking=False)            # device -> host read of the step's result
        return logits

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    n0 = ops.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)] if per_step is not None else None
    t0 = time.perf_counter()
    e0.record()
    for i in range(warmup, total):
        if marks:
            marks[i - warmup].record()
        one(i)
    if marks:
        marks[steps].record()
    e1.record()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) * 1e3
    if marks:
        per_step.extend(marks[i].elapsed_time(marks[i + 1]) for i in range(steps))
    launches = ops.launch_count() - n0
    ops.raise_on_device_error()
    ms = e0.elapsed_time(e1) / steps
    if use_engine:
        ms = wall / steps                                    # end to end: the host's clock around the loop
    h2d = getattr(runner, "last_h2d_bytes", 0)
    for b in range(batch):
        runner.finish(b)
    del runner
    torch.cuda.empty_cache()
    return ms, launches, h2d, batch * 4


def time_e2e(model, cfg, batch, steps, warmup):
    """Decode tokens per second through the Python entry point's engine: requests are submitted as
    host token lists, prefilled by the scheduler, and then exactly K decode steps of
    LLMEngine.step() are timed with the host's clock.  Every step packs its inputs into pinned host
    memory, copies them to the device, runs the model, samples on the device and reads the sampled
    ids back to the host."""
    import torch
    from transformers_neuronx_b200.config import EngineConfig
    from transformers_neuronx_b200.engine import LLMEngine
    total = steps + warmup
    prompt_len = CONTEXT - total - 1
    eng = LLMEngine(model, EngineConfig(dtype=DTYPE, max_num_seqs=batch, max_batch_tokens=batch * prompt_len,
                                        max_tokens=batch * CONTEXT, max_model_len=CONTEXT))   # all prompts in one step
    g = torch.Generator().manual_seed(3)
    for b in range(batch):
        prompt = torch.randint(3, cfg.vocab_size, (prompt_len,), generator=g).tolist()
        eng.add_request(prompt, total + 1, stop_on_eos=False)
    while any(r.computed < len(r.prompt) for r in eng.scheduler.running) or eng.scheduler.waiting:
        eng.step()                                            # prefill (not timed)
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    run0 = eng.stats["tokens_run"]
    h2d = 0
    t0 = time.perf_counter()
    for _ in range(steps):
        eng.step()
        h2d = max(h2d, eng.runner.last_h2d_bytes)
    torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) * 1e3 / steps
    assert eng.stats["tokens_run"] - run0 == batch * steps, "every timed step must decode the whole batch"
    del eng
    torch.cuda.empty_cache()
    return ms, h2d, batch * 4


def time_prefill(model, cfg, steps, warmup):
    import torch
    from transformers_neuronx_b200.engine import StepEntry, StepRunner
    runner = StepRunner(model, 16, PREFILL_TOKENS // 16, 1, CONTEXT)
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(3, cfg.vocab_size, (PREFILL_TOKENS,), generator=g).tolist()
    times = []
    for i in range(warmup + steps):
        runner.add_request("p")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        runner.step([StepEntry("p", prompt, [PREFILL_TOKENS - 1])])
        e1.record()
        torch.cuda.synchronize()
        runner.finish("p")
        if i >= warmup:
            times.append(e0.elapsed_time(e1))
    del runner
    return sorted(times)[len(times) // 2]


def workload_decode30b(steps, warmup):
    """OPT-30B sizes, batch 16, context ending at 2,048, greedy."""
    import torch
    model, cfg = build(OPT_30B["num_hidden_layers"], base=OPT_30B)
    ms, _, _, _ = time_decode(model, cfg, 16, steps, warmup)
    nbytes = decode_bytes(model, cfg, 16, CONTEXT - steps / 2)
    hbm, _, _ = peaks()
    out = {"tokens_per_s": round(16 / (ms / 1e3), 1), "ms_per_step": round(ms, 3), "batch": 16, "context": CONTEXT,
           "layers": cfg.num_hidden_layers, "roofline_frac": round(nbytes / (ms / 1e3) / 1e9 / hbm, 4)}
    del model
    torch.cuda.empty_cache()
    return out


def workload_mixed13b():
    """OPT-13B sizes, 32 requests with prompts of 64..1,536 tokens, a budget of 512 tokens a step (one
    prompt portion beside the decode tokens of the others), 256 new tokens each at temperature 0.7,
    through LLMEngine.generate: new tokens per second of wall clock, prefill included; the same
    workload has run once before as warm-up (kernels loaded, every graph captured)."""
    import torch
    from transformers_neuronx_b200.config import EngineConfig
    from transformers_neuronx_b200.engine import LLMEngine, SamplingParams
    model, cfg = build(OPT_13B["num_hidden_layers"], base=OPT_13B)
    g = torch.Generator().manual_seed(4)
    lens = torch.randint(64, 1537, (32,), generator=g).tolist()
    prompts = [torch.randint(3, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    eng = LLMEngine(model, EngineConfig(dtype=DTYPE, max_num_seqs=32, max_batch_tokens=512,
                                        max_tokens=32 * 1792, max_model_len=CONTEXT))
    params = [SamplingParams(temperature=0.7, seed=i) for i in range(32)]
    eng.generate(prompts, 256, params, stop_on_eos=False)
    torch.cuda.synchronize()
    steps0, pre0 = eng.stats["steps"], eng.stats["preemptions"]
    t0 = time.perf_counter()
    out = eng.generate(prompts, 256, params, stop_on_eos=False)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    n_new = sum(len(o) for o in out)
    res = {"new_tokens_per_s": round(n_new / dt, 1), "seconds": round(dt, 3), "requests": 32, "prompt_tokens": sum(lens),
           "new_tokens": n_new, "steps": eng.stats["steps"] - steps0, "preemptions": eng.stats["preemptions"] - pre0,
           "token_budget": 512, "layers": cfg.num_hidden_layers}
    del eng, model
    torch.cuda.empty_cache()
    return res


def workload_family(steps, warmup, sizes=None):
    """Every published size of the family at its full depth: decode at batch 8 (66B: batch 4, so that
    weights and cache fit one GPU) with the context ending at 2,048, batch 1, and a 2,048-token prefill,
    each with its fraction of the measured peak.  The two smallest models' weights are about the size of
    the L2 cache, so their "hbm" fractions say how far the step is from launch-bound, not from DRAM."""
    import torch
    hbm, tflops, _ = peaks()
    rows = {}
    for name in sizes or list(OPT_FAMILY):
        base = OPT_FAMILY[name]
        try:
            model, cfg = build(base["num_hidden_layers"], base=base)
        except torch.OutOfMemoryError as e:
            rows[name] = {"does_not_fit": str(e).split(".")[0]}
            torch.cuda.empty_cache()
            continue
        batch = 4 if name == "66b" else 8
        row = {"layers": cfg.num_hidden_layers, "hidden": cfg.hidden_size, "head_dim": cfg.head_dim,
               "weights_gb": round(model.parameter_bytes() / 1e9, 2)}
        for b in (batch, 1):
            ms, launches, _, _ = time_decode(model, cfg, b, steps, warmup)
            nbytes = decode_bytes(model, cfg, b, CONTEXT - steps / 2)
            row[f"decode_b{b}"] = {"tokens_per_s": round(b / (ms / 1e3), 1), "ms_per_step": round(ms, 3),
                                   "frac_hbm": round(nbytes / (ms / 1e3) / 1e9 / hbm, 4), "launches_per_step": launches // steps}
        pf = time_prefill(model, cfg, 3, 3)
        row["prefill_2048"] = {"ms": round(pf, 3), "tokens_per_s": round(PREFILL_TOKENS / (pf / 1e3), 1),
                               "frac_flops": round(prefill_flops(cfg, PREFILL_TOKENS) / (pf / 1e3) / (tflops * 1e12), 4)}
        rows[name] = row
        del model
        torch.cuda.empty_cache()
    return rows


def workload_sweep(steps, warmup):
    """The decode step over batch x context at the default layer sizes: ms a step and the fraction of the
    measured HBM copy rate, for every pair whose cache fits."""
    import torch
    hbm, _, _ = peaks()
    model, cfg = build(OPT_6_7B["num_hidden_layers"])
    rows = {}
    for end in (256, 512, 1024, 2048):
        row = {}
        for batch in (1, 8, 16, 32, 64, 128, 256):
            if batch * end > 144 * 2048:
                continue
            ms, _, _, _ = time_decode(model, cfg, batch, steps, warmup, end=end, tight_pool=True)
            nbytes = decode_bytes(model, cfg, batch, end - steps / 2)
            row[f"b{batch}"] = [round(ms, 3), round(nbytes / (ms / 1e3) / 1e9 / hbm, 3)]
        rows[f"ctx{end}"] = row
    del model
    torch.cuda.empty_cache()
    return rows


def extra_workload(name, steps, warmup, sizes=None):
    """One of the further workloads alone, printed as one JSON line of its own."""
    if name == "family":
        res = workload_family(steps, warmup, sizes)
    elif name == "sweep":
        res = workload_sweep(steps, warmup)
    else:
        res = workload_decode30b(steps, warmup) if name == "decode30b" else workload_mixed13b()
    print(json.dumps(dict({"workload": name}, **res)))
    return 0


def percentiles(xs):
    xs = sorted(xs)
    pick = lambda q: xs[min(len(xs) - 1, int(round(q / 100 * (len(xs) - 1))))]
    return {f"p{q}": round(pick(q), 4) for q in (0, 50, 90, 95, 99, 100)}


def reference_arm():
    why = ("aws-neuron/transformers-neuronx needs torch_neuronx, libneuronxla and the neuronx-cc compiler for "
           "Trainium/Inferentia; none exists for CUDA, so its OPT path cannot run on a B200")
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=OPT_6_7B["num_hidden_layers"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--skip-points", action="store_true", help="leave out everything under `points`")
    ap.add_argument("--skip-large", action="store_true", help="leave out the OPT-13B and OPT-30B workloads")
    ap.add_argument("--dtype", default="float16", choices=["float16", "bfloat16"],
                    help="the serving type (float16 is what OPT checkpoints are stored in)")
    ap.add_argument("--workload", default=None, choices=["decode30b", "mixed13b", "family", "sweep"],
                    help="run one of the further workloads instead of the default line")
    ap.add_argument("--sizes", default=None, help="for --workload family: comma-separated sizes (default: all of 125m .. 66b)")
    ap.add_argument("--only", default=None, choices=["decode", "prefill"],
                    help="run just this part and print its time (for profiling a small case)")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_arm()
    if a.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus must be 1")
        return 2
    a.warmup = max(a.warmup, 3)
    global DTYPE
    DTYPE = a.dtype
    if a.workload:
        return extra_workload(a.workload, a.steps, a.warmup, a.sizes.split(",") if a.sizes else None)
    import torch
    hbm_gbs, tflops, peak_src = peaks()
    model, cfg = build(a.layers)
    L = cfg.num_hidden_layers

    if a.only == "decode":
        ms, launches, _, _ = time_decode(model, cfg, a.batch, a.steps, a.warmup)
        print(json.dumps({"only": "decode", "batch": a.batch, "layers": L, "ms_per_step": round(ms, 4), "launches": launches}))
        return 0
    if a.only == "prefill":
        ms = time_prefill(model, cfg, a.steps, a.warmup)
        print(json.dumps({"only": "prefill", "tokens": PREFILL_TOKENS, "layers": L, "ms": round(ms, 4)}))
        return 0
    clocks = ClockSampler()
    clocks.start()
    ms, launches, _, _ = time_decode(model, cfg, a.batch, a.steps, a.warmup)
    clk = clocks.stop()
    value = a.batch / (ms / 1e3)
    e2e_ms, h2d, d2h = time_e2e(model, cfg, a.batch, a.steps, a.warmup)
    ctx_mean = CONTEXT - a.steps / 2
    nbytes = decode_bytes(model, cfg, a.batch, ctx_mean)
    achieved = nbytes / (ms / 1e3) / 1e9
    pf_ms = time_prefill(model, cfg, max(3, min(a.steps, 5)), 3)
    pf_flops = prefill_flops(cfg, PREFILL_TOKENS)
    points = {}
    if not a.skip_points:
        for b in (1, 64):
            m, _, _, _ = time_decode(model, cfg, b, a.steps, a.warmup)
            points[f"decode_b{b}"] = round(b / (m / 1e3), 1)
            points[f"decode_b{b}_frac"] = round(decode_bytes(model, cfg, b, ctx_mean) / (m / 1e3) / 1e9 / hbm_gbs, 4)
        # the metric is "1,024-token prompts decoded to 2,048": the same batch with the context ending earlier
        for end in (1024, 1536, 2048):
            m, _, _, _ = time_decode(model, cfg, a.batch, a.steps, a.warmup, end=end)
            points[f"decode_b{a.batch}_ctx{end}"] = round(a.batch / (m / 1e3), 1)
        # every step's own time over 256 consecutive decode steps (contexts 1,792 .. 2,048)
        per_step = []
        time_decode(model, cfg, a.batch, 256, a.warmup, per_step=per_step)
        for k, v in percentiles(per_step).items():
            points[f"step_ms_{k}"] = v
    del model
    torch.cuda.empty_cache()
    if not a.skip_points and not a.skip_large and a.layers == OPT_6_7B["num_hidden_layers"]:
        r30 = workload_decode30b(a.steps, a.warmup)
        points["opt30b_decode_b16"] = r30["tokens_per_s"]
        points["opt30b_decode_b16_frac"] = r30["roofline_frac"]
        r13 = workload_mixed13b()
        points["opt13b_mixed_new_tokens_per_s"] = r13["new_tokens_per_s"]
        points["opt13b_mixed_steps"] = r13["steps"]
    out = {
        "metric": "decode tokens/s (OPT-6.7B sizes, batch 8, context 2048, 1 B200)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": SHORT[DTYPE], "data": "synthetic (random weights N(0,0.02), uniform token ids, synthetic cache contents)",
        "config": {"model": "OPT-6.7B sizes", "layers": L, "layers_of_model": OPT_6_7B["num_hidden_layers"],
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "head_dim": cfg.head_dim,
                   "ffn_dim": cfg.ffn_dim, "vocab": cfg.vocab_size, "max_positions": cfg.max_position_embeddings,
                   "global_batch": a.batch, "seq_len": CONTEXT, "page_size": 16, "parallelism": "none (1 GPU)",
                   "l2": "inputs larger than L2 (weights read once per step)", "peaks": peak_src},
        "e2e": {"value": round(a.batch / (e2e_ms / 1e3), 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "clocks": clk,
        "prefill": {"value": round(PREFILL_TOKENS / (pf_ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pf_ms, 3),
                    "frac": round(pf_flops / (pf_ms / 1e3) / (tflops * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s",
                     "frac": round(achieved / hbm_gbs, 4)},
        "points": points,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
