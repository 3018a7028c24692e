"""Timings of single kernels over sizes and plans, as the summaries under profiles/ quote them.

    python -m transformers_neuronx_b200.kernels.microbench sampling
    python -m transformers_neuronx_b200.kernels.microbench attention-sizes
    python -m transformers_neuronx_b200.kernels.microbench attention-plans [--context 2040] [--rows 1,2,...] [--heads 32,40,56]
    python -m transformers_neuronx_b200.kernels.microbench gemm-plans [--models 30b,13b,6.7b,head]
    python -m transformers_neuronx_b200.kernels.microbench gemm-tokens [--models 6.7b] [--tokens 8,16,...]
    python -m transformers_neuronx_b200.kernels.microbench gemm-splits [--models 1.3b,...,66b] [--tokens 8]

Every number is a CUDA-event time on one GPU: kernels that read more than the second-level cache
holds between two calls are replayed back to back from one CUDA graph over several copies of their
inputs; products are timed one call at a time with the cache flushed before each.  The plan sweeps
impose every plan a kernel could run (the test hooks of kernels/ops.py) beside the library's own
choice, which is how the rules in ops.decode_attention_plan and gemm_tc.cu: plan_many_tokens were
drawn and are checked.
"""
from __future__ import annotations

import argparse
import json
import math
import statistics

import torch

from . import ops

DEV = "cuda:0"


def _graph_time(call, n_calls: int) -> float:
    """Microseconds per call of `call(i)`, i = 0 .. n_calls - 1, captured once and replayed twice."""
    for i in range(2):
        call(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(n_calls):
            call(i)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1000 / (2 * n_calls)


# ---- sampling -----------------------------------------------------------------------------------
def sampling(vocab: int = 50272) -> None:
    """The sampling kernel with 1, 2, 4, 8 thread blocks a row and with its own choice."""
    kinds = (("greedy", {}), ("temperature", dict(T=0.8)), ("T+top_k", dict(T=0.8, k=50)),
             ("T+top_p", dict(T=0.8, p=0.9)), ("T+k+p", dict(T=0.8, k=50, p=0.9)))

    def one(n, blocks, T=0.0, k=None, p=None):
        ops.sample_force_blocks_per_row(blocks)
        logits = torch.randn(n, vocab, device=DEV) * 2
        out = torch.empty(n, dtype=torch.int32, device=DEV)
        full = lambda v, dt: torch.full((n,), v, dtype=dt, device=DEV)
        args = dict(temperature=full(T, torch.float32), seeds=full(1, torch.int64),
                    counters=torch.arange(n, dtype=torch.int64, device=DEV))
        if k is not None:
            args["top_k"] = full(k, torch.int32)
        if p is not None:
            args["top_p"] = full(p, torch.float32)
        return _graph_time(lambda i: ops.sample(logits, out, **args), 20)

    try:
        for n in (1, 8, 16, 64):
            for name, kw in kinds:
                cells = "  ".join(f"b{b}={one(n, b, **kw):6.1f}" for b in (1, 2, 4, 8))
                print(f"rows {n:3d} {name:12s}: {cells}  own choice={one(n, None, **kw):6.1f} us", flush=True)
    finally:
        ops.sample_force_blocks_per_row(None)


# ---- attention ------------------------------------------------------------------------------------
class _DecodeCase:
    """R decode rows over contexts of `ctx` tokens, the cache in as many copies as hold 500 MB."""

    def __init__(self, R, H, KV, d, ctx):
        pp = -(-ctx // 16)
        n_pages = R * pp
        n = max(2, min(32, int(500e6 // (n_pages * 2 * KV * 16 * d * 2)) + 1))
        self.caches = [torch.randn(n_pages, 2, KV, 16, d, device=DEV).bfloat16() for _ in range(n)]
        self.bt = torch.randperm(n_pages, device=DEV).to(torch.int32).view(R, pp).contiguous()
        self.q = torch.randn(R, H * d, device=DEV).bfloat16()
        self.out = torch.empty_like(self.q)
        self.req = torch.arange(R, dtype=torch.int32, device=DEV)
        self.pos = torch.full((R,), ctx - 1, dtype=torch.int32, device=DEV)
        self.H, self.ctx, self.scale = H, ctx, 1 / math.sqrt(d)
        self.bytes = R * ctx * 2 * KV * d * 2

    def time(self, **plan) -> float:
        n = len(self.caches)
        call = lambda i: ops.attention_decode(self.q, self.caches[i % n], self.bt, self.req, self.pos, self.out, self.H,
                                              self.scale, 0, max_kv_len=self.ctx, **plan)
        return _graph_time(call, 2 * n)


def attention_sizes() -> None:
    """Both prefill attention kernels (one 2,048-token prompt) and the decode kernel (contexts of 2,040)
    at head sizes and head counts beside the flagship's."""
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    print("prefill attention, one prompt of 2,048 tokens, causal FLOP counted once")
    for (H, KV, d) in ((32, 32, 64), (32, 32, 80), (32, 32, 96), (32, 32, 112), (32, 32, 128), (32, 8, 128), (16, 16, 256)):
        T = 2048
        cache = torch.randn(T // 16, 2, KV, 16, d, device=DEV).bfloat16()
        bt = torch.arange(T // 16, dtype=torch.int32, device=DEV).reshape(1, -1)
        q = torch.randn(T, H * d, device=DEV).bfloat16()
        out = torch.empty_like(q)
        tiles = list(range(0, T, ops.ATTN_PREFILL_TILE))
        a = (q, cache, bt, i32([0] * len(tiles)), i32(tiles), i32([0]), i32([T]), i32([0]), out, H, 1 / math.sqrt(d), 0)
        flops = 4 * H * d * T * T / 2

        def timed(f):
            for _ in range(3):
                f(*a)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                f(*a)
            e1.record()
            torch.cuda.synchronize()
            ops.raise_on_device_error()
            return e0.elapsed_time(e1) * 100
        t1 = timed(ops.attention_prefill)
        line = f"  heads {H} kv {KV} d {d}: mma.sync {t1:7.1f} us = {flops / t1 / 1e6:5.0f} TFLOP/s"
        if ops.attention_prefill_tc_supported(q, cache, out):
            t2 = timed(ops.attention_prefill_tc)
            line += f"   tcgen05 {t2:7.1f} us = {flops / t2 / 1e6:5.0f} TFLOP/s"
        print(line, flush=True)
    print("decode attention, contexts of 2,040")
    for (H, KV, d) in ((32, 32, 64), (32, 32, 80), (32, 32, 96), (32, 32, 128), (32, 8, 128), (16, 16, 256), (40, 40, 128),
                       (56, 56, 128), (12, 12, 64)):
        for R in (1, 8, 64):
            case = _DecodeCase(R, H, KV, d, 2040)
            us = case.time()
            print(f"  heads {H} kv {KV} d {d} rows {R:2d}: {us:7.1f} us, {case.bytes / 1e6:7.1f} MB, {case.bytes / us / 1e6:5.2f} TB/s",
                  flush=True)
            del case


def attention_plans(context: int = 2040, rows=(1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64), heads=(32, 40, 56)) -> None:
    """Every plan of the decode attention kernel (4, 8, 16 warps a block; 1 to 16 splits) against
    ops.decode_attention_plan's choice, 1 to 64 rows of 32, 40 and 56 heads of 128 dims (or the rows and heads given:
    --rows 32,64,128,256 --heads 32 --context 256 is the many-short-contexts case)."""
    ratios = []
    for H in heads:
        for R in rows:
            case = _DecodeCase(R, H, H, 128, context)
            own = case.time()
            plans = {}
            for w in (4, 8, 16):
                for S in (1, 2, 3, 4, 6, 8, 12, 16):
                    if (S == 1 or R * H * S <= 4096) and S * 8 <= -(-context // 16) * 2:
                        plans[f"w{w}s{S}"] = round(case.time(n_splits=S, warps=w), 1)
            best = sorted(plans.items(), key=lambda kv: kv[1])[:3]
            ratios.append(own / best[0][1])
            print(json.dumps(dict(heads=H, rows=R, pairs=R * H, MB=round(case.bytes / 1e6, 1), own_choice_us=round(own, 1),
                                  ratio_to_best=round(ratios[-1], 3), best=best)), flush=True)
            del case
    print(f"own choice / best plan: mean {statistics.mean(ratios):.3f}, worst {max(ratios):.3f}")


# ---- products -----------------------------------------------------------------------------------
GEMM_SHAPES = {
    "30b": [(21504, 7168, False), (7168, 7168, True), (28672, 7168, False), (7168, 28672, True)],
    "13b": [(15360, 5120, False), (5120, 5120, True), (20480, 5120, False), (5120, 20480, True)],
    "6.7b": [(12288, 4096, False), (4096, 4096, True), (16384, 4096, False), (4096, 16384, True)],
    "head": [(50272, 7168, False), (50272, 4096, False)],
}


def gemm_plans(models=("30b", "13b", "6.7b", "head")) -> None:
    """Every kernel that could run a product of 129 to 2,048 tokens against the estimates' own choice
    (gemm_tc.cu: plan_many_tokens), each call on a flushed cache."""
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)

    def timed(a, w, out, bias, res):
        ts = []
        for _ in range(7):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            ops.gemm_tc(a, w, out, bias=bias, residual=res)
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        return statistics.median(ts)

    ratios = []
    try:
        for name in models:
            for (N, K, with_res) in GEMM_SHAPES[name]:
                w = (torch.randn(N, K, device=DEV) * 0.02).bfloat16()
                bias = torch.randn(N, device=DEV)
                for M in (129, 160, 192, 255, 256, 320, 384, 512, 640, 768, 1024, 1280, 1536, 2048):
                    a = torch.randn(M, K, device=DEV).bfloat16()
                    res = torch.randn(M, N, device=DEV) if with_res else None
                    out = res if with_res else torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
                    ops.gemm_tc_force_plan(None)
                    ops.gemm_tc(a, w, out, bias=bias, residual=res)
                    times = {"own choice": timed(a, w, out, bias, res)}
                    for plan in ops.GEMM_PLANS:
                        ops.gemm_tc_force_plan(plan)
                        try:
                            ops.gemm_tc(a, w, out, bias=bias, residual=res)
                        except ops.KernelError:
                            continue                      # the sizes do not allow this plan
                        times[plan] = timed(a, w, out, bias, res)
                    ops.gemm_tc_force_plan(None)
                    ops.raise_on_device_error()
                    best = min((v, k) for k, v in times.items() if k != "own choice")
                    ratios.append(times["own choice"] / best[0])
                    print(json.dumps(dict(sizes=name, N=N, K=K, M=M, ratio_to_best=round(ratios[-1], 3), best=best[1],
                                          us={k: round(v, 1) for k, v in times.items()})), flush=True)
    finally:
        ops.gemm_tc_force_plan(None)
    print(f"own choice / best kernel: mean {statistics.mean(ratios):.3f}, worst {max(ratios):.3f}, "
          f"more than 10 % behind in {sum(r > 1.1 for r in ratios)} of {len(ratios)}")


FEW_TOKEN_SHAPES = {     # the four products of a layer: (N, K, adds into the 32-bit residual stream)
    name: [(3 * h, h, False), (h, h, True), (4 * h, h, False), (h, 4 * h, True)]
    for name, h in (("1.3b", 2048), ("2.7b", 2560), ("6.7b", 4096), ("13b", 5120), ("30b", 7168), ("66b", 9216))
}


def _rotating_product_time(M, N, K, with_res, dtype, **kw) -> float:
    """Microseconds of one product whose weights come from memory: 16 calls over as many copies of the
    matrix as exceed the second-level cache several times, replayed back to back from one CUDA graph."""
    copies = max(2, int(600e6 // (N * K * 2)) + 1)
    ws = [(torch.randn(N, K, device=DEV) * 0.02).to(dtype) for _ in range(copies)]
    a = torch.randn(M, K, device=DEV).to(dtype)
    bias = torch.randn(N, device=DEV)
    out = torch.zeros(M, N, device=DEV, dtype=torch.float32 if with_res else dtype)
    res = out if with_res else None
    return _graph_time(lambda i: ops.gemm_tc(a, ws[i % copies], out, bias=bias, residual=res, **kw), 16)


def gemm_tokens(models=("6.7b",), tokens=(1, 2, 4, 8, 16, 32, 64, 96, 128, 160, 192, 256, 384, 512), dtype=torch.float16) -> None:
    """A layer's products by the number of tokens: time and the rate at which the weights stream."""
    for name in models:
        for (N, K, with_res) in FEW_TOKEN_SHAPES[name]:
            row = {"sizes": name, "N": N, "K": K}
            for M in tokens:
                us = _rotating_product_time(M, N, K, with_res, dtype)
                row[f"M{M}"] = [round(us, 1), round(N * K * 2 / us / 1e6, 2)]          # us, TB/s of weights
            ops.raise_on_device_error()
            print(json.dumps(row), flush=True)


def gemm_splits(models=("1.3b", "2.7b", "6.7b", "13b", "30b", "66b"), tokens=8, dtype=torch.float16) -> None:
    """The few-token product with K split 1, 2, 4 and 8 ways in clusters beside the library's own choice
    (gemm_tc.cu: tnx_gemm_tc_plan), at the layer sizes of the family."""
    ratios = []
    for name in models:
        for (N, K, with_res) in FEW_TOKEN_SHAPES[name]:
            times = {"own choice": _rotating_product_time(tokens, N, K, with_res, dtype, few_tokens_kernel=False)}
            for sp in (1, 2, 4, 8):
                if sp * 4 <= -(-K // 64):
                    times[f"split_{sp}"] = _rotating_product_time(tokens, N, K, with_res, dtype, splits=sp, cluster=True)
            ops.raise_on_device_error()
            best = min((v, k) for k, v in times.items() if k != "own choice")
            ratios.append(times["own choice"] / best[0])
            print(json.dumps(dict(sizes=name, N=N, K=K, M=tokens, ratio_to_best=round(ratios[-1], 3), best=best[1],
                                  us={k: round(v, 1) for k, v in times.items()})), flush=True)
    print(f"own choice / best split: mean {statistics.mean(ratios):.3f}, worst {max(ratios):.3f}")


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="what", required=True)
    sub.add_parser("sampling").add_argument("--vocab", type=int, default=50272)
    sub.add_parser("attention-sizes")
    apl = sub.add_parser("attention-plans")
    apl.add_argument("--context", type=int, default=2040)
    apl.add_argument("--rows", default="1,2,3,4,6,8,12,16,24,32,48,64")
    apl.add_argument("--heads", default="32,40,56")
    sub.add_parser("gemm-plans").add_argument("--models", default="30b,13b,6.7b,head")
    gt = sub.add_parser("gemm-tokens")
    gt.add_argument("--models", default="6.7b")
    gt.add_argument("--tokens", default="1,2,4,8,16,32,64,96,128,160,192,256,384,512")
    gs = sub.add_parser("gemm-splits")
    gs.add_argument("--models", default="1.3b,2.7b,6.7b,13b,30b,66b")
    gs.add_argument("--tokens", type=int, default=8)
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("these timings need a GPU")
    if args.what == "sampling":
        sampling(args.vocab)
    elif args.what == "attention-sizes":
        attention_sizes()
    elif args.what == "attention-plans":
        attention_plans(args.context, tuple(int(r) for r in args.rows.split(",")), tuple(int(h) for h in args.heads.split(",")))
    elif args.what == "gemm-tokens":
        gemm_tokens(tuple(args.models.split(",")), tuple(int(t) for t in args.tokens.split(",")))
    elif args.what == "gemm-splits":
        gemm_splits(tuple(args.models.split(",")), args.tokens)
    else:
        gemm_plans(tuple(args.models.split(",")))


if __name__ == "__main__":
    main()
