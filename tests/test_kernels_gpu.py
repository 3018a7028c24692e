"""Each kernel alone against a plain 32-bit torch reference of the same operation, at other sizes
than the engine's tiny models use (widths and vocabularies that are no power of two, head sizes in
steps of 16, several key/value groups)."""
import math

import pytest
import torch

from plain import opt_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from transformers_neuronx_b200.kernels import ops as o
    return o


def rel_err(got, want):
    return float((got.float() - want.float()).abs().max()) / max(float(want.float().abs().max()), 1e-30)


# ---- matrix products ------------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K", [(1, 48, 40), (7, 130, 72), (64, 64, 16), (65, 257, 1000), (200, 96, 320)])
@pytest.mark.parametrize("combo", ["fff", "bbf", "bbb", "fbf", "bfb"])
def test_gemm_simt(M, N, K, combo):
    dt = {"f": torch.float32, "b": torch.bfloat16}
    g = torch.Generator(device="cpu").manual_seed(M * 1000 + N)
    a = torch.randn(M, K, generator=g).to(dt[combo[0]]).to(DEV)
    w = torch.randn(N, K, generator=g).to(dt[combo[1]]).to(DEV)
    bias = torch.randn(N, generator=g).to(DEV)
    out = torch.empty(M, N, dtype=dt[combo[2]], device=DEV)
    ops().gemm_simt(a, w, out, bias=bias, activation="relu")
    want = torch.relu(a.float() @ w.float().t() + bias)
    assert rel_err(out, want) <= (1e-5 if combo[2] == "f" else 5e-3)
    if combo[2] == "f":
        res = torch.randn(M, N, generator=g).to(DEV)
        want2 = a.float() @ w.float().t() + res
        ops().gemm_simt(a, w, res, residual=res)        # in place on the residual stream
        assert rel_err(res, want2) <= 1e-5


def test_gemm_simt_rows_do_not_depend_on_the_batch():
    a = torch.randn(70, 96, device=DEV)
    w = torch.randn(50, 96, device=DEV)
    full = torch.empty(70, 50, device=DEV)
    one = torch.empty(1, 50, device=DEV)
    ops().gemm_simt(a, w, full)
    ops().gemm_simt(a[33:34], w, one)
    assert torch.equal(full[33:34], one)                 # bit for bit


TC_SHAPES = [(1, 128, 64), (3, 96, 320), (8, 256, 2112), (40, 4096, 4096), (128, 4096, 4096), (96, 12288, 4096), (72, 1000, 328), (130, 4096, 16384), (100, 520, 8200),
             (250, 12288, 4096), (16, 4096, 1024), (17, 1000, 96), (33, 200, 136), (64, 512, 4096),
             (65, 384, 256), (128, 128, 64), (200, 1000, 328), (300, 520, 1032), (2048, 768, 512),
             (1024, 4096, 512), (1000, 4000, 328), (300, 9000, 136), (513, 7100, 72), (520, 7102, 72), (2100, 2300, 1096),
             (1280, 2048, 16384), (2000, 3300, 8200), (1100, 4090, 4096),     # the first and the third share tiles out by K blocks (long K; four runs a tile)
             (256, 4096, 4096), (384, 4096, 8192), (384, 12288, 4096), (300, 4000, 4104)]   # 128 x 256 tiles, K split 4, 2, 1, 2 ways in clusters


@pytest.mark.parametrize("M,N,K", TC_SHAPES)
def test_gemm_tc(M, N, K):
    o = ops()
    g = torch.Generator(device="cpu").manual_seed(M + N + K)
    a = (torch.randn(M, K, generator=g)).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16().to(DEV)
    bias = torch.randn(N, generator=g).to(DEV)
    want = a.float() @ w.float().t()
    tc = dict(few_tokens_kernel=False)                  # the tensor-core kernel also for one to four tokens
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    o.gemm_tc(a, w, out, **tc)
    o.raise_on_device_error()
    assert rel_err(out, want) <= 2e-5, "plain product"
    outb = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    o.gemm_tc(a, w, outb, bias=bias, activation="relu", **tc)
    assert rel_err(outb, torch.relu(want + bias)) <= 5e-3, "bias + relu -> bf16"
    res = torch.randn(M, N, generator=g).to(DEV)
    want3 = want + bias + res
    o.gemm_tc(a, w, res, bias=bias, residual=res, **tc)
    o.raise_on_device_error()
    assert rel_err(res, want3) <= 2e-5, "bias + residual in place"
    res2 = torch.randn(M, N, generator=g).to(DEV)
    keep = res2.clone()
    out4 = torch.full((M, N), 7.0, dtype=torch.float32, device=DEV)
    o.gemm_tc(a, w, out4, residual=res2)
    o.raise_on_device_error()
    assert rel_err(out4, want + keep) <= 2e-5 and torch.equal(res2, keep), "residual beside the output"


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (1, 4099, 4096), (2, 1000, 328), (2, 515, 16384), (3, 96, 320),
                                   (4, 12288, 4096), (4, 50, 8), (1, 7, 28672), (3, 300, 10920)])
def test_gemv_few_tokens(M, N, K):
    """The kernel for one to four tokens: the weights streamed through the multiply-add units."""
    o = ops()
    g = torch.Generator(device="cpu").manual_seed(M * 7 + N + K)
    a = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16().to(DEV)
    bias = torch.randn(N, generator=g).to(DEV)
    want = a.float() @ w.float().t()
    launches = o.launch_count()
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    o.gemv(a, w, out)
    assert rel_err(out, want) <= 2e-5, "plain product"
    outb = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    o.gemv(a, w, outb, bias=bias, activation="relu")
    assert rel_err(outb, torch.relu(want + bias)) <= 5e-3, "bias + relu -> bf16"
    res = torch.randn(M, N, generator=g).to(DEV)
    want3 = want + bias + res
    o.gemv(a, w, res, bias=bias, residual=res)
    assert rel_err(res, want3) <= 2e-5, "bias + residual in place"
    # a token's row is the same alone and beside others, bit for bit
    one = torch.empty(1, N, dtype=torch.float32, device=DEV)
    o.gemv(a[M - 1:M], w, one)
    assert torch.equal(one[0], out[M - 1])
    # rows of a wider buffer (the fused q/k/v output, a slice of the activations)
    wide = torch.zeros(M, N + 24, dtype=torch.float32, device=DEV)
    o.gemv(a, w, wide[:, 8:8 + N])
    assert torch.equal(wide[:, 8:8 + N], out) and float(wide[:, :8].abs().max()) == 0.0
    if M == 1:                                           # gemm_tc hands a single token to this kernel
        again = torch.empty_like(out)
        o.gemm_tc(a, w, again)
        assert torch.equal(again, out)


@pytest.mark.parametrize("M,N,K", [(1, 4099, 4096), (1, 520, 328), (2, 300, 10920), (1, 96, 16384), (4, 64, 640)])
@pytest.mark.parametrize("affine", [True, False])
def test_gemv_with_the_layer_norm_inside(M, N, K, affine):
    """The few-token product that normalizes its own input rows: the same numbers as the LayerNorm kernel
    followed by the product (the normalized rows rounded to bfloat16 in both), against 32-bit torch."""
    o = ops()
    g = torch.Generator(device="cpu").manual_seed(M + N + K)
    x = (torch.randn(M, K + 4, generator=g) * 3 + 0.5).to(DEV)[:, :K]           # a row pitch of its own
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16().to(DEV)
    gamma = (1 + 0.1 * torch.randn(K, generator=g)).to(DEV) if affine else None
    beta = (0.1 * torch.randn(K, generator=g)).to(DEV) if affine else None
    bias = torch.randn(N, generator=g).to(DEV)
    eps = 1e-5
    h = torch.nn.functional.layer_norm(x.float(), (K,), gamma, beta, eps)
    want = h.bfloat16().float() @ w.float().t() + bias
    assert o.gemv_layer_norm_supported(x[:1], w, torch.empty(1, N, dtype=torch.bfloat16, device=DEV))
    outb = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    o.gemv_layer_norm(x, gamma, beta, eps, w, outb, bias=bias, activation="relu")
    assert rel_err(outb, torch.relu(want)) <= 5e-3
    res0 = torch.randn(M, N, generator=g).to(DEV)
    res = res0.clone()
    o.gemv_layer_norm(x, gamma, beta, eps, w, res, bias=bias, residual=res)
    # the two-kernel way, with the engine's own LayerNorm kernel
    hk = torch.empty(M, K, dtype=torch.bfloat16, device=DEV)
    o.layer_norm(x.contiguous(), gamma, beta, eps, out_act=hk)
    two = res0.clone()
    o.gemv(hk, w, two, bias=bias, residual=two)
    assert rel_err(res, want + res0) <= 3e-3          # a normalized value next to a rounding boundary may round the other way
    assert rel_err(res, two) <= 3e-3


@pytest.mark.parametrize("M,N,K,splits", [(8, 256, 4096, 4), (64, 130, 1024, 16), (1, 128, 512, 2), (20, 300, 1160, 3),
                                          (100, 300, 2048, 4), (128, 256, 4096, 16)])
def test_gemm_tc_split_k(M, N, K, splits):
    o = ops()
    g = torch.Generator(device="cpu").manual_seed(splits)
    a = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16().to(DEV)
    bias = torch.randn(N, generator=g).to(DEV)
    want = torch.relu(a.float() @ w.float().t() + bias)
    out1 = torch.empty(M, N, dtype=torch.float32, device=DEV)
    out2 = torch.empty_like(out1)
    o.gemm_tc(a, w, out1, bias=bias, activation="relu", splits=splits)
    o.gemm_tc(a, w, out2, bias=bias, activation="relu", splits=splits)      # the counters were left at zero
    o.raise_on_device_error()
    assert rel_err(out1, want) <= 2e-5
    assert torch.equal(out1, out2), "the order of the additions is fixed"


@pytest.mark.parametrize("M,N,K,splits", [(8, 256, 4096, 4), (64, 130, 1024, 8), (2, 128, 512, 2), (20, 300, 1160, 3),
                                          (16, 4096, 4096, 8), (33, 520, 2048, 5), (64, 1000, 4104, 7), (5, 96, 640, 8),
                                          (100, 520, 2048, 4), (128, 4096, 4096, 2), (70, 130, 1160, 3), (97, 1000, 8200, 8),
                                          (24, 512, 2048, 4), (48, 1024, 4096, 8), (64, 256, 1024, 2), (120, 384, 512, 2)])
def test_gemm_tc_split_k_in_clusters(M, N, K, splits):
    """K split over the CTAs of a cluster, partial tiles added through distributed shared memory: the bands sent
    to their owners by bulk copies (2, 4 or 8 splits, aligned output, tile and bands fit the stages: every tile
    width is among the cases), fetched by the owners with 16-byte loads (128 tokens with 4 or 8 splits) or one by
    one (other splits, or an output whose rows are not 16-byte aligned)."""
    o = ops()
    g = torch.Generator(device="cpu").manual_seed(splits + M)
    a = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16().to(DEV)
    bias = torch.randn(N, generator=g).to(DEV)
    want = a.float() @ w.float().t()
    out1 = torch.empty(M, N, dtype=torch.float32, device=DEV)
    out2 = torch.empty_like(out1)
    o.gemm_tc(a, w, out1, bias=bias, activation="relu", splits=splits, cluster=True)
    o.gemm_tc(a, w, out2, bias=bias, activation="relu", splits=splits, cluster=True)
    o.raise_on_device_error()
    assert rel_err(out1, torch.relu(want + bias)) <= 2e-5
    assert torch.equal(out1, out2), "the order of the additions is fixed"
    res = torch.randn(M, N, generator=g).to(DEV)
    want3 = want + bias + res
    o.gemm_tc(a, w, res, bias=bias, residual=res, splits=splits, cluster=True)
    assert rel_err(res, want3) <= 2e-5, "bias + residual in place"
    outb = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    o.gemm_tc(a, w, outb, splits=splits, cluster=True)
    o.raise_on_device_error()
    assert rel_err(outb, want) <= 5e-3
    # the same sums as with scratch memory: both add the partial tiles in split order
    out3 = torch.empty_like(out1)
    o.gemm_tc(a, w, out3, bias=bias, activation="relu", splits=splits)
    assert torch.equal(out1, out3)


@pytest.mark.parametrize("M,N,K", [(300, 1000, 7168), (129, 520, 1160), (640, 2100, 4104), (257, 9000, 512)])
def test_gemm_tc_every_many_token_kernel(M, N, K):
    """Each kernel that the plan for more than 128 tokens can choose, imposed in turn on sizes that fill
    no tile: the same product, bias, activation and residual from all of them."""
    o = ops()
    g = torch.Generator(device="cpu").manual_seed(M + N)
    a = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16().to(DEV)
    bias = torch.randn(N, generator=g).to(DEV)
    res0 = torch.randn(M, N, generator=g).to(DEV)
    want = a.float() @ w.float().t() + bias
    ran = []
    try:
        for plan in o.GEMM_PLANS:
            o.gemm_tc_force_plan(plan)
            out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
            try:
                o.gemm_tc(a, w, out, bias=bias, activation="relu")
            except o.KernelError:
                continue                                    # the sizes do not allow this plan
            res = res0.clone()
            o.gemm_tc(a, w, res, bias=bias, residual=res)
            o.raise_on_device_error()
            assert rel_err(out, torch.relu(want)) <= 5e-3, plan
            assert rel_err(res, want + res0) <= 2e-5, plan
            ran.append(plan)
    finally:
        o.gemm_tc_force_plan(None)
    assert {"tiles_128", "pairs", "persistent"} <= set(ran), ran


def test_gemm_tc_plan_is_near_the_best_kernel():
    """The estimates that choose a kernel for more than 128 tokens were fitted on some layer sizes; here
    they are held against the fastest of all kernels at others (the 30B model's K of 7,168 and 28,672,
    a vocabulary-sized N), every call on cold caches."""
    o = ops()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)

    def timed(a, w, out, reps=5):
        ts = []
        for _ in range(reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            o.gemm_tc(a, w, out)
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return sorted(ts)[len(ts) // 2]

    def measure(a, w, out):
        o.gemm_tc_force_plan(None)
        o.gemm_tc(a, w, out)
        chosen = timed(a, w, out)
        best = {}
        for plan in o.GEMM_PLANS:
            o.gemm_tc_force_plan(plan)
            try:
                o.gemm_tc(a, w, out)
            except o.KernelError:
                continue
            best[plan] = timed(a, w, out)
        o.raise_on_device_error()
        name = min(best, key=best.get)
        return chosen / best[name], name

    worst = []
    try:
        for (M, N, K) in [(384, 21504, 7168), (512, 21504, 7168), (1024, 7168, 7168), (192, 28672, 7168),
                          (640, 28672, 7168), (256, 7168, 28672), (1280, 7168, 28672), (384, 50272, 4096)]:
            a = torch.randn(M, K, device=DEV).bfloat16()
            w = (torch.randn(N, K, device=DEV) * 0.02).bfloat16()
            out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
            ratio, name = measure(a, w, out)
            for _ in range(2):                      # a time is a sample (clocks ramp, a neighbour's job): what is asserted is
                if ratio <= 1.2:                    # the choice, so a shape that looks bad is measured again before it counts
                    break
                ratio, name = min((ratio, name), measure(a, w, out))
            worst.append((ratio, (M, N, K), name))
    finally:
        o.gemm_tc_force_plan(None)
    ratio, shape, name = max(worst)
    assert ratio <= 1.2, f"{shape}: the chosen kernel takes {ratio:.2f} times as long as {name}"


def test_gemm_tc_finds_a_planted_column():
    """One large entry far along K and in the last rows of the last tile: a kernel that drops the
    tail of K, a tile edge or a swizzled chunk misses it."""
    o = ops()
    M, N, K = 130, 260, 1096
    a = torch.zeros(M, K, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(N, K, dtype=torch.bfloat16, device=DEV)
    a[129, 1095] = 3.0
    w[259, 1095] = 5.0
    a[5, 77] = 2.0
    w[131, 77] = -4.0
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    o.gemm_tc(a, w, out)
    want = torch.zeros(M, N, device=DEV)
    want[129, 259] = 15.0
    want[5, 131] = -8.0
    assert torch.equal(out, want)


def test_gemm_tc_refuses_unaligned_sizes():
    o = ops()
    a = torch.zeros(4, 12, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(8, 12, dtype=torch.bfloat16, device=DEV)
    out = torch.empty(4, 8, dtype=torch.float32, device=DEV)
    assert not o.gemm_tc_supported(a, w, out)
    with pytest.raises(o.KernelError, match="multiples of 8"):
        o.gemm_tc(a, w, out)


# ---- attention over the paged cache ----------------------------------------------------------------
def plain_attention(q, k, v, n_heads, n_kv, scale, first_pos, window):
    """q [Tq, n_heads, d] at positions first_pos.., k/v [Tk, n_kv, d] -> [Tq, n_heads, d], by the
    plain implementation's own functions."""
    rep = n_heads // n_kv
    qh = q.float().transpose(0, 1)
    kh = k.float().transpose(0, 1).repeat_interleave(rep, dim=0)
    vh = v.float().transpose(0, 1).repeat_interleave(rep, dim=0)
    s = P.attention_scores(qh, kh, q.shape[-1], scale)
    mask = P.causal_mask(q.shape[0], k.shape[0], first_pos, window)
    return P.attention_context(P.masked_softmax(s, mask[None]), vh).transpose(0, 1)


class PagedCase:
    """Requests with contexts and portions; keys/values scattered over shuffled pages."""

    def __init__(self, lens, n_heads, n_kv, d, dtype, seed=0, plant=True, poison=float("nan")):
        # lens: list of (ctx_len, q_len)
        g = torch.Generator().manual_seed(seed)
        self.lens, self.n_heads, self.n_kv, self.d, self.dtype = lens, n_heads, n_kv, d, dtype
        ps = 16
        total_pages = sum(-(-(c + q) // ps) for c, q in lens) + 3
        perm = torch.randperm(total_pages, generator=g).tolist()
        self.cache = torch.full((total_pages, 2, n_kv, ps, d), poison, dtype=dtype)   # unwritten rows are poison
        self.k, self.v, self.q = [], [], []
        tables, tok_req, positions, q_start, tile_req, tile_q0, decode_rows = [], [], [], [], [], [], []
        row = 0
        for r, (c, ql) in enumerate(lens):
            T = c + ql
            k = torch.randn(T, n_kv, d, generator=g)
            v = torch.randn(T, n_kv, d, generator=g)
            q = torch.randn(ql, n_heads, d, generator=g)
            if plant and T > 20:
                # one far key (at a page's edge) that every head of the last query must find
                far = 15 if T > 40 else 0
                k[far] *= 0.1
                q[-1] = k[far].repeat_interleave(n_heads // n_kv, dim=0) * 60.0
                v[far] += 5.0
            k, v, q = k.to(dtype), v.to(dtype), q.to(dtype)
            pages = [perm.pop() for _ in range(-(-T // ps))]
            for t in range(T):
                self.cache[pages[t // ps], 0, :, t % ps] = k[t]
                self.cache[pages[t // ps], 1, :, t % ps] = v[t]
            tables.append(pages)
            self.k.append(k); self.v.append(v); self.q.append(q)
            q_start.append(row)
            tok_req += [r] * ql
            positions += list(range(c, c + ql))
            if ql == 1:
                decode_rows.append(row)
            else:
                for q0 in range(0, ql, ops().ATTN_PREFILL_TILE):
                    tile_req.append(r); tile_q0.append(q0)
            row += ql
        mb = max(len(t) for t in tables)
        bt = torch.full((len(lens), mb), -1, dtype=torch.int32)
        for r, t in enumerate(tables):
            bt[r, :len(t)] = torch.tensor(t, dtype=torch.int32)
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
        self.bt = bt.to(DEV)
        self.tok_req, self.positions = i32(tok_req), i32(positions)
        self.q_start, self.q_len, self.ctx_len = i32(q_start), i32([q for _, q in lens]), i32([c for c, _ in lens])
        self.tile_req, self.tile_q0, self.decode_rows = i32(tile_req), i32(tile_q0), i32(decode_rows)
        self.q_flat = torch.cat([q.reshape(q.shape[0], -1) for q in self.q]).to(DEV)
        self.cache = self.cache.to(DEV)
        self.N = row

    def release_behind(self, window):
        """What the cache manager does behind a sliding window: pages that no query of a request can
        read any more (all their keys lie before the first query's window) leave the block table
        (-1) and their contents are gone (poisoned here, as if another request had taken them)."""
        bt = self.bt.cpu().clone()
        gone = []
        for r, (c, ql) in enumerate(self.lens):
            first_needed = max(0, c - window + 1) // 16            # the first query sits at position c
            for b in range(first_needed):
                gone.append(int(bt[r, b])); bt[r, b] = -1
        if gone:
            self.cache[torch.tensor(gone, device=self.cache.device)] = float("nan") if self.dtype != torch.float32 else 7e4
        self.bt = bt.to(self.bt.device)
        return len(gone)

    def want(self, scale, window):
        outs = []
        for (c, ql), q, k, v in zip(self.lens, self.q, self.k, self.v):
            outs.append(plain_attention(q, k, v, self.n_heads, self.n_kv, scale, c, window).reshape(ql, -1))
        return torch.cat(outs).to(DEV)


ATT_SHAPES = [(4, 4, 16), (3, 3, 32), (6, 2, 48), (8, 8, 64), (5, 1, 80), (4, 4, 96), (3, 3, 112), (4, 2, 128), (2, 1, 160),
              (2, 2, 192), (2, 2, 256)]


@pytest.mark.parametrize("n_heads,n_kv,d", ATT_SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 37])
def test_attention_simt(n_heads, n_kv, d, dtype, window):
    case = PagedCase([(0, 5), (17, 1), (40, 33), (100, 1), (3, 70)], n_heads, n_kv, d, dtype, seed=d)
    scale = 1.0 / math.sqrt(d)
    out = torch.zeros(case.N, n_heads * d, dtype=dtype, device=DEV)
    ops().attention_simt(case.q_flat, case.cache, case.bt, case.tok_req, case.positions, out, n_heads, scale, window or 0)
    assert rel_err(out, case.want(scale, window)) <= (1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("n_heads,n_kv,d", ATT_SHAPES)
@pytest.mark.parametrize("window", [None, 50])
@pytest.mark.parametrize("n_splits,warps", [(None, None), (1, 4), (3, 4), (7, 4), (1, 8), (2, 8), (5, 8), (1, 16), (3, 16), (20, 8), (44, 4)])
def test_attention_decode(n_heads, n_kv, d, window, n_splits, warps):
    lens = [(0, 1), (15, 1), (16, 1), (17, 1), (255, 1), (256, 1), (700, 1), (63, 1)]
    case = PagedCase(lens, n_heads, n_kv, d, torch.bfloat16, seed=d + 1)
    scale = 0.7 / math.sqrt(d)
    out = torch.zeros(case.N, n_heads * d, dtype=torch.bfloat16, device=DEV)
    o = ops()
    if warps == 16 and d > 128:
        pytest.skip("sixteen warps a block are for heads of up to 128 dims")
    for _ in range(2):          # twice: the split counters must be back at zero
        out.zero_()
        o.attention_decode(case.q_flat, case.cache, case.bt, case.tok_req, case.positions, out, n_heads, scale,
                           window or 0, max_kv_len=701, n_splits=n_splits, warps=warps)
        assert rel_err(out, case.want(scale, window)) <= 1e-2


@pytest.mark.parametrize("n_heads,n_kv,d", [(4, 4, 128), (6, 2, 64), (3, 1, 80), (2, 2, 256), (2, 2, 48), (4, 2, 96), (2, 1, 160),
                                            (2, 2, 192), (3, 3, 112)])
@pytest.mark.parametrize("n_splits,warps", [(1, 4), (3, 4), (1, 8), (3, 8), (None, None)])
def test_attention_decode_appends_the_new_token(n_heads, n_kv, d, n_splits, warps):
    """The decode kernel writes the token's own key and value into its page and reads them back: the
    result and the cache must be those of an append followed by attention."""
    lens = [(0, 1), (15, 1), (16, 1), (17, 1), (255, 1), (256, 1), (700, 1), (63, 1)]
    case = PagedCase(lens, n_heads, n_kv, d, torch.bfloat16, seed=d + 3)
    scale = 0.9 / math.sqrt(d)
    full = case.cache.clone()
    k_new = torch.zeros(case.N, n_kv * d + 8, dtype=torch.bfloat16, device=DEV)[:, :n_kv * d]     # a row pitch of its own
    v_new = torch.zeros(case.N, n_kv * d + 8, dtype=torch.bfloat16, device=DEV)[:, :n_kv * d]
    pages = case.bt.cpu()
    for r, (c, _) in enumerate(lens):                       # take the last token out of the cache again
        pg, slot = int(pages[r, c // 16]), c % 16
        k_new[r] = full[pg, 0, :, slot].reshape(-1)
        v_new[r] = full[pg, 1, :, slot].reshape(-1)
        case.cache[pg, :, :, slot] = float("nan")
    out = torch.zeros(case.N, n_heads * d, dtype=torch.bfloat16, device=DEV)
    ops().attention_decode(case.q_flat, case.cache, case.bt, case.tok_req, case.positions, out, n_heads, scale,
                           0, max_kv_len=701, n_splits=n_splits, warps=warps, new_kv=(k_new, v_new))
    assert rel_err(out, case.want(scale, None)) <= 1e-2
    written = ~torch.isnan(full.float())
    assert torch.equal(case.cache[written], full[written]), "the cache holds the appended keys and values"
    assert bool(torch.isnan(case.cache.float()[~written]).all()), "nothing else was written"


def test_attention_decode_row_list():
    """Only the rows named are computed (a mixed batch: the others belong to the prefill kernel)."""
    lens = [(5, 1), (0, 40), (99, 1), (10, 3), (33, 1)]
    case = PagedCase(lens, 4, 4, 64, torch.bfloat16, seed=9)
    scale = 1.0 / 8
    out = torch.zeros(case.N, 4 * 64, dtype=torch.bfloat16, device=DEV)
    ops().attention_decode(case.q_flat, case.cache, case.bt, case.tok_req, case.positions, out, 4, scale, 0,
                           rows=case.decode_rows, max_kv_len=100)
    want = case.want(scale, None)
    rows = case.decode_rows.long()
    assert rel_err(out[rows], want[rows]) <= 1e-2
    others = torch.ones(case.N, dtype=torch.bool, device=DEV)
    others[rows] = False
    assert float(out[others].float().abs().max()) == 0.0


@pytest.mark.parametrize("n_heads,n_kv,d", ATT_SHAPES)
@pytest.mark.parametrize("window", [None, 45])
def test_attention_prefill(n_heads, n_kv, d, window):
    lens = [(0, 2), (0, 64), (0, 65), (30, 7), (64, 130), (15, 17), (200, 300), (5, 1)]
    case = PagedCase(lens, n_heads, n_kv, d, torch.bfloat16, seed=d + 2)
    scale = 1.0 / math.sqrt(d)
    out = torch.zeros(case.N, n_heads * d, dtype=torch.bfloat16, device=DEV)
    ops().attention_prefill(case.q_flat, case.cache, case.bt, case.tile_req, case.tile_q0, case.q_start, case.q_len,
                            case.ctx_len, out, n_heads, scale, window or 0)
    want = case.want(scale, window)
    keep = torch.ones(case.N, dtype=torch.bool, device=DEV)
    keep[case.decode_rows.long()] = False          # the single-row request is not in the tile list
    assert rel_err(out[keep], want[keep]) <= 1.5e-2
    assert float(out[~keep].float().abs().max()) == 0.0


# ---- norms, embedding, cache append, sampling -----------------------------------------------------------
@pytest.mark.parametrize("rows,H", [(1, 16), (5, 96), (33, 1000), (4, 4096), (2, 12288)])
@pytest.mark.parametrize("affine", [True, False])
def test_layer_norm(rows, H, affine):
    g = torch.Generator().manual_seed(H)
    x = (torch.randn(rows, H, generator=g) * 3 + 1.5).to(DEV)
    w = torch.randn(H, generator=g).to(DEV) if affine else None
    b = torch.randn(H, generator=g).to(DEV) if affine else None
    for eps in (1e-5, 1e-2):
        want = P.layer_norm(x.cpu(), None if w is None else w.cpu(), None if b is None else b.cpu(), eps).to(DEV)
        o32 = torch.empty(rows, H, device=DEV)
        ob = torch.empty(rows, H, dtype=torch.bfloat16, device=DEV)
        ops().layer_norm(x, w, b, eps, out_f32=o32, out_act=ob)
        assert rel_err(o32, want) <= 1e-5
        assert rel_err(ob, want) <= 5e-3
    picks = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    o = torch.empty(2, H, device=DEV)
    ops().layer_norm(x, w, b, 1e-5, out_act=o, rows=picks)
    want = P.layer_norm(x.cpu()[[rows - 1, 0]], None if w is None else w.cpu(), None if b is None else b.cpu(), 1e-5)
    assert rel_err(o, want.to(DEV)) <= 1e-5
    xin = x.clone()
    ops().layer_norm(xin, w, b, 1e-5, out_f32=xin)              # in place, as a post-norm block uses it
    assert rel_err(xin, P.layer_norm(x.cpu(), None if w is None else w.cpu(), None if b is None else b.cpu(), 1e-5).to(DEV)) <= 1e-5


@pytest.mark.parametrize("H", [768, 4096, 5120])
def test_layer_norm_of_few_rows_and_of_many_is_the_same(H):
    """Up to 256 rows the kernel fetches the scale and the shift before it waits for the kernel ahead of it, beyond
    it reads them where it uses them: a row's result is the same bits either way (a decode row and a row of a
    prompt portion), also when the kernel ahead of it is one of the engine's own that lets it in early."""
    o = ops()
    g = torch.Generator().manual_seed(H)
    x = (torch.randn(600, H, generator=g) * 2 + 0.5).to(DEV)
    w, b = torch.randn(H, generator=g).to(DEV), torch.randn(H, generator=g).to(DEV)
    many = torch.empty(600, H, dtype=torch.bfloat16, device=DEV)
    o.layer_norm(x, w, b, 1e-5, out_act=many)
    for rows in (1, 8, 64, 256):
        few = torch.empty(rows, H, dtype=torch.bfloat16, device=DEV)
        o.layer_norm(x[:rows], w, b, 1e-5, out_act=few)
        assert torch.equal(few, many[:rows])
    # behind a product of the engine (which lets the next kernel start early) that writes the rows it normalises
    a = torch.randn(8, 256, generator=g).bfloat16().to(DEV)
    wt = (torch.randn(H, 256, generator=g) / 16).bfloat16().to(DEV)
    y = torch.zeros(8, H, device=DEV)
    outs = []
    for _ in range(3):
        y.zero_()
        o.gemm_tc(a, wt, y)
        z = torch.empty(8, H, dtype=torch.bfloat16, device=DEV)
        o.layer_norm(y, w, b, 1e-5, out_act=z)
        outs.append(z)
    o.raise_on_device_error()
    want = P.layer_norm((a.float() @ wt.float().t()).cpu(), w.cpu(), b.cpu(), 1e-5).to(DEV)
    assert rel_err(outs[0], want) <= 5e-3
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])


@pytest.mark.parametrize("tdt", [torch.float32, torch.bfloat16])
def test_embedding(tdt):
    V, H, Pn, off = 301, 72, 50, 2
    g = torch.Generator().manual_seed(1)
    tok = torch.randn(V, H, generator=g).to(tdt)
    pos = torch.randn(Pn + off, H, generator=g).to(tdt)
    ids = torch.tensor([0, 300, 17, 5, 5], dtype=torch.int32)
    ps = torch.tensor([0, 49, 3, 20, 21], dtype=torch.int32)
    want = P.token_embedding(ids, tok.float()) + P.learned_position_embedding(ps, pos.float(), off)
    x = torch.empty(5, H, device=DEV)
    xa = torch.empty(5, H, dtype=torch.bfloat16, device=DEV)
    ops().embed(tok.to(DEV), None, ids.to(DEV), pos.to(DEV), ps.to(DEV), off, x, xa)
    assert rel_err(x, want.to(DEV)) <= 1e-6 and rel_err(xa, want.to(DEV)) <= 5e-3
    pre = torch.randn(5, H, generator=g)
    ops().embed(None, pre.to(DEV), ids.to(DEV), pos.to(DEV), ps.to(DEV), off, x, None)
    assert rel_err(x, (pre + P.learned_position_embedding(ps, pos.float(), off)).to(DEV)) <= 1e-6
    e = torch.empty(5, H, dtype=torch.bfloat16, device=DEV)
    ops().gather_rows(tok.to(DEV), ids.to(DEV), e)
    assert rel_err(e, tok.float()[ids.long()].to(DEV)) <= 5e-3


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_kv_append(dt):
    n_kv, d, ps, pages = 3, 48, 16, 7
    N = 20
    g = torch.Generator().manual_seed(2)
    qkv = torch.randn(N, (5 + 2 * n_kv) * d, generator=g).to(dt).to(DEV)
    k, v = qkv[:, 5 * d:(5 + n_kv) * d], qkv[:, (5 + n_kv) * d:]
    slots = torch.randperm(pages * ps, generator=g)[:N].to(torch.int32)
    cache = torch.zeros(pages, 2, n_kv, ps, d, dtype=dt, device=DEV)
    ops().kv_append(k, v, slots.to(DEV), cache, ps)
    for n in range(N):
        pg, r = int(slots[n]) // ps, int(slots[n]) % ps
        assert torch.equal(cache[pg, 0, :, r].reshape(-1), k[n]) and torch.equal(cache[pg, 1, :, r].reshape(-1), v[n])
    assert int((cache != 0).sum()) <= 2 * N * n_kv * d


@pytest.mark.parametrize("shape,dtype", [((9, 2, 3, 16, 48), torch.bfloat16), ((7, 33), torch.float32), ((5, 2, 2, 16, 128), torch.float16),
                                         ((6, 1000003), torch.uint8)])
def test_copy_rows(shape, dtype):
    """Rows copied within a tensor (pages of a cache, slots of a state tensor): sources and destinations
    disjoint, pairs with a -1 or with equal ends skipped, everything else untouched."""
    g = torch.Generator().manual_seed(len(shape))
    t = (torch.randn(*shape, generator=g) * 50).to(dtype).to(DEV) if dtype != torch.uint8 else \
        torch.randint(0, 255, shape, dtype=torch.uint8, generator=g).to(DEV)
    before = t.clone()
    pairs = torch.tensor([[0, 3], [1, 4], [1, 2], [-1, 0], [0, -1]], dtype=torch.int32, device=DEV)
    ops().copy_rows(t, pairs)
    want = before.clone()
    for s, d in ((0, 3), (1, 4), (1, 2)):
        want[d] = before[s]
    assert torch.equal(t, want)
    with pytest.raises(ops().KernelError):
        ops().copy_rows(t.transpose(0, 1) if t.dim() > 1 else t[::2], pairs)


def test_sampling_greedy_and_ties():
    logits = torch.randn(9, 50272, generator=torch.Generator().manual_seed(3)).to(DEV)
    logits[2, 777] = logits[2, 40000] = 99.0                  # a tie: the lowest index wins
    out = torch.empty(9, dtype=torch.int32, device=DEV)
    ops().sample(logits, out)
    want = P.greedy_token(logits.cpu())
    assert out.cpu().tolist() == want.tolist() and int(out[2]) == 777
    t0 = torch.zeros(9, device=DEV)
    ops().sample(logits, out, temperature=t0, suppress_id=777)
    assert int(out[2]) == 40000


def _draws(logits_row, n, temperature, top_k=0, top_p=1.0, suppress=-1, seed=5):
    V = logits_row.numel()
    logits = logits_row.to(DEV)[None].repeat(n, 1).contiguous()
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    ops().sample(logits, out, temperature=torch.full((n,), temperature, device=DEV),
                 top_k=torch.full((n,), top_k, dtype=torch.int32, device=DEV),
                 top_p=torch.full((n,), top_p, device=DEV),
                 seeds=torch.full((n,), seed, dtype=torch.int64, device=DEV),
                 counters=torch.arange(n, dtype=torch.int64, device=DEV), suppress_id=suppress)
    return out.cpu()


@pytest.mark.parametrize("kw", [dict(temperature=1.0), dict(temperature=0.7, top_k=5), dict(temperature=1.3, top_p=0.8),
                                dict(temperature=0.9, top_k=12, top_p=0.6), dict(temperature=1.0, suppress=3)])
def test_sampling_distribution(kw):
    V, n = 37, 40000
    row = torch.randn(V, generator=torch.Generator().manual_seed(11)) * 2
    got = _draws(row, n, **kw)
    sup = [kw["suppress"]] if kw.get("suppress", -1) >= 0 else None
    p = P.sampling_distribution(row[None], kw["temperature"], kw.get("top_k") or None, kw.get("top_p", 1.0), sup)[0]
    counts = torch.bincount(got.long(), minlength=V).float()
    assert int(counts[p == 0].sum()) == 0, "a token outside the kept set was drawn"
    keep = p > 0
    chi2 = float((((counts - n * p) ** 2)[keep] / (n * p[keep])).sum())
    dof = int(keep.sum()) - 1
    assert chi2 < dof + 6 * math.sqrt(2 * max(dof, 1)) + 10, f"chi2 {chi2:.1f} for {dof} degrees of freedom"
    again = _draws(row, n, **kw)
    assert torch.equal(got, again), "a draw is a function of logits, parameters, seed and counter"
    other = _draws(row, n, seed=6, **kw)
    assert int(keep.sum()) == 1 or not torch.equal(got, other)


@pytest.mark.parametrize("V", [37, 1000, 50272])
def test_sampling_with_a_fixed_uniform_number_matches_the_reference_choice(V):
    """deterministic: the kernel takes the kept tokens from the most likely down and chooses the one
    at which the summed probability reaches one half, which the plain on-device choice of the
    reference gives exactly (rows where one half lies within 2e-6 of a summed probability aside: the
    kernel's exponentials are 32-bit)."""
    g = torch.Generator().manual_seed(V)
    cases = [(None, 1.0, 1, 1.0), (5, 1.0, 1, 0.7), (50, 0.9, 1, 1.3), (None, 0.6, 1, 2.0), (20, 0.3, 4, 3.0),
             (3, 0.5, 8, 5.0), (None, 0.05, 6, 4.0), (1, 1.0, 1, 1.0)]
    n = 12 * len(cases)
    logits = torch.randn(n, V, generator=g) * 2.5
    ks, ps, ms, ts = [], [], [], []
    for i in range(n):
        k, p, m, t = cases[i % len(cases)]
        ks.append(k or 0); ps.append(p); ms.append(m); ts.append(t)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    ops().sample(logits.to(DEV), out, temperature=torch.tensor(ts, device=DEV), top_k=torch.tensor(ks, dtype=torch.int32, device=DEV),
                 top_p=torch.tensor(ps, device=DEV), min_keep=torch.tensor(ms, dtype=torch.int32, device=DEV), deterministic=True)
    got = out.cpu().tolist()
    checked = 0
    for i in range(n):
        want, margin = P.sample_on_device(logits[i], ks[i] or None, ps[i], ms[i], ts[i])
        if margin > 2e-6:
            assert got[i] == want, f"row {i} (top_k {ks[i]}, top_p {ps[i]}, at least {ms[i]}, temperature {ts[i]})"
            checked += 1
    assert checked > n * 0.8
    # without a top_p array the same kernel variant runs (it needs the mass histogram)
    out2 = torch.empty(n, dtype=torch.int32, device=DEV)
    ops().sample(logits.to(DEV), out2, temperature=torch.tensor(ts, device=DEV), deterministic=True)
    for i in range(0, n, 7):
        want, margin = P.sample_on_device(logits[i], None, 1.0, 1, ts[i])
        assert margin <= 2e-6 or int(out2[i]) == want


@pytest.mark.parametrize("V", [5, 37, 4099, 50272])
def test_sampling_does_not_depend_on_the_blocks_a_row(V):
    """A row is shared out over 1, 2, 4 or 8 thread blocks of a cluster (few rows: more blocks each); all
    sums are integers and added up across the cluster, so every way draws the same tokens: greedy with a
    tie across slices, temperature, top-k, top-p with a least number of tokens, the fixed draw, suppressed ids."""
    o = ops()
    g = torch.Generator().manual_seed(V)
    n = 24
    logits = (torch.randn(n, V, generator=g) * 2.5)
    logits[1, 0] = logits[1, V - 1] = 50.0                    # a tie between the first block's slice and the last's
    logits[2] = float("-inf")                                 # nothing to draw from: token 0
    temps = [0.0, 0.0, 1.0, 1.0, 0.7, 1.3, 0.9, 2.0] * 3
    ks = [0, 0, 0, 0, 5, 0, 12, 3] * 3
    ps = [1.0, 1.0, 1.0, 1.0, 1.0, 0.8, 0.6, 0.3] * 3
    ms = [1, 1, 1, 1, 1, 1, 2, 4] * 3
    dev = logits.to(DEV)
    results = {}
    try:
        for blocks in (1, 2, 4, 8):
            o.sample_force_blocks_per_row(blocks)
            for det in (False, True):
                out = torch.full((n,), -7, dtype=torch.int32, device=DEV)
                o.sample(dev, out, temperature=torch.tensor(temps, device=DEV), top_k=torch.tensor(ks, dtype=torch.int32, device=DEV),
                         top_p=torch.tensor(ps, device=DEV), min_keep=torch.tensor(ms, dtype=torch.int32, device=DEV),
                         seeds=torch.arange(n, dtype=torch.int64, device=DEV) + 3,
                         counters=torch.arange(n, dtype=torch.int64, device=DEV) * 5, deterministic=det, suppress_id=min(3, V - 1))
                results[(blocks, det)] = out.cpu().tolist()
            out = torch.full((n,), -7, dtype=torch.int32, device=DEV)
            o.sample(dev, out, temperature=torch.tensor(temps, device=DEV))          # the variant without top-p
            results[(blocks, "plain")] = out.cpu().tolist()
    finally:
        o.sample_force_blocks_per_row(None)
    for kind in (False, True, "plain"):
        for blocks in (2, 4, 8):
            assert results[(blocks, kind)] == results[(1, kind)], (blocks, kind)
        assert all(0 <= t < V for t in results[(1, kind)])
    assert results[(1, False)][1] == 0 and results[(1, False)][2] == 0


def test_sampling_top_p_keeps_at_least_min_tokens():
    V, n = 41, 20000
    row = torch.randn(V, generator=torch.Generator().manual_seed(13)) * 3
    logits = row.to(DEV)[None].repeat(n, 1).contiguous()
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    full = lambda v, dt: torch.full((n,), v, dtype=dt, device=DEV)
    for k, p, m in ((0, 0.2, 5), (10, 0.1, 3), (4, 0.1, 9), (0, 0.9999, 2)):
        ops().sample(logits, out, temperature=full(1.5, torch.float32), top_k=full(k, torch.int32), top_p=full(p, torch.float32),
                     min_keep=full(m, torch.int32), seeds=full(3, torch.int64), counters=torch.arange(n, dtype=torch.int64, device=DEV))
        scores = row / 1.5
        vals, idx = torch.topk(scores, k or V)
        keep = P.top_p_on_device(vals, p, m)
        kept = set(idx[keep].tolist())
        drawn = set(out.cpu().tolist())
        assert drawn <= kept, (k, p, m)
        probs = torch.softmax(vals[keep], -1)
        likely = {int(t) for t, q in zip(idx[keep], probs) if q * n > 50}
        assert likely <= drawn, (k, p, m)


def test_sampling_large_vocabulary_top_k():
    V = 50272
    row = torch.randn(V, generator=torch.Generator().manual_seed(12))
    got = _draws(row, 2000, temperature=1.0, top_k=50)
    top = set(torch.topk(row, 50).indices.tolist())
    assert set(got.tolist()) <= top and len(set(got.tolist())) > 25


@pytest.mark.parametrize("n_heads,n_kv", [(4, 2), (3, 3), (8, 1)])
@pytest.mark.parametrize("window", [None, 45, 200])
@pytest.mark.parametrize("d", [128, 64, 80, 96, 112])
def test_attention_prefill_tc(n_heads, n_kv, window, d):
    """The tcgen05 prefill kernel (head sizes 64 to 128 in steps of 16; those between use the layout of 128
    with a partly filled second slice).  Unwritten rows of pages hold a large finite
    number: they are loaded with their page and must be weighted by exactly zero."""
    lens = [(0, 2), (0, 64), (0, 129), (30, 7), (64, 130), (15, 17), (200, 300), (5, 1), (1000, 260)]
    case = PagedCase(lens, n_heads, n_kv, d, torch.bfloat16, seed=77, poison=3.0e4)
    scale = 1.0 / math.sqrt(d)
    out = torch.zeros(case.N, n_heads * d, dtype=torch.bfloat16, device=DEV)
    o = ops()
    assert o.attention_prefill_tc_supported(case.q_flat, case.cache, out)
    o.attention_prefill_tc(case.q_flat, case.cache, case.bt, case.tile_req, case.tile_q0, case.q_start, case.q_len,
                           case.ctx_len, out, n_heads, scale, window or 0)
    o.raise_on_device_error()
    want = case.want(scale, window)
    keep = torch.ones(case.N, dtype=torch.bool, device=DEV)
    keep[case.decode_rows.long()] = False
    assert rel_err(out[keep], want[keep]) <= 1.5e-2
    assert float(out[~keep].float().abs().max()) == 0.0


@pytest.mark.parametrize("d", [128, 64, 80])
def test_attention_prefill_tc_more_pages_than_fit_in_shared_memory(d):
    """A context of more than 2,048 keys: the page numbers beyond the first 128 are read from global memory."""
    n_heads = 2
    case = PagedCase([(2900, 150), (0, 300)], n_heads, n_heads, d, torch.bfloat16, seed=5, poison=1.0e4)
    scale = 1.0 / math.sqrt(d)
    out = torch.zeros(case.N, n_heads * d, dtype=torch.bfloat16, device=DEV)
    ops().attention_prefill_tc(case.q_flat, case.cache, case.bt, case.tile_req, case.tile_q0, case.q_start, case.q_len,
                               case.ctx_len, out, n_heads, scale, 0)
    ops().raise_on_device_error()
    assert rel_err(out, case.want(scale, None)) <= 1.5e-2



@pytest.mark.parametrize("d", [128, 64, 48, 96])
def test_attention_kernels_with_pages_released_behind_the_window(d):
    """Behind a sliding window the cache manager gives pages back while a request runs: their block
    table entries are -1 and their contents belong to someone else.  Every attention kernel must
    leave them alone: the tcgen05 prefill kernel (which copies whole tiles of four pages and must
    not wait for bytes of pages it does not copy), the mma.sync prefill kernel, the decode kernel
    and the 32-bit kernel."""
    window, n_heads = 45, 2
    lens = [(200, 130), (100, 1), (64, 70), (333, 1), (50, 3), (16, 40), (47, 1)]
    scale = 1.0 / math.sqrt(d)
    o = ops()
    for kind in ("prefill_tc", "prefill", "decode", "simt"):
        if kind == "prefill_tc" and d not in (64, 80, 96, 112, 128):
            continue
        # (the tcgen05 kernel multiplies unwritten rows of pages that it does hold by zero: those must be finite)
        case = PagedCase(lens, n_heads, n_heads, d, torch.bfloat16, seed=31 + d,
                         **({"poison": 3.0e4} if kind == "prefill_tc" else {}))
        assert case.release_behind(window) >= 20
        want = case.want(scale, window)
        out = torch.zeros(case.N, n_heads * d, dtype=torch.bfloat16, device=DEV)
        multi = torch.ones(case.N, dtype=torch.bool, device=DEV)
        multi[case.decode_rows.long()] = False
        if kind == "prefill_tc":
            o.attention_prefill_tc(case.q_flat, case.cache, case.bt, case.tile_req, case.tile_q0, case.q_start, case.q_len,
                                   case.ctx_len, out, n_heads, scale, window)
            rows = multi
        elif kind == "prefill":
            o.attention_prefill(case.q_flat, case.cache, case.bt, case.tile_req, case.tile_q0, case.q_start, case.q_len,
                                case.ctx_len, out, n_heads, scale, window)
            rows = multi
        elif kind == "decode":
            o.attention_decode(case.q_flat, case.cache, case.bt, case.tok_req, case.positions, out, n_heads, scale, window,
                               rows=case.decode_rows, max_kv_len=400)
            rows = ~multi
        else:
            o.attention_simt(case.q_flat, case.cache, case.bt, case.tok_req, case.positions, out, n_heads, scale, window)
            rows = torch.ones_like(multi)
        o.raise_on_device_error()
        assert torch.isfinite(out.float()).all(), kind
        assert rel_err(out[rows], want[rows]) <= 1.5e-2, kind
