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
    ops().gemm_simt(a, w, out, bias=bias, relu=True)
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


TC_SHAPES = [(1, 128, 64), (3, 96, 320), (16, 4096, 1024), (17, 1000, 96), (33, 200, 136), (64, 512, 4096),
             (65, 384, 256), (128, 128, 64), (200, 1000, 328), (300, 520, 1032), (2048, 768, 512)]


@pytest.mark.parametrize("M,N,K", TC_SHAPES)
def test_gemm_tc(M, N, K):
    o = ops()
    g = torch.Generator(device="cpu").manual_seed(M + N + K)
    a = (torch.randn(M, K, generator=g)).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16().to(DEV)
    bias = torch.randn(N, generator=g).to(DEV)
    want = a.float() @ w.float().t()
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    o.gemm_tc(a, w, out)
    o.raise_on_device_error()
    assert rel_err(out, want) <= 2e-5, "plain product"
    outb = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    o.gemm_tc(a, w, outb, bias=bias, relu=True)
    assert rel_err(outb, torch.relu(want + bias)) <= 5e-3, "bias + relu -> bf16"
    res = torch.randn(M, N, generator=g).to(DEV)
    want3 = want + bias + res
    o.gemm_tc(a, w, res, bias=bias, residual=res)
    o.raise_on_device_error()
    assert rel_err(res, want3) <= 2e-5, "bias + residual in place"


@pytest.mark.parametrize("M,N,K,splits", [(8, 256, 4096, 4), (64, 130, 1024, 16), (1, 128, 512, 2), (20, 300, 1160, 3)])
def test_gemm_tc_split_k(M, N, K, splits):
    o = ops()
    g = torch.Generator(device="cpu").manual_seed(splits)
    a = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16().to(DEV)
    bias = torch.randn(N, generator=g).to(DEV)
    want = torch.relu(a.float() @ w.float().t() + bias)
    out1 = torch.empty(M, N, dtype=torch.float32, device=DEV)
    out2 = torch.empty_like(out1)
    o.gemm_tc(a, w, out1, bias=bias, relu=True, splits=splits)
    o.gemm_tc(a, w, out2, bias=bias, relu=True, splits=splits)      # the counters were left at zero
    o.raise_on_device_error()
    assert rel_err(out1, want) <= 2e-5
    assert torch.equal(out1, out2), "the order of the additions is fixed"


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
