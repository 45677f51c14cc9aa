"""The CTA-pair GEMM (tcgen05 cta_group::2, 256 x 256 and 256 x 128 tiles over two SMs) against torch.matmul in
fp32, for the three operand layouts, ragged tails, bias, fp32 accumulate and the split-K path."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module", params=[256, 128], ids=["pair256x256", "pair256x128"])
def gemm(request):
    from dual_mod_public_b200.ops.cuda_ops import load_library
    from dual_mod_public_b200.ops.gemm import Tcgen05Gemm
    g = Tcgen05Gemm(load_library(), torch.device(DEV))
    g.pair = True
    g.pair_width(request.param)
    yield g
    g.pair_width(0)


def rnd(*s, seed=0):
    g = torch.Generator().manual_seed(seed + sum(s))
    return torch.randn(*s, generator=g).to(DEV).bfloat16()


def check(got, ref, what):
    err = (got.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 2e-2 * scale + 1e-3, f"{what}: err {err:.4g} scale {scale:.4g}"


SHAPES = [(512, 256, 128), (512, 512, 64), (2048, 4096, 1024), (1000, 1024, 1024), (2048, 1024, 2816),
          (4096, 32000, 1024), (520, 264, 72), (65536, 1024, 1024)]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_linear(gemm, M, N, K):
    x, w = rnd(M, K), rnd(N, K, seed=1)
    y = gemm.linear(x, w)
    gemm.check()
    check(y, x.float() @ w.float().t(), "y")
    if M * N <= 1 << 24:
        yf = gemm.linear(x, w, torch.float32)
        check(yf, x.float() @ w.float().t(), "y fp32")
        b = rnd(N, seed=2)
        check(gemm.linear(x, w, bias=b), x.float() @ w.float().t() + b.float(), "y + bias")
    gemm.check()


@pytest.mark.parametrize("M,N,K", SHAPES[:5] + [(520, 264, 72)])
def test_linear_dx(gemm, M, N, K):
    dy, w = rnd(M, N), rnd(N, K, seed=1)
    dx = gemm.linear_dx(dy, w)
    gemm.check()
    check(dx, dy.float() @ w.float(), "dx")


@pytest.mark.parametrize("rows,N,K", [(512, 512, 256), (2048, 4096, 1024), (16384, 512, 256), (8256, 520, 264),
                                      (65536, 1024, 1024)])
def test_linear_dw_acc(gemm, rows, N, K):
    dy, x = rnd(rows, N), rnd(rows, K, seed=1)
    dW = torch.ones(N, K, device=DEV)
    gemm.linear_dw_acc(dW, dy, x)
    gemm.check()
    check(dW, 1 + dy.float().t() @ x.float(), "dW")


def test_repeated_launches_reuse_the_pipeline(gemm):
    x, w = rnd(4096, 1024), rnd(4096, 1024, seed=1)
    ref = x.float() @ w.float().t()
    for _ in range(5):
        check(gemm.linear(x, w), ref, "y")
    gemm.check()


def test_the_narrow_route_takes_the_sweep_input_gradient():
    """DMB_GEMM_PAIR=narrow: bf16 results with too few 256-wide tiles for the SMs go to 256 x 128 pair tiles."""
    from dual_mod_public_b200.ops.cuda_ops import load_library
    from dual_mod_public_b200.ops.gemm import Tcgen05Gemm
    g = Tcgen05Gemm(load_library(), torch.device(DEV))
    g.pair = "narrow"
    dy, w = rnd(2048, 4096), rnd(4096, 1024, seed=1)
    check(g.linear_dx(dy, w), dy.float() @ w.float(), "dx")
    x, w2 = rnd(1024, 2304), rnd(2304, 2304, seed=2)
    check(g.linear(x, w2), x.float() @ w2.float().t(), "y")
    g.check()
