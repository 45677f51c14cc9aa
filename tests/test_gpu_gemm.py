"""tcgen05 GEMM against torch.matmul in fp32, for the three operand layouts and for
shapes with ragged M / K tails."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def gemm():
    from dual_mod_public_b200.ops.cuda_ops import load_library
    from dual_mod_public_b200.ops.gemm import Tcgen05Gemm
    return Tcgen05Gemm(load_library(), torch.device(DEV))


def rnd(*s, seed=0):
    g = torch.Generator().manual_seed(seed + sum(s))
    return torch.randn(*s, generator=g).to(DEV).bfloat16()


def check(got, ref, what):
    err = (got.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 2e-2 * scale + 1e-3, f"{what}: err {err:.4g} scale {scale:.4g}"


SHAPES = [(128, 256, 64), (256, 512, 128), (2048, 4096, 1024), (300, 1024, 1024), (2048, 1024, 2816),
          (4096, 32000, 1024), (136, 264, 72)]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_linear(gemm, M, N, K):
    x, w = rnd(M, K), rnd(N, K, seed=1)
    assert gemm.ok_tn(x, w)
    y = gemm.linear(x, w)
    gemm.check()
    check(y, x.float() @ w.float().t(), "y")
    yf = gemm.linear(x, w, torch.float32)
    check(yf, x.float() @ w.float().t(), "y fp32")
    b = rnd(N, seed=2)
    check(gemm.linear(x, w, bias=b), x.float() @ w.float().t() + b.float(), "y + bias")


@pytest.mark.parametrize("M,N,K", SHAPES[:5] + [(136, 264, 72)])
def test_linear_dx(gemm, M, N, K):
    dy, w = rnd(M, N), rnd(N, K, seed=1)
    assert gemm.ok_nn(dy, w)
    dx = gemm.linear_dx(dy, w)
    gemm.check()
    check(dx, dy.float() @ w.float(), "dx")


# the last two have a long reduction and few output tiles: the split-K path with even and ragged slices
@pytest.mark.parametrize("M,N,K", SHAPES[:5] + [(136, 264, 72), (16384, 512, 256), (8256, 264, 136)])
def test_linear_dw_acc(gemm, M, N, K):
    rows = M
    dy, x = rnd(rows, N), rnd(rows, K, seed=1)
    dW = torch.ones(N, K, device=DEV)
    assert gemm.ok_tn_dw(dW, dy, x)
    gemm.linear_dw_acc(dW, dy, x)
    gemm.check()
    check(dW, 1 + dy.float().t() @ x.float(), "dW")


def test_strided_rows(gemm):
    big = rnd(64, 96, 512)
    x = big[:, 16:80].reshape(-1, 512) if False else big.view(-1, 512)[::1]
    w = rnd(1024, 512, seed=3)
    xs = big.view(-1, 1024)[:, :512]                 # row stride 1024, 512 wide
    y = gemm.linear(xs, w)
    check(y, xs.float() @ w.float().t(), "strided x")
