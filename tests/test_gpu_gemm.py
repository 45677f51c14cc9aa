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


# few output tiles and a long reduction with a bf16 result: the two CTAs of a cluster split each tile's K range and
# add their accumulators through shared memory (the input gradient of a sweep is the first shape)
@pytest.mark.parametrize("M,N,K", [(2048, 1024, 4096), (1000, 520, 4160), (512, 256, 8192), (128, 256, 2048 + 72)])
def test_bf16_results_through_the_k_split(gemm, M, N, K):
    x, w = rnd(M, K), rnd(N, K, seed=1)
    ref = x.float() @ w.float().t()
    assert gemm.ksplit
    y_split = gemm.linear(x, w)
    gemm.ksplit = False
    y_plain = gemm.linear(x, w)
    gemm.ksplit = True
    gemm.check()
    check(y_split, ref, "y, K split")
    check(y_plain, ref, "y, one CTA per tile")
    wide = torch.zeros(M, N + 64, device=DEV, dtype=torch.bfloat16)
    gemm.linear(x, w, out=wide[:, 32:32 + N])
    gemm.check()
    check(wide[:, 32:32 + N], ref, "y into a column block")
    assert wide[:, :32].abs().max().item() == 0 and wide[:, 32 + N:].abs().max().item() == 0
    wn = rnd(K, N, seed=3)
    check(gemm.linear_dx(x, wn), x.float() @ wn.float(), "dx, K split")
    b = rnd(N, seed=4)
    check(gemm.linear(x, w, bias=b), ref + b.float(), "y + bias, K split")
    for _ in range(3):                                   # back-to-back launches: barriers and tensor memory start clean
        check(gemm.linear(x, w), ref, "y, repeated")
    gemm.check()


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


@pytest.mark.parametrize("rows,d,R", [(4096, 2304, 144), (512, 256, 16), (1000, 1024, 72)])
def test_factor_gemms_into_column_blocks(gemm, rows, d, R):
    """The shapes of a factored write law: a down GEMM onto 4R stacked rank columns, narrow up GEMMs from a
    rank-column block of one matrix into a d-column block of another (`out=` views with their own row
    strides), the transposed pair for the input gradient, and the weight gradients of both factors."""
    x = rnd(rows, d)
    D = rnd(4 * R, d, seed=1) * 0.05
    U = [rnd(d, R, seed=2 + i) * 0.05 for i in range(4)]
    assert gemm.ok_tn(x, D)
    t = gemm.linear(x, D)
    check(t, x.float() @ D.float().t(), "down")
    raw = torch.full((rows, 4 * d), 7.0, dtype=torch.bfloat16, device=DEV)
    for i in (0, 2, 3):                                       # block 1 stays untouched
        ti, oi = t[:, i * R:(i + 1) * R], raw[:, i * d:(i + 1) * d]
        assert gemm.ok_tn(ti, U[i]) and gemm.ok_out(oi, ti, d)
        gemm.linear(ti, U[i], out=oi)
        check(oi, ti.float() @ U[i].float().t(), f"up {i}")
    assert (raw[:, d:2 * d] == 7.0).all()
    dcg = rnd(rows, 4 * d, seed=9)
    dt = torch.full((rows, 4 * R), 7.0, dtype=torch.bfloat16, device=DEV)
    for i in (0, 1, 3):
        gi, oi = dcg[:, i * d:(i + 1) * d], dt[:, i * R:(i + 1) * R]
        assert gemm.ok_nn(gi, U[i]) and gemm.ok_out(oi, gi, R)
        gemm.linear_dx(gi, U[i], out=oi)
        check(oi, gi.float() @ U[i].float(), f"d down-out {i}")
    assert (dt[:, 2 * R:3 * R] == 7.0).all()
    dt[:, 2 * R:3 * R] = 0
    du = gemm.linear_dx(dt, D)
    check(du, dt.float() @ D.float(), "d read")
    dU = torch.ones(d, R, device=DEV)
    gi, ti = dcg[:, d:2 * d], t[:, R:2 * R]
    assert gemm.ok_tn_dw(dU, gi, ti)
    gemm.linear_dw_acc(dU, gi, ti)
    check(dU, 1 + gi.float().t() @ ti.float(), "dU")
    dD = torch.ones(4 * R, d, device=DEV)
    assert gemm.ok_tn_dw(dD, dt, x)
    gemm.linear_dw_acc(dD, dt, x)
    check(dD, 1 + dt.float().t() @ x.float(), "dD")
    gemm.check()
