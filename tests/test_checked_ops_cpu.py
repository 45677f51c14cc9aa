"""The launch-argument checker: clean on every engine path, and loud on the errors it exists for."""

import pytest
import torch

from dual_mod_public_b200 import DualModConfig
from dual_mod_public_b200.engines.schedule import uniform_chunks
from dual_mod_public_b200.engines.wave3d import Wave3DEngine
from dual_mod_public_b200.engines.wavescan import WaveScanEngine
from dual_mod_public_b200.models import DualModLM
from dual_mod_public_b200.ops import TorchOps
from dual_mod_public_b200.ops.checked import CheckedOps, OpArgumentError, maybe_checked

from helpers import perturb

MRK = dict(ctx_mod="mult_res", k_ctx_norm="rms", gate_rank=8, ctx_rank=8, kmod_vraw_heads=1, v_clamp_tau=0.8)


def build(T=32, **kw):
    torch.manual_seed(0)
    cfg = DualModConfig(d_model=64, n_layers=2, n_heads=4, vocab_size=61, max_seq_len=64, gate_bias_init=0.0,
                        checkpoint_chunk=0, ctx_proj_init_std=0.02, dtype="fp32", **kw)
    m = DualModLM(cfg).eval()
    perturb(m)
    return cfg, m


@pytest.mark.parametrize("kw", [dict(), dict(local_window=9), MRK, dict(ctx_mod="fusion", gate_type_v="independent")])
def test_engines_pass_the_checker_and_results_do_not_change(kw):
    cfg, m = build(**kw)
    g = torch.Generator().manual_seed(1)
    idx, tgt = torch.randint(0, 61, (2, 32), generator=g), torch.randint(0, 61, (2, 32), generator=g)
    for make in (lambda ops: WaveScanEngine(m, [uniform_chunks(32, 8, 3)], 2, 32, backend="fused", ops=ops),
                 lambda ops: Wave3DEngine(m, [3], 2, 32, C=8, backend="fused", ops=ops)):
        plain, checked = make(TorchOps()), make(CheckedOps(TorchOps(), check_finite=True))
        outs = []
        for eng in (plain, checked):
            eng.zero_grads()
            eng.pack()
            loss = eng.train_step(idx, tgt).clone()
            outs.append((loss, eng.grads.flat.clone()))
        assert checked.ops.calls_checked > 50
        assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


def test_checker_names_the_broken_rule(monkeypatch):
    ops = CheckedOps(TorchOps(), check_finite=True)
    B, T, h, dh, c = 2, 32, 4, 16, 8
    q, Kc, Vc = torch.randn(B, c, h, dh), torch.randn(B, T, h, dh), torch.randn(B, T, h, dh)
    ops.prefix_fwd(q, Kc, Vc, 16, 0.25)
    with pytest.raises(OpArgumentError, match="pos0"):
        ops.prefix_fwd(q, Kc, Vc, T + 8, 0.25)
    strict = CheckedOps(TorchOps(), strict_layout=True)
    with pytest.raises(OpArgumentError, match="not dense"):
        strict.prefix_fwd(q.transpose(2, 3).contiguous().transpose(2, 3), Kc, Vc, 16, 0.25)
    with pytest.raises(OpArgumentError, match="heads"):
        ops.prefix_fwd(q[:, :, :2], Kc, Vc, 16, 0.25)
    odd = torch.randn(B, T, h, dh + 2)[..., 1:dh + 1]                   # rows start 4 bytes off a 16-byte boundary
    with pytest.raises(OpArgumentError, match="aligned|boundary"):
        strict.prefix_fwd(q, odd, Vc, 16, 0.25)
    ops.prefix_fwd(q, odd, Vc, 16, 0.25)                                  # the torch statement takes any layout
    x, w = torch.randn(6, 8), torch.randn(5, 8)
    buf = torch.zeros(6, 16)
    ops.linear(x, w, out=buf[:, 8:13])
    with pytest.raises(OpArgumentError, match="overlaps the read tensor"):
        big = torch.randn(6, 16)
        ops.linear(big[:, :8], w, out=big[:, 4:9])
    with pytest.raises(OpArgumentError, match="inner sizes"):
        ops.linear(x, torch.randn(5, 7))
    # row slices of one buffer interleave without overlapping: accepted; the same rows twice: refused
    acc = torch.zeros(B, T, h, dh)
    o_c, lse_c = ops.prefix_fwd(q, Kc, Vc, 16, 0.25)
    args = (torch.randn(B, c, h, dh), q, q.clone(), q.clone(), q.clone(), q.clone(), o_c, lse_c, q.clone(), lse_c.clone(), 0.25, 0)
    ops.tail_bwd(*args, torch.zeros(B, c, h, dh), acc[:, 0:8], acc[:, 8:16], torch.zeros(B, c, h, dh), torch.zeros(B, c, h))
    with pytest.raises(OpArgumentError, match="overlaps the written tensor"):
        ops.tail_bwd(*args, torch.zeros(B, c, h, dh), acc[:, 0:8], acc[:, 4:12], torch.zeros(B, c, h, dh), torch.zeros(B, c, h))
    with pytest.raises(OpArgumentError, match="ids in"):
        ops.embed_bwd(torch.zeros(10, 4), torch.tensor([1, 12]), torch.randn(2, 4))
    with pytest.raises(OpArgumentError, match="non-finite"):
        ops.linear(torch.full((6, 8), float("inf")), w)
    assert ops.name == TorchOps().name and ops.calls_checked > 5                  # attributes pass through
    monkeypatch.setenv("DMB_CHECK_ARGS", "1")
    assert isinstance(maybe_checked(TorchOps()), CheckedOps)
    monkeypatch.delenv("DMB_CHECK_ARGS")
    t = TorchOps()
    assert maybe_checked(t) is t


def test_engines_wrap_their_table_on_request(monkeypatch):
    cfg, m = build()
    monkeypatch.setenv("DMB_CHECK_ARGS", "1")
    eng = WaveScanEngine(m, [uniform_chunks(32, 8, 2)], 2, 32, backend="fused", ops=TorchOps())
    assert isinstance(eng.ops, CheckedOps)
    g = torch.Generator().manual_seed(1)
    eng.pack()
    eng.train_step(torch.randint(0, 61, (2, 32), generator=g), torch.randint(0, 61, (2, 32), generator=g))
    assert eng.ops.calls_checked > 50
    monkeypatch.delenv("DMB_CHECK_ARGS")
    assert not isinstance(WaveScanEngine(m, [uniform_chunks(32, 8, 2)], 2, 32, backend="fused", ops=TorchOps()).ops, CheckedOps)


def test_gemm_routing_rule():
    """Which kernel a GEMM goes to: the cluster K split only for bf16 results with few tiles and a long reduction."""
    from dual_mod_public_b200.ops.gemm import gemm_kernel_for as route
    sms = 148
    assert route(2048, 1024, 4096, 0, 0, False, True, sms) == "dmb_gemm_bf16_ksplit2"      # input gradient of a sweep
    assert route(2048, 4096, 1024, 0, 0, False, True, sms) == "dmb_gemm_bf16"              # forward GEMM of a sweep
    assert route(2048, 1024, 4096, 1, 0, False, True, sms) == "dmb_gemm_bf16"              # fp32 result: workspace split-K
    assert route(2048, 1024, 4096, 0, 0, False, False, sms) == "dmb_gemm_bf16"
    assert route(65536, 1024, 2816, 0, 0, False, True, sms) == "dmb_gemm_bf16"             # many tiles
    assert route(1024, 2304, 2304, 0, 0, False, True, sms) == "dmb_gemm_bf16_ksplit2"      # 72 tiles, 144 CTAs
    assert route(1024, 2560, 2304, 0, 0, False, True, sms) == "dmb_gemm_bf16"              # 80 tiles: over half the SMs
    assert route(65536, 1024, 1024, 0, 0, True, True, sms) == "dmb_gemm_bf16_pair"
    assert route(256, 128, 64, 0, 0, True, True, sms) == "dmb_gemm_bf16"
    assert route(2048, 1024, 4096, 0, 0, "narrow", True, sms) == "dmb_gemm_bf16_pair"
    assert route(65536, 1024, 1024, 0, 0, "narrow", True, sms) == "dmb_gemm_bf16"
