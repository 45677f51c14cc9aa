"""Randomised consistency of the two engine backends on CPU (fp32): the hand-derived backward over the op
table (the statement every kernel is tested against) and autograd through the reference cell, on random
schedules (ragged chunks, few sweeps), sliding windows, raw-pinned heads, factored operators and both
write-law families; and the wavefront engine against its autograd statement on random (C, K, window)."""

import copy
import random

import pytest
import torch

from dual_mod_public_b200 import DualModConfig
from dual_mod_public_b200.engines.wave3d import Wave3DEngine, wavefront_model_forward
from dual_mod_public_b200.engines.wavescan import WaveScanEngine
from dual_mod_public_b200.models import DualModLM
from dual_mod_public_b200.ops import TorchOps

from helpers import perturb

MRK = dict(ctx_mod="mult_res", k_ctx_norm="rms")


def random_case(seed):
    r = random.Random(seed)
    kw = dict(MRK) if r.random() < 0.5 else {}
    if r.random() < 0.5:
        kw.update(gate_rank=r.choice([8, 16]), ctx_rank=r.choice([8, 16]))
    elif "ctx_mod" in kw and r.random() < 0.5:
        kw.update(gate_rank=4, ctx_rank=4)                     # ranks the factored path refuses (not a multiple of 8)
    if r.random() < 0.4:
        kw["kmod_vraw_heads"] = r.choice([1, 2])
    if "ctx_mod" in kw and r.random() < 0.5:
        kw["v_clamp_tau"] = r.choice([0.5, 2.0])
    T = r.choice([24, 32, 40])
    if r.random() < 0.5:
        kw["local_window"] = r.randint(3, T)
    # ragged schedule: chunks of 1..12 positions, 1..c sweeps each
    cells, p = [], 0
    while p < T:
        c = min(T - p, r.choice([1, 3, 4, 8, 12]))
        cells.append((p, c, r.randint(1, c)))
        p += c
    return kw, T, cells


def build(T, **kw):
    torch.manual_seed(0)
    cfg = DualModConfig(d_model=64, n_layers=2, n_heads=4, vocab_size=61, max_seq_len=64, gate_bias_init=0.0,
                        checkpoint_chunk=0, ctx_proj_init_std=0.02, dtype="fp32", **kw)
    m = DualModLM(cfg).eval()
    perturb(m)
    return cfg, m


def grads(eng, m, idx, tgt):
    eng.zero_grads()
    eng.pack()
    loss = eng.train_step(idx, tgt).clone()
    return loss, {n: eng.grads.get(p).clone() for n, p in m.named_parameters()}


def rel(a, b):
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("seed", range(10))
def test_fused_statement_equals_autograd_on_random_schedules(seed):
    kw, T, cells = random_case(seed)
    cfg, m = build(T, **kw)
    g = torch.Generator().manual_seed(seed)
    idx = torch.randint(0, cfg.vocab_size, (2, T), generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (2, T), generator=g)
    tgt[1, T // 2] = -1
    e_f = WaveScanEngine(m, [cells], 2, T, backend="fused", ops=TorchOps(), loss_rows=16)
    e_g = WaveScanEngine(m, [cells], 2, T, backend="generic", ops=TorchOps(), loss_rows=16)
    lf, gf = grads(e_f, m, idx, tgt)
    lg, gg = grads(e_g, m, idx, tgt)
    assert abs(lf.item() - lg.item()) < 1e-5, (kw, cells)
    for n in gg:
        assert rel(gf[n], gg[n]) < 2e-4, (n, kw, cells)
    assert e_f.debug_scan() == []


@pytest.mark.parametrize("seed", range(6))
def test_wavefront_engine_equals_its_statement_on_random_shapes(seed):
    r = random.Random(100 + seed)
    kw = dict(MRK, gate_rank=8, ctx_rank=8) if r.random() < 0.5 else {}
    C = r.choice([4, 8])
    n = r.choice([3, 4, 5])
    T, K = C * n, r.randint(1, C * n)
    if r.random() < 0.5:
        kw["local_window"] = r.randint(2, T)
    cfg, m = build(T, **kw)
    g = torch.Generator().manual_seed(seed)
    idx = torch.randint(0, cfg.vocab_size, (2, T), generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (2, T), generator=g)
    eng = Wave3DEngine(m, [K], 2, T, C=C, backend="fused", ops=TorchOps(), loss_rows=16)
    le, ge = grads(eng, m, idx, tgt)

    def statement(model):
        params = dict(model.named_parameters())
        logits = wavefront_model_forward(model, idx, C, K)
        loss = torch.nn.functional.cross_entropy(logits.flatten(0, 1), tgt.flatten())
        gs = torch.autograd.grad(loss, list(params.values()), allow_unused=True)
        return loss, {n_: g_ for (n_, _), g_ in zip(params.items(), gs) if g_ is not None}

    # deep sweep chains can be ill-conditioned in fp32 (a rounding of one weight moves the gradient by 1e-5 and
    # more): judge the engine against a float64 statement, with the fp32 statement's own error as the noise floor
    l32, g32 = statement(m)
    m64 = copy.deepcopy(m).double()
    m64.rope_cos, m64.rope_sin = m64.rope_cos.double(), m64.rope_sin.double()
    l64, g64 = statement(m64)
    assert abs(le.item() - l64.item()) < 1e-5, (kw, C, K, T)
    for n_, ref in g64.items():
        floor = rel(g32[n_].double(), ref)
        assert rel(ge[n_].double(), ref) < 2 * floor + 2e-5, (n_, floor, kw, C, K, T)
