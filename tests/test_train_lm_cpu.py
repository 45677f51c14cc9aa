"""Governors (pure host logic) and the LM trainer loop on CPU: ladder, skip via the optimizer's
predicate, injected storm -> wedge -> rewind, checkpoint + resume, metrics records."""

import json
import math
import os

import torch

from dual_mod_public_b200.train import governors as G
from dual_mod_public_b200.train.train_lm import main as train_main
from helpers import free_port


def test_skip_rule_grace_threshold_breaker():
    r = G.SkipRule(skip_factor=3.0, grace_steps=3)
    assert r.threshold(False) == 0.0
    for _ in range(3):
        assert not r.decide(1.0, 2.0, False)
        r.update(1.0, 2.0, False, False)
    assert abs(r.threshold(False) - 3.0) < 1e-9 and r.threshold(True) == 0.0      # per batch type
    assert r.decide(10.0, 2.0, False) and not r.decide(2.9, 2.0, False)
    assert r.decide(float("nan"), 2.0, False) and r.decide(1.0, float("inf"), True)
    # a flat level shift re-warms after 5 finite skips; a storm (wild swings) never does
    for i in range(4):
        assert not r.update(5.0, 2.0, False, True)
    assert r.update(5.2, 2.0, False, True) and abs(r.ema[False] - 5.2) < 1e-9
    s = G.SkipRule(skip_factor=3.0, grace_steps=1)
    s.update(1.0, 2.0, False, False)
    for gn in (1e3, 1e6, 40.0, 1e9, 77.0, 1e4):
        assert not s.update(gn, 2.0, False, True)
    assert abs(s.ema[False] - 1.0) < 1e-9 and s.skipped_total == 6
    h = G.SkipRule(gn_hard=7.0)
    assert h.threshold(False) == 7.0
    t = G.SkipRule()
    t.load_state_dict(r.state_dict())
    assert t.ema == r.ema and t.cnt == r.cnt


def test_rank_outlier_mask_and_clip():
    keep, void = G.rank_outlier_mask([1.0, 1.1, 0.9, 50.0], factor=4.0, max_bad=1)
    assert keep == [True, True, True, False] and not void
    keep, void = G.rank_outlier_mask([1.0, float("nan"), 60.0, 1.0], factor=4.0, max_bad=1)
    assert keep == [True, False, False, True] and void
    assert G.rank_outlier_mask([float("nan")] * 2)[1]
    c = G.CalibratedClip(max_norm=1.0, clip_mult=2.0, grace_steps=2)
    assert c.threshold(False) == 1.0
    c.update(3.0, False)
    c.update(3.0, False)
    assert abs(c.threshold(False) - 6.0) < 1e-9 and c.threshold(True) == 1.0


def test_governor_creep_rewind_injector(tmp_path):
    g = G.ChainRhoGovernor(beta=0.0, alpha=0.5, trigger=10.0, floor=0.1)
    assert g.update(5.0) == 1.0 and abs(g.update(1000.0) - 0.1) < 0.91 and g.update(float("nan")) == 0.1
    g.reset()
    assert g.mult == 1.0
    cd = G.CreepDetector(ratio=2.0, lag=5, beta=0.0)
    assert not any(cd.update(1.0) for _ in range(10))
    assert any(cd.update(1.0 + 0.5 * i) for i in range(10))
    dropped = []
    rw = G.RewindGovernor(window=6, skip_thresh=3, ring=2, snap_interval=10, lookback=10, max_rewinds=2, seed=5,
                          seed_stride=100, log_path=str(tmp_path / "rw.jsonl"), drop=dropped.append)
    for s in range(1, 41):
        rw.note(s, False)
        if rw.want_snapshot(s):
            rw.add_snapshot(s, f"h{s}")
    assert [s for s, _ in rw.ring] == [30, 40] and dropped == ["h10", "h20"]
    for s in range(41, 44):
        rw.note(s, True)
    assert rw.wedged()
    snap, handle, seed = rw.choose(43)
    assert (snap, handle, seed) == (30, "h30", 105) and 40 in rw.tainted and not rw.wedged()
    assert rw.choose(50) is not None and rw.choose(60) is None                       # at most 2 rewinds
    assert len(open(tmp_path / "rw.jsonl").read().strip().splitlines()) == 2
    inj = G.FaultInjector({"DMB_FAKE_SPIKE_STEPS": "3,4", "DMB_FAKE_STORM": "10:12", "DMB_FAKE_NAN_STEPS": "7"})
    assert inj.active and inj.spiked(3) and inj.spiked(11) and not inj.spiked(12)
    assert inj.apply(3, 1.0, 2.0)[0] == 1e4 and math.isnan(inj.apply(7, 1.0, 2.0)[1])
    assert not G.FaultInjector({}).active


def _records(out):
    return [json.loads(l) for l in open(os.path.join(out, "metrics.jsonl"))]


def test_trainer_loop_checkpoint_resume(tmp_path):
    out = str(tmp_path / "run")
    common = ["--recipe", "tiny", "--synthetic", "--device", "cpu", "--out_dir", out, "--warmup_steps", "2",
              "--log_every", "100", "--ckpt_every", "4", "--lr", "3e-3"]
    r1 = train_main(common + ["--total_steps", "9"])
    recs = _records(out)
    assert r1["step"] == 9 and r1["applied"] == 9 and len(recs) == 9
    assert [r["train/K"] for r in recs] == [2, 2, 2, 4, 4, 4, 4, 16, 16][:9] or recs[3]["train/is_probe"]
    assert recs[-1]["train/loss"] < recs[0]["train/loss"]
    ck = torch.load(os.path.join(out, "ckpt_latest.pt"), weights_only=False)
    assert ck["step"] == 8 and set(ck) >= {"model", "optimizer", "step", "applied", "model_cfg", "gn_ema", "gn_cnt"}
    assert os.path.exists(os.path.join(out, "ckpt_prev.pt"))
    r2 = train_main(common + ["--total_steps", "12", "--resume", "auto"])
    assert r2["step"] == 12 and r2["applied"] == 12
    assert [r["step"] for r in _records(out)][-3:] == [9, 10, 11]


def test_injected_storm_is_skipped_and_rewound(tmp_path, monkeypatch):
    out = str(tmp_path / "storm")
    monkeypatch.setenv("DMB_FAKE_STORM", "8:12")
    r = train_main(["--recipe", "tiny", "--synthetic", "--device", "cpu", "--out_dir", out, "--total_steps", "16",
                    "--warmup_steps", "2", "--log_every", "100", "--auto_rewind", "--snap_interval", "3",
                    "--rewind_window", "6", "--rewind_skip_thresh", "3", "--rewind_lookback", "2",
                    "--probe_frac", "0"])
    recs = _records(out)
    skipped = [x["step"] for x in recs if x["train/skipped"]]
    assert skipped[:3] == [8, 9, 10] and r["rewinds"] >= 1
    ev = [json.loads(l) for l in open(os.path.join(out, "rewind_events.jsonl"))]
    assert ev[0]["detected_step"] == 10 and ev[0]["reload_from_step"] == 6
    ticks = [x["tick"] for x in recs]
    assert ticks == sorted(ticks) and len(set(ticks)) == len(ticks)               # monotonic across the rewind
    assert r["step"] == 16


TINY = ["--recipe", "tiny", "--synthetic", "--device", "cpu", "--warmup_steps", "2", "--log_every", "100",
        "--probe_frac", "0"]


def test_group_doctrines_and_state_regrouping():
    from dual_mod_public_b200 import preset
    from dual_mod_public_b200.models import DualModLM
    from dual_mod_public_b200.parallel import hybrid_optim as H
    from dual_mod_public_b200.parallel.fused_optim import FusedDPAdamW, default_buckets
    torch.manual_seed(0)
    m = DualModLM(preset("tiny_cpu"))
    n_all = len(H.named_unique(m))
    split, every = H.optimizer_groups(m, "split", 0.1), H.optimizer_groups(m, "all", 0.1)
    assert len(split) == 2 and len(every) == 1 and len(every[0]["params"]) == n_all
    assert all(p.dim() >= 2 for p in split[0]["params"]) and split[1]["weight_decay"] == 0.0
    dm = H.optimizer_groups(m, "split", 0.1, only=lambda n: H.matches(n, H.DM_NAMES))
    trunk = H.optimizer_groups(m, "split", 0.1, only=lambda n: not H.matches(n, H.DM_NAMES))
    assert sum(len(g["params"]) for g in dm + trunk) == n_all and dm
    cd = H.recall_only(split, m)
    frozen = [p for g in cd if g["lr_mult"] == 0.0 for p in g["params"]]
    assert any(p is m.blocks[0].mlp.w1.weight for p in frozen)
    assert not any(p is m.blocks[0].attn.w_kctx.weight for p in frozen)
    # one step under "all", then carry the moments into the "split" layout: same moments per parameter
    o1 = FusedDPAdamW(every, default_buckets(m), lr=1e-3, use_kernel=False)
    for p in m.parameters():
        o1.grad_buffers().get(p).normal_()
    o1.step()
    sd = o1.state_dict()
    o2 = FusedDPAdamW(split, default_buckets(m), lr=1e-3, use_kernel=False)
    o2.load_state_dict(H.regroup_state(sd, m, o2.param_groups, 0.1))
    sd2 = o2.state_dict()
    old = {id(p): sd["state"][i]["exp_avg"] for i, p in enumerate(every[0]["params"])}
    i = 0
    for g in o2.param_groups:
        for p in g["params"]:
            assert torch.equal(sd2["state"][i]["exp_avg"], old[id(p)])
            i += 1
    assert H.regroup_state(sd2, m, o2.param_groups) is sd2


def test_two_speed_optimizer_steps_the_dual_mod_half_on_the_mean_gradient(tmp_path):
    out = str(tmp_path / "hyb")
    r = train_main(TINY + ["--out_dir", out, "--total_steps", "6", "--dm_accum", "3", "--dm_lr", "1e-3",
                           "--ckpt_every", "5", "--lr", "3e-3"])
    recs = _records(out)
    assert [x["train/dm_stepped"] for x in recs] == [False, False, True, False, False, True]
    ck = torch.load(os.path.join(out, "ckpt_latest.pt"), weights_only=False)
    assert "optimizer_dm" in ck and len(ck["optimizer_dm"]["state"]) > 0
    assert r["applied"] == 6 and recs[-1]["train/loss"] < recs[0]["train/loss"]
    # the same checkpoint resumes a one-optimizer run (moments regrouped) and a two-speed run
    train_main(TINY + ["--out_dir", out, "--total_steps", "8", "--resume", "auto", "--dm_accum", "2"])


def test_hybrid_halves_match_separate_adamw_on_accumulated_gradients():
    from dual_mod_public_b200 import preset
    from dual_mod_public_b200.models import DualModLM
    from dual_mod_public_b200.parallel import hybrid_optim as H
    from dual_mod_public_b200.parallel.fused_optim import NcclAdamW
    torch.manual_seed(0)
    m = DualModLM(preset("tiny_cpu"))
    ref = {n: p.detach().clone() for n, p in m.named_parameters()}
    is_dm = lambda n: H.matches(n, H.DM_NAMES)
    mk = lambda only: NcclAdamW(H.optimizer_groups(m, "split", 0.0, only=only), lr=1e-2, max_norm=0.0)
    hy = H.HybridAdamW(mk(lambda n: not is_dm(n)), mk(is_dm), dm_accum=2)
    G_ = hy.grad_buffers()
    grads = []
    for it in range(2):
        hy.zero_grad()
        g = {n: torch.randn_like(p) * 0.01 for n, p in m.named_parameters()}
        for n, p in m.named_parameters():
            G_.get(p).add_(g[n])
        grads.append(g)
        ctrl = hy.step().tolist()
        assert ctrl[3] == float(it == 1)
    name = "blocks.0.attn.w_kctx.weight"
    mean_g = 0.5 * (grads[0][name] + grads[1][name])
    # first AdamW step from zero moments moves every entry by lr * g / (|g| + eps)
    moved = dict(m.named_parameters())[name].detach() - ref[name]
    assert torch.allclose(moved, -1e-2 * mean_g / (mean_g.abs() + 1e-8), atol=2e-5)
    trunk = "blocks.0.mlp.w1.weight"
    assert not torch.equal(dict(m.named_parameters())[trunk].detach(), ref[trunk])


def test_cooldown_moves_only_the_write_law(tmp_path):
    out = str(tmp_path / "cd")
    train_main(TINY + ["--out_dir", out, "--total_steps", "3", "--ckpt_every", "2", "--lr", "3e-3"])
    before = torch.load(os.path.join(out, "ckpt_latest.pt"), weights_only=False)["model"]
    r = train_main(TINY + ["--out_dir", out, "--total_steps", "50", "--resume", "auto", "--cooldown_steps", "3",
                           "--cooldown_lr_start", "1e-3", "--cooldown_lr_end", "1e-4"])
    assert r["applied"] == 3 + 3
    snaps = [f for f in os.listdir(out) if f.startswith("snap_cooldown_")]
    assert len(snaps) == 1
    after = torch.load(os.path.join(out, snaps[0]), weights_only=False)["model"]
    assert torch.equal(after["blocks.0.mlp.w1.weight"], before["blocks.0.mlp.w1.weight"])
    assert torch.equal(after["tok_emb.weight"], before["tok_emb.weight"])
    assert not torch.equal(after["blocks.0.attn.w_kctx.weight"], before["blocks.0.attn.w_kctx.weight"])
    lrs = [x["train/lr"] for x in _records(out)][-3:]
    assert abs(lrs[0] - 1e-3) < 1e-9 and lrs[0] > lrs[1] > lrs[2] > 1e-4


def test_sam_step_restores_the_weights_and_reports_sharpness(tmp_path):
    from dual_mod_public_b200 import preset
    from dual_mod_public_b200.engines.schedule import uniform_chunks
    from dual_mod_public_b200.train import Trainer
    cfg = preset("tiny_cpu")
    mk = lambda: Trainer(cfg, [uniform_chunks(64, 16, 4)], seq_len=64, micro_batch=2, local_batch=4, lr=0.0,
                         device="cpu", autocast_bf16=False, use_graphs=False, seed=3)
    a, b = mk(), mk()
    toks = torch.randint(0, cfg.vocab_size, (4, 65), generator=torch.Generator().manual_seed(1))
    sam = [p for n, p in a.model.named_parameters() if "w_kctx" in n or "w_vctx" in n]
    la = a.sam_step(toks, sam, rho=0.05)
    lb = b.step(toks)
    assert math.isfinite(a.sam_sharpness) and la != lb               # the reported loss is at theta + eps
    # lr = 0: the weights must be exactly where they started
    for (n, p), (_, q) in zip(a.model.named_parameters(), b.model.named_parameters()):
        assert torch.equal(p, q), n
    # the gradient the optimizer saw differs from the plain one only through the perturbation
    ga, gb = a.opt.grad_buffers().get(sam[0]), b.opt.grad_buffers().get(
        [p for n, p in b.model.named_parameters() if "w_kctx" in n][0])
    assert not torch.equal(ga, gb) and torch.allclose(ga, gb, atol=0.3 * gb.abs().max().item())
    out = str(tmp_path / "sam")
    train_main(TINY + ["--out_dir", out, "--total_steps", "3", "--sam", "--sam_every", "2", "--telemetry_every", "2"])
    recs = _records(out)
    assert [x["train/sam_active"] for x in recs] == [1, 0, 1] and "train/sam_sharp" in recs[0]
    assert "gates/g_k_L00" in recs[0] and "vtail/p999_L00" in recs[2] and "telemetry/g_v_mean_all_layers" in recs[0]


def test_observability_keys(tmp_path):
    out = str(tmp_path / "obs")
    train_main(["--recipe", "tiny", "--synthetic", "--device", "cpu", "--warmup_steps", "2", "--log_every", "100",
                "--out_dir", out, "--total_steps", "8", "--probe_frac", "0.5", "--val_every", "3", "--val_batches", "1",
                "--val_exact_K", "16", "--eager_val_every", "3", "--eager_val_len", "40"])
    recs = _records(out)
    x = [r for r in recs if "val/loss_eager_xcheck" in r]
    assert x and all(abs(r["val/loss_eager_xcheck"] - r["val/loss_engine_xcheck"]) < 1e-4 for r in x)
    assert any("probe/loss" in r and "probe/grad_norm" in r for r in recs)
    assert any("base/loss" in r for r in recs) and all(("probe/loss" in r) != ("base/loss" in r) for r in recs)
    v = [r for r in recs if "val/loss" in r]
    assert v and all("val/loss_exact" in r and "val/base_minus_k16" in r and "val/base_K" in r for r in v)
    # at the deepest rung of the tiny recipe (c = K = 16) the base operator is the exact one
    assert abs(v[-1]["val/loss_deep"] - v[-1]["val/loss_exact"]) < 1e-5


def _lm_rank(rank, world, port, out, extra, env):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), **env)
    train_main(["--recipe", "tiny", "--synthetic", "--device", "cpu", "--warmup_steps", "2", "--log_every", "100",
                "--probe_frac", "0", "--out_dir", out, "--total_steps", "5", "--lr", "3e-3"] + extra)


def _spawn_lm(tmp_path, name, extra, env=None, world=2):
    import torch.multiprocessing as mp
    out = str(tmp_path / name)
    ctx = mp.get_context("spawn")
    port = free_port()
    procs = [ctx.Process(target=_lm_rank, args=(r, world, port, out, extra, env or {})) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
        assert p.exitcode == 0
    return _records(out)


def test_ranks_drop_a_spiking_rank_and_keep_training(tmp_path):
    # four ranks: with two, the median of (1, spike) hides the spike
    recs = _spawn_lm(tmp_path, "rs", ["--rank_outlier_factor", "4"], env={"DMB_FAKE_RANK_SPIKE": "3:1"}, world=4)
    assert [r["train/rank_excl"] for r in recs] == [0, 0, 0, 1, 0]
    assert not any(r["train/skipped"] for r in recs) and all(math.isfinite(r["train/loss"]) for r in recs)


def test_two_ranks_two_speed_optimizer_and_sam(tmp_path):
    recs = _spawn_lm(tmp_path, "hy", ["--dm_accum", "2", "--sam", "--sam_every", "2"])
    assert [r["train/dm_stepped"] for r in recs] == [False, True, False, True, False]
    assert [r["train/sam_active"] for r in recs] == [1, 0, 1, 0, 1]
    assert recs[-1]["train/loss"] < recs[0]["train/loss"] + 0.05


def test_wild_norm_triggers_a_buffer_scan(tmp_path, monkeypatch, capsys):
    monkeypatch.setenv("DMB_FAKE_NAN_STEPS", "2")
    out = str(tmp_path / "scan")
    # a non-finite loss voids the step; the norm itself stays finite, so force the scan through the norm as well
    monkeypatch.setenv("DMB_FAKE_SPIKE_STEPS", "3")
    monkeypatch.setenv("DMB_FAKE_SPIKE_X", "1e9")
    train_main(TINY + ["--out_dir", out, "--total_steps", "5"])
    recs = _records(out)
    assert recs[2]["train/skipped"] and recs[3]["train/skipped"]


def test_trainer_stops_when_a_peer_wait_ran_out(tmp_path, monkeypatch, capsys):
    """The optimizer's status word set by hand at step 5 (what its kernels do when a bounded wait for a peer
    runs out): the loop names the peer and the phase, writes its newest resident snapshot and stops."""
    import pytest

    from dual_mod_public_b200.parallel.fused_optim import PeerWaitExpired
    from dual_mod_public_b200.train.trainer import Trainer
    out = str(tmp_path / "lost")
    real_step = Trainer.step

    def step(self, tokens, **kw):
        if self.steps_done == 5:
            self.opt.status[0], self.opt.status[1] = 1, 3
        return real_step(self, tokens, **kw)

    monkeypatch.setattr(Trainer, "step", step)
    with pytest.raises(PeerWaitExpired, match="rank 3 at the opening barrier"):
        train_main(TINY + ["--out_dir", out, "--total_steps", "12", "--auto_rewind", "--snap_interval", "2"])
    assert "resident snapshot of step 4" in capsys.readouterr().out
    ck = torch.load(os.path.join(out, "ckpt_emergency_rank0.pt"), weights_only=False)
    assert ck["step"] == 4 and "model" in ck and "optimizer" in ck
    steps = [x["step"] for x in _records(out)]
    assert steps == [0, 1, 2, 3, 4]                                                # nothing logged as trained after it
