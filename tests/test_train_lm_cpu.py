"""Governors (pure host logic) and the LM trainer loop on CPU: ladder, skip via the optimizer's
predicate, injected storm -> wedge -> rewind, checkpoint + resume, metrics records."""

import json
import math
import os

import torch

from dual_mod_public_b200.train import governors as G
from dual_mod_public_b200.train.train_lm import main as train_main


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
