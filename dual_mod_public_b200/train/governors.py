"""Host-side stability machinery of the trainers.  Every decision here is a pure function of values that
are identical on all ranks (the global gradient norm out of the fused optimizer, the step number, the
all-gathered per-rank norms), so every rank takes the same branch without extra communication.

  SkipRule            outlier batch skip: EMA of accepted gradient norms per batch type (base / probe),
                      grace period, always skip non-finite, hard cap, deadlock breaker for genuine level
                      shifts, bounded EMA tracking on soft skips
  CalibratedClip      clip threshold = clip_mult x EMA of accepted norms per batch type after the grace
                      period (probe-aware), else the fixed max_norm
  rank_outlier_mask   per-rank rejection: ranks whose local norm is far above the median are excluded
  ChainRhoGovernor    LR multiplier from a smoothed instability signal (log-scaled cut, auto-release)
  CreepDetector       slow upward drift of the norm EMA relative to a trailing reference
  RewindGovernor      ring of healthy snapshots, wedge detection over a window of skips, rewind to a
                      snapshot older than the look-back with a rotated data seed, taint set, event log
  MetricsLogger       metrics.jsonl with a monotonic tick (rewinds make steps non-monotonic)
  FaultInjector       env-var driven fake spikes / storms / non-finite losses for testing the above

Reference parity: lm/train_340m/train_flagship.py:939-1003 (governor, skip, breaker), :1167-1261
(auto-rewind); lm/train_1p3b/train_hero_wave3d.py:894-920 (rank outliers), :936-997 (calibrated clip,
skip with hard cap), :1003-1016 (creep), :752-827 / :1107-1194 (rewind policy), :659-702 (metrics).
"""

from __future__ import annotations

import json
import math
import os
import time
from collections import deque
from dataclasses import dataclass, field


# ---------------------------------------------------------------------------------------------------
@dataclass
class SkipRule:
    skip_factor: float = 5.0        # skip when gn > skip_factor x EMA (after the grace period)
    grace_steps: int = 50           # accepted steps of a batch type before its EMA is trusted
    ema_beta: float = 0.98
    gn_hard: float = 0.0            # > 0: absolute cap, active from step 0
    breaker_len: int = 5            # consecutive finite skips that may re-warm the EMA ...
    breaker_flat: float = 2.0       # ... if their max < flat x min (a level shift, not a storm)
    breaker_near: float = 50.0      # ... and the level is < near x the old EMA
    soft_track: float = 0.0         # > 0: a skipped finite norm still moves the EMA, by at most this factor
    ema: dict = field(default_factory=lambda: {False: None, True: None})
    cnt: dict = field(default_factory=lambda: {False: 0, True: 0})
    consec: dict = field(default_factory=lambda: {False: [], True: []})
    skipped_total: int = 0

    def threshold(self, is_probe: bool) -> float:
        """Norm above which the coming step must be skipped (0 = no limit): what the fused optimizer
        kernel gets as `skip_norm`, so the decision is taken on the device with rank-identical bytes."""
        thr = 0.0
        e = self.ema[is_probe]
        if e is not None and self.cnt[is_probe] >= self.grace_steps:
            thr = self.skip_factor * e
        if self.gn_hard > 0:
            thr = self.gn_hard if thr == 0.0 else min(thr, self.gn_hard)
        return thr

    def decide(self, gn: float, loss: float, is_probe: bool) -> bool:
        """The skip decision for a finished backward (host statement of what the kernel does with
        `threshold`, plus the non-finite rule)."""
        if not (math.isfinite(gn) and math.isfinite(loss)):
            return True
        thr = self.threshold(is_probe)
        return thr > 0 and gn > thr

    def update(self, gn: float, loss: float, is_probe: bool, skipped: bool) -> bool:
        """Book-keeping after the step.  Returns True when the breaker re-warmed the EMA (the next
        step of this batch type will pass)."""
        finite = math.isfinite(gn) and math.isfinite(loss)
        rewarmed = False
        if skipped:
            self.skipped_total += 1
            if finite:
                c = self.consec[is_probe]
                c.append(gn)
                e = self.ema[is_probe]
                if len(c) >= self.breaker_len:
                    last = c[-self.breaker_len:]
                    if max(last) < self.breaker_flat * min(last) and e is not None and gn < self.breaker_near * e:
                        self.ema[is_probe], self.consec[is_probe], rewarmed = gn, [], True
                if not rewarmed and self.soft_track > 0 and e is not None:
                    self.ema[is_probe] = min(e * self.soft_track, self.ema_beta * e + (1 - self.ema_beta) * gn)
            return rewarmed
        self.consec[is_probe] = []
        e = self.ema[is_probe]
        self.ema[is_probe] = gn if e is None else self.ema_beta * e + (1 - self.ema_beta) * gn
        self.cnt[is_probe] += 1
        return False

    def state_dict(self):
        return {"gn_ema": dict(self.ema), "gn_cnt": dict(self.cnt), "skipped_total": self.skipped_total}

    def load_state_dict(self, sd):
        self.ema = {bool(k): v for k, v in sd.get("gn_ema", {}).items()} or {False: None, True: None}
        self.cnt = {bool(k): v for k, v in sd.get("gn_cnt", {}).items()} or {False: 0, True: 0}
        for k in (False, True):
            self.ema.setdefault(k, None)
            self.cnt.setdefault(k, 0)
        self.skipped_total = sd.get("skipped_total", 0)
        self.consec = {False: [], True: []}


# ---------------------------------------------------------------------------------------------------
@dataclass
class CalibratedClip:
    max_norm: float = 1.0
    clip_mult: float = 0.0          # 0 = fixed max_norm
    grace_steps: int = 50
    ema_beta: float = 0.98
    ema: dict = field(default_factory=lambda: {False: None, True: None})
    cnt: dict = field(default_factory=lambda: {False: 0, True: 0})

    def threshold(self, is_probe: bool) -> float:
        e = self.ema[is_probe]
        if self.clip_mult > 0 and e is not None and self.cnt[is_probe] >= self.grace_steps:
            return self.clip_mult * e
        return self.max_norm

    def update(self, gn: float, is_probe: bool):
        if math.isfinite(gn):
            e = self.ema[is_probe]
            self.ema[is_probe] = gn if e is None else self.ema_beta * e + (1 - self.ema_beta) * gn
            self.cnt[is_probe] += 1

    def state_dict(self):
        return {"clip_ema": dict(self.ema), "clip_cnt": dict(self.cnt)}

    def load_state_dict(self, sd):
        for k, v in sd.get("clip_ema", {}).items():
            self.ema[bool(k)] = v
        for k, v in sd.get("clip_cnt", {}).items():
            self.cnt[bool(k)] = v


# ---------------------------------------------------------------------------------------------------
def rank_outlier_mask(norms, factor=4.0, max_bad=1):
    """norms: the local gradient norm of every rank (the same list on every rank).  A rank is an
    outlier when its norm is non-finite or exceeds factor x the median of the finite norms.  Returns
    (keep: list[bool], skip_step: bool): more than `max_bad` outliers voids the whole step."""
    finite = sorted(n for n in norms if math.isfinite(n))
    if not finite:
        return [False] * len(norms), True
    med = finite[len(finite) // 2] if len(finite) % 2 else 0.5 * (finite[len(finite) // 2 - 1] + finite[len(finite) // 2])
    keep = [math.isfinite(n) and (factor <= 0 or n <= factor * max(med, 1e-30)) for n in norms]
    bad = len(norms) - sum(keep)
    return keep, bad > max_bad or sum(keep) == 0


# ---------------------------------------------------------------------------------------------------
@dataclass
class ChainRhoGovernor:
    """LR multiplier in [floor, 1]: 1 - alpha * log10(rho_ema / trigger), applied with a one-step lag.
    `rho` is any scalar that climbs exponentially before a blow-up (the engines expose the largest
    per-cell gradient amplification; the trainer falls back to gn / EMA)."""
    beta: float = 0.9
    alpha: float = 0.5
    trigger: float = 10.0
    floor: float = 0.1
    rho_ema: float | None = None
    mult: float = 1.0

    def update(self, rho: float) -> float:
        r = rho if math.isfinite(rho) else 1e30
        self.rho_ema = r if self.rho_ema is None else self.beta * self.rho_ema + (1 - self.beta) * r
        self.mult = min(1.0, max(self.floor, 1.0 - self.alpha * math.log10(max(self.rho_ema, 1e-9) / self.trigger)))
        return self.mult

    def reset(self):
        self.rho_ema, self.mult = None, 1.0


@dataclass
class CreepDetector:
    """Flags a slow climb: the fast EMA of the norm above `ratio` x a reference EMA that lags by `lag`
    accepted steps."""
    ratio: float = 3.0
    lag: int = 200
    beta: float = 0.98
    fast: float | None = None
    hist: deque = field(default_factory=lambda: deque(maxlen=4096))

    def update(self, gn: float) -> bool:
        if not math.isfinite(gn):
            return False
        self.fast = gn if self.fast is None else self.beta * self.fast + (1 - self.beta) * gn
        self.hist.append(self.fast)
        if len(self.hist) <= self.lag:
            return False
        return self.fast > self.ratio * self.hist[-1 - self.lag]


# ---------------------------------------------------------------------------------------------------
class RewindGovernor:
    """Ring of healthy snapshots + wedge detection.

    `note(step, skipped)` after every step; `want_snapshot(step)` says when the caller should write a
    ring snapshot (every `snap_interval` steps, only if the recent window is skip-free) and
    `add_snapshot(step, handle)` registers it (handle = path or an in-memory checkpoint); `wedged()`
    is True when the window holds `skip_thresh` skips; `choose(step)` returns (snap_step, handle,
    new_seed) for the newest snapshot at least `lookback` steps old that is not tainted, or None when
    the rewind limit is reached.  Steps rewound over become tainted targets: a later rewind never lands
    on a snapshot that already led into a wedge (never-regress policy)."""

    def __init__(self, window=50, skip_thresh=10, ring=4, snap_interval=100, lookback=100, max_rewinds=8,
                 seed=0, seed_stride=1000, log_path=None, drop=None):
        self.window, self.skip_thresh, self.ring_len = window, skip_thresh, ring
        self.snap_interval, self.lookback, self.max_rewinds = snap_interval, lookback, max_rewinds
        self.seed, self.seed_stride, self.log_path = seed, seed_stride, log_path
        self.recent = deque(maxlen=window)
        self.ring = []                                   # [(step, handle)]
        self.tainted = set()
        self.count = 0
        self.drop = drop or (lambda handle: None)        # called for handles that leave the ring
        self.t0 = time.time()

    def note(self, step, skipped):
        self.recent.append(1 if skipped else 0)

    def want_snapshot(self, step):
        return step > 0 and step % self.snap_interval == 0 and sum(self.recent) == 0

    def add_snapshot(self, step, handle):
        self.ring = [(s, h) for s, h in self.ring if s != step]
        self.ring.append((step, handle))
        self.ring.sort(key=lambda t: t[0])
        while len(self.ring) > self.ring_len:
            _, old = self.ring.pop(0)
            self.drop(old)

    def wedged(self):
        return sum(self.recent) >= self.skip_thresh and bool(self.ring)

    def choose(self, step, extra=None):
        cands = [(s, h) for s, h in self.ring if s <= step - self.lookback and s not in self.tainted]
        if not cands:
            cands = [(s, h) for s, h in self.ring if s not in self.tainted][:1] or self.ring[:1]
        self.count += 1
        if self.count > self.max_rewinds or not cands:
            return None
        snap_step, handle = cands[-1]
        new_seed = self.seed + self.seed_stride * self.count
        # everything newer than the target led into the wedge
        for s, _ in self.ring:
            if s > snap_step:
                self.tainted.add(s)
        self.ring = [(s, h) for s, h in self.ring if s <= snap_step]
        self.recent.clear()
        if self.log_path:
            os.makedirs(os.path.dirname(os.path.abspath(self.log_path)), exist_ok=True)
            with open(self.log_path, "a") as f:
                f.write(json.dumps({"reload_num": self.count, "detected_step": step, "reload_from_step": snap_step,
                                    "lost_steps": step - snap_step, "new_seed": new_seed,
                                    "wall_s": time.time() - self.t0, **(extra or {})}) + "\n")
        return snap_step, handle, new_seed

    def state_dict(self):
        return {"tainted": sorted(self.tainted), "rewind_count": self.count}

    def load_state_dict(self, sd):
        self.tainted = set(sd.get("tainted", []))
        self.count = sd.get("rewind_count", 0)


# ---------------------------------------------------------------------------------------------------
class MetricsLogger:
    """One JSON object per line in `<out_dir>/metrics.jsonl`.  `tick` increases by one per record
    whatever the step does, so plots stay monotonic across rewinds."""

    def __init__(self, out_dir, enabled=True, tick=0, wandb_project="", wandb_name="", wandb_config=None):
        """wandb_project: also mirror every record to that project (run `wandb_name`, resumable by name;
        the record's tick is the x axis, because rewinds make steps non-monotonic).  The mirror is dropped
        with a message when the package is missing or the service cannot be reached."""
        self.enabled, self.tick = enabled, tick
        self.path = os.path.join(out_dir, "metrics.jsonl")
        self._wb = None
        if enabled:
            os.makedirs(out_dir, exist_ok=True)
            self._f = open(self.path, "a")
            if wandb_project:
                try:
                    import wandb
                    self._wb = wandb.init(project=wandb_project, name=wandb_name or os.path.basename(out_dir),
                                          id=wandb_name or None, resume="allow", config=wandb_config or {})
                except Exception as e:                           # optional mirror: never stop a run for it
                    print(f"metrics mirror disabled: {e}", flush=True)

    def log(self, step, **kv):
        self.tick += 1
        if not self.enabled:
            return
        rec = {"step": int(step), "tick": self.tick, "time": time.time()}
        rec.update({k: (float(v) if isinstance(v, (int, float)) and not isinstance(v, bool) else v) for k, v in kv.items()})
        self._f.write(json.dumps(rec) + "\n")
        self._f.flush()
        if self._wb is not None:
            self._wb.log({k: v for k, v in rec.items() if isinstance(v, (int, float, bool))}, step=self.tick)

    def close(self):
        if self.enabled:
            self._f.close()
            if self._wb is not None:
                self._wb.finish()


# ---------------------------------------------------------------------------------------------------
class FaultInjector:
    """Host-side fault injection for exercising the governors, driven by environment variables:

      DMB_FAKE_SPIKE_STEPS="120,121"   multiply the reported gradient norm at these steps by DMB_FAKE_SPIKE_X (1e4)
      DMB_FAKE_STORM="300:340"         the same for a whole range (a wedge)
      DMB_FAKE_NAN_STEPS="77"          report a non-finite loss at these steps
      DMB_FAKE_RANK_SPIKE="50:1"       at step 50, rank 1 reports its local gradient norm multiplied by the same
                                       factor to the per-rank outlier check (which then drops that rank)

    The injection acts on the values the governors see (and on the skip threshold the optimizer kernel
    receives), never on device memory."""

    def __init__(self, env=None):
        env = os.environ if env is None else env
        ints = lambda s: {int(x) for x in s.split(",") if x.strip()}
        self.spikes = ints(env.get("DMB_FAKE_SPIKE_STEPS", ""))
        self.nans = ints(env.get("DMB_FAKE_NAN_STEPS", ""))
        self.factor = float(env.get("DMB_FAKE_SPIKE_X", "1e4"))
        storm = env.get("DMB_FAKE_STORM", "")
        self.storm = tuple(int(x) for x in storm.split(":")) if storm else None
        rs = env.get("DMB_FAKE_RANK_SPIKE", "")
        self.rank_spike = tuple(int(x) for x in rs.split(":")) if rs else None

    def rank_factor(self, step, rank):
        """What `rank` multiplies its reported local norm by at `step` (1.0 = nothing injected)."""
        return self.factor if self.rank_spike == (step, rank) else 1.0

    @property
    def active(self):
        return bool(self.spikes or self.nans or self.storm or self.rank_spike)

    def spiked(self, step, trajectory=0):
        """`trajectory` counts the rewinds so far: a storm belongs to the original data order, so the
        rotated data seed of a rewind dodges it (single spikes are tied to the step and recur)."""
        return step in self.spikes or (trajectory == 0 and self.storm is not None
                                       and self.storm[0] <= step < self.storm[1])

    def apply(self, step, gn, loss, trajectory=0):
        if self.spiked(step, trajectory):
            gn = gn * self.factor
        if step in self.nans:
            loss = float("nan")
        return gn, loss
