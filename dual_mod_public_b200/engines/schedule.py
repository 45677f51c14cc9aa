"""Cell schedules: how a sequence of T positions is cut into chunks and how many
Jacobi sweeps each chunk gets.

A schedule is a tuple of `Cell(pos0, c, sweeps)` covering [0, T) in order.
Sweeps == c is exact (the intra-chunk dependency is strictly lower triangular).
Reference parity: engines/wavescan/engine/schedule.py:14-69 (uniform chunks,
the exact c=1 schedule, the random mixed-size pool) and the (c, K) ladders of
lm/train_340m/train_flagship.py:60-100 and lm/train_1p3b/train_hero_wave3d.py:108-153.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import NamedTuple, Sequence

import numpy as np


class Cell(NamedTuple):
    pos0: int
    c: int
    sweeps: int


def check_schedule(cells: Sequence[Cell], T: int, max_sweeps: int | None = None) -> None:
    pos = 0
    for cell in cells:
        p, c, k = cell
        assert p == pos and c > 0 and 1 <= k <= (c if max_sweeps is None else max_sweeps), f"bad cell {cell} at {pos}"
        pos += c
    assert pos == T, f"schedule covers {pos} of {T} positions"


def uniform_chunks(T: int, c: int, n_sweeps: int | None = None) -> list[Cell]:
    """Fixed-size chunks (last one may be short); n_sweeps=None means exact (K=c)."""
    out = []
    for p in range(0, T, c):
        cc = min(c, T - p)
        out.append(Cell(p, cc, cc if n_sweeps is None else min(n_sweeps, cc)))
    return out


def exact_sequential(T: int) -> list[Cell]:
    """One position per cell: the oracle schedule through the cell code."""
    return [Cell(j, 1, 1) for j in range(T)]


@dataclass
class WaveScanSchedule:
    """Random pool of mixed-size schedules: chunk sizes drawn from `chunk_probs`,
    sweeps per size from `sweeps` (default K = c/2), optional random first-cell
    offset so chunk boundaries move between pool entries."""
    chunk_probs: dict = field(default_factory=lambda: {8: 0.2, 16: 0.4, 32: 0.4})
    sweeps: dict = field(default_factory=lambda: {8: 4, 16: 8, 32: 16})
    pool_size: int = 8
    random_offset: bool = True
    seed: int = 0

    def __post_init__(self):
        assert abs(sum(self.chunk_probs.values()) - 1.0) < 1e-9
        assert all(c in self.sweeps for c in self.chunk_probs)

    def _k(self, c: int) -> int:
        return min(self.sweeps.get(c, c), c)     # truncated chunks run exact

    def draw(self, T: int, rng: np.random.Generator) -> list[Cell]:
        sizes = np.array(sorted(self.chunk_probs))
        probs = np.array([self.chunk_probs[int(c)] for c in sizes])
        cells, pos = [], 0
        if self.random_offset:
            off = int(rng.integers(0, int(sizes.max())))
            if off:
                cells.append(Cell(0, off, self._k(off)))
                pos = off
        while pos < T:
            c = min(int(rng.choice(sizes, p=probs)), T - pos)
            cells.append(Cell(pos, c, self._k(c)))
            pos += c
        return cells

    def draw_pool(self, T: int) -> list[list[Cell]]:
        rng = np.random.default_rng(self.seed)
        return [self.draw(T, rng) for _ in range(self.pool_size)]


@dataclass
class KLadder:
    """Staircase curriculum over (chunk, sweeps) rungs.

    Training is cut into phases at the step fractions `bounds`; phase i trains at
    `rungs[i]`.  A fraction `probe_frac` of the steps after `probe_start` are
    probes that run one rung deeper (or `probe_mult` x the base sweeps), which keeps
    the deeper operator's gradient path alive.  `sid_of` is a pure function of the
    step, so every rank and every resumed run picks the same rung.

    `rungs` entries are (c, K).  `extra_top=True` lets the last phase probe one
    rung past the last base phase (the 340M ladder has 4 rungs for 3 phases);
    otherwise the last phase has no probes (the 1.3B ladder).
    """
    rungs: tuple = ((64, 8), (64, 16), (64, 32), (64, 64))
    bounds: tuple = (0.075, 0.70)
    probe_frac: float = 0.1
    probe_start: int = 0
    probe_mult: int | None = None
    total_steps: int = 1000

    @property
    def n_phases(self) -> int:
        return len(self.bounds) + 1

    def phase_of(self, step: int) -> int:
        prog = step / max(1, self.total_steps)
        return sum(1 for b in self.bounds if prog >= b)

    def _is_probe_step(self, step: int) -> bool:
        pf = self.probe_frac
        if pf <= 0:
            return False
        if abs(pf - 0.1) < 1e-12:
            return step % 10 == 3
        return int(step * pf) != int((step - 1) * pf)

    def sid_of(self, step: int) -> tuple[int, bool]:
        """(rung index, is_probe)."""
        ph = self.phase_of(step)
        deeper = self.probe_mult is not None or ph + 1 < len(self.rungs)
        if step >= self.probe_start and deeper and self._is_probe_step(step):
            return (ph if self.probe_mult else ph + 1), True
        return ph, False

    def cell_shape(self, step: int) -> tuple[int, int]:
        """(c, K) to run at this step."""
        sid, probe = self.sid_of(step)
        c, k = self.rungs[sid]
        if probe and self.probe_mult:
            k = min(c, k * self.probe_mult)
        return c, k

    def schedule(self, step: int, T: int) -> list[Cell]:
        c, k = self.cell_shape(step)
        return uniform_chunks(T, c, k)


def cosine_lr(step: int, total: int, warmup: int, lr: float, min_lr: float) -> float:
    """Linear warm-up then cosine decay to min_lr; steps past `total` stay at min_lr."""
    import math
    if step < warmup:
        return lr * (step + 1) / max(1, warmup)
    prog = min(1.0, (step - warmup) / max(1, total - warmup))
    return min_lr + 0.5 * (lr - min_lr) * (1.0 + math.cos(math.pi * prog))
