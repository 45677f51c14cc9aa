"""Host-side peer watch for the data-parallel step.

The fused optimizer kernel waits on flags that its peers write; if a peer process is gone the wait runs
into its time limit and the kernel reports a status word, but by then a launch has already touched the
peer's memory.  `PeerWatch` gives the ranks a way to learn of a lost peer on the HOST, before the next
launch: every rank publishes the step it is about to run in a key-value store (the process group's own
TCP store or any `torch.distributed.Store`), and checks that every peer has published the same step
within `timeout` seconds.  A rank that raised, exited between steps or never started is reported as
`PeerLost(ranks)` on every surviving rank, which can then checkpoint and leave without hanging in a
collective.

Cost: one store `set` and world-1 store reads per step (tens of microseconds each on one node), so it
is opt-in (`Trainer(peer_watch=...)`, `train_lm --peer_watch_s`).

Reference parity: the reference relies on NCCL timeouts and `TORCH_NCCL_ASYNC_ERROR_HANDLING`
(lm/train_1p3b/launch_hero_wave3d.sh:27-31); this is the host-side counterpart its trainers lack.
"""

from __future__ import annotations

import time


class PeerLost(RuntimeError):
    def __init__(self, ranks, step):
        super().__init__(f"peer rank(s) {sorted(ranks)} did not reach step {step}")
        self.ranks, self.step = sorted(ranks), step


class PeerWatch:
    def __init__(self, store, rank, world, timeout=5.0, prefix="dmb_alive", poll=0.01):
        self.store, self.rank, self.world = store, rank, world
        self.timeout, self.prefix, self.poll = timeout, prefix, poll

    def _key(self, r):
        return f"{self.prefix}/{r}"

    def beat(self, step):
        """Publish that this rank is about to run `step`."""
        self.store.set(self._key(self.rank), str(int(step)))

    def _read(self, r):
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                return -1
            return int(self.store.get(self._key(r)).decode())
        except Exception:
            return -1

    def check(self, step):
        """Block until every peer has published a step >= `step`, or raise `PeerLost` after `timeout`."""
        t0, pending = time.monotonic(), set(range(self.world)) - {self.rank}
        while pending:
            pending = {r for r in pending if self._read(r) < step}
            if not pending:
                return
            if time.monotonic() - t0 > self.timeout:
                raise PeerLost(pending, step)
            time.sleep(self.poll)

    def sync(self, step):
        self.beat(step)
        self.check(step)
