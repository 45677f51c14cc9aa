"""Failure detection on the host, among CPU ranks: a rank that leaves between steps (or raises) is
reported to the survivors as PeerLost before their next launch; healthy ranks pass."""

import socket
import time

import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

from dual_mod_public_b200.parallel.heartbeat import PeerLost, PeerWatch


def _rank(rank, world, port, leave_at, q):
    store = dist.TCPStore("127.0.0.1", port, world, is_master=rank == 0, timeout=__import__("datetime").timedelta(seconds=20))
    # start-up is slow and uneven for spawned processes: meet once with a long limit, so that in the steps
    # below only the rank that leaves can exceed the watch's limit
    PeerWatch(store, rank, world, timeout=60.0, prefix="start").sync(0)
    w = PeerWatch(store, rank, world, timeout=5.0)
    try:
        for step in range(5):
            if rank == 1 and step == leave_at:
                q.put((rank, "left", step))
                if rank != 0:
                    return                                   # leaves between steps, nothing in flight
            w.sync(step)
        q.put((rank, "done", 5))
    except PeerLost as e:
        q.put((rank, "lost", (e.ranks, e.step)))
    if rank == 0:
        time.sleep(6.5)                                      # keep the store up until the others are done


@pytest.mark.parametrize("leave_at", [2, 99])
def test_lost_peer_is_reported_on_the_host(leave_at):
    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with socket.socket() as sk:                              # a port the system says is free
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    procs = [ctx.Process(target=_rank, args=(r, world, port, leave_at, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(world):
        r, what, info = q.get(timeout=60)
        got[r] = (what, info)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    if leave_at == 2:
        assert got[1] == ("left", 2)
        assert got[0] == ("lost", ([1], 2)) and got[2] == ("lost", ([1], 2))
    else:
        assert all(v == ("done", 5) for v in got.values())


def test_peer_watch_with_a_plain_dict_store():
    class DictStore(dict):
        def set(self, k, v):
            self[k] = v.encode()

        def get(self, k):
            return self[k]

        def check(self, keys):
            return all(k in self for k in keys)
    s = DictStore()
    a, b = PeerWatch(s, 0, 2, timeout=0.05), PeerWatch(s, 1, 2, timeout=0.05)
    a.beat(0)
    b.beat(0)
    a.check(0)
    b.check(0)
    a.beat(1)
    with pytest.raises(PeerLost) as e:
        a.check(1)
    assert e.value.ranks == [1] and e.value.step == 1
