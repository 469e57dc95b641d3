"""CPU, three ranks over a TCP store: a rank that leaves between steps, and a rank that goes silent.

The scripted-failing-peer style of the reference's tests (a table of misbehaviours on the other side of a boundary,
crates/eidola-app-core/tests/chat_harness/mod.rs:100-108), applied to the tensor-parallel group: the surviving ranks
must learn of the loss on the host BEFORE their next launch and abort their communicator, so that no collective can
block.  The communicator here is a stub that records the abort; nothing touches a GPU."""
import multiprocessing as mp
import socket
import time

import pytest


class StubComm:
    def __init__(self):
        self.aborts = 0
        self.err = 0

    def async_error(self):
        return self.err

    def abort(self):
        self.aborts += 1


def _rank(rank, world, port, script, q):
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    from datetime import timedelta

    from torch.distributed import TCPStore

    from eidola_b200.host import PeerLost, StepGuard
    store = TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=30))
    comm = StubComm()
    guard = StepGuard(store, rank, world, comm, deadline_s=1.0)
    done = 0
    try:
        for step in range(1, 6):
            if script.get(rank) == ("leave", step):
                guard.leave()  # between steps: nothing of this rank is in flight
                q.put((rank, "left", done, comm.aborts))
                break
            if script.get(rank) == ("silent", step):
                time.sleep(3.0)  # never announces: a wedged process
                q.put((rank, "silent", done, comm.aborts))
                break
            guard.announce(step)
            guard.wait_peers(step)
            done = step  # the step would be launched here
        else:
            q.put((rank, "finished", done, comm.aborts))
    except PeerLost as e:
        q.put((rank, "peer_lost:" + ",".join(map(str, e.ranks)), done, comm.aborts))
    if rank == 0:
        time.sleep(3.5)  # the store's server outlives its clients


def _run(script):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, 3, port, script, q)) for r in range(3)]
    for p in procs:
        p.start()
    out = {}
    for _ in range(3):
        r, what, done, aborts = q.get(timeout=60)
        out[r] = (what, done, aborts)
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    return out


def test_healthy_group_runs_every_step():
    out = _run({})
    assert all(v == ("finished", 5, 0) for v in out.values()), out


def test_a_rank_that_leaves_between_steps_is_noticed_before_the_next_launch():
    out = _run({2: ("leave", 3)})
    assert out[2][0] == "left" and out[2][1] == 2
    for r in (0, 1):
        what, done, aborts = out[r]
        assert what == "peer_lost:2" and done == 2 and aborts == 1, out  # step 3 was never launched; one abort each


def test_a_silent_rank_turns_into_an_abort_at_the_deadline():
    out = _run({1: ("silent", 2)})
    for r in (0, 2):
        what, done, aborts = out[r]
        assert what == "peer_lost:1" and done == 1 and aborts == 1, out


def test_guard_deadline_with_an_injected_clock():
    """Pure host logic: a fake store and clock, no processes."""
    from eidola_b200.host import PeerLost, StepGuard

    class Store(dict):
        def set(self, k, v):
            self[k] = v

        def get(self, k):
            return self[k]

    now = [0.0]
    comm = StubComm()
    store = Store()
    g = StepGuard(store, 0, 2, comm, deadline_s=2.0, clock=lambda: now[0], sleep=lambda s: now.__setitem__(0, now[0] + 0.5))
    store.set("eb/step/1", "4")
    g.wait_peers(4)  # already there
    with pytest.raises(PeerLost) as e:
        g.wait_peers(5)
    assert e.value.ranks == [1] and comm.aborts == 1 and 2.0 < now[0] <= 3.0
    comm2 = StubComm()
    comm2.err = 7  # the communicator itself reports an asynchronous error
    g2 = StepGuard(store, 0, 2, comm2, deadline_s=100.0, clock=lambda: 0.0, sleep=lambda s: None)
    with pytest.raises(PeerLost):
        g2.wait_peers(9)
    assert comm2.aborts == 1
