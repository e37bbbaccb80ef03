"""Multi-rank failure detection on CPU (gloo): a peer that leaves, vanishes or reports a failure stops the others with
``RankLostError`` between steps; nothing hangs and no GPU is involved."""
import os
import socket
import subprocess
import sys
import time

import pytest

from tensorrt_edge_llm_b200.parallel.health import GuardedComm, HealthMonitor, RankLostError

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(scenario, world=3):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1")
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "_health_worker.py"), scenario, str(port)], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    t0 = time.time()
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=60)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[killed by the test: hung]"
        outs.append((p.returncode, out))
    return outs, time.time() - t0


def test_healthy_job_finishes():
    outs, _ = _run("healthy", world=2)
    assert [rc for rc, _ in outs] == [0, 0], outs


@pytest.mark.parametrize("scenario,why", [("leave", "left the job"), ("raise", "bad weights"), ("vanish", "heartbeat")])
def test_lost_peer_stops_the_others(scenario, why):
    outs, took = _run(scenario)
    assert took < 40
    for rank in (0, 2):
        rc, out = outs[rank]
        assert rc == 42, (rank, out)
        # rank 2 may learn of it from rank 1's flag or, if rank 0 (which hosts the store) has already stopped, from the store
        assert "lost rank 1" in out or (rank == 2 and "lost rank -1" in out), out
    assert why in outs[0][1] or scenario == "vanish", outs[0][1]
    assert outs[1][0] in (0, 3)


class _FakeStore:
    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v.encode()

    def get(self, k):
        return self.d[k]

    def check(self, keys):
        return all(k in self.d for k in keys)


def test_monitor_and_guard_with_a_fake_store():
    store = _FakeStore()
    a = HealthMonitor(store, 0, 2, interval_s=0.02, timeout_s=0.15).start()
    b = HealthMonitor(store, 1, 2, interval_s=0.02, timeout_s=0.15).start()
    time.sleep(0.1)
    a.check()
    b.stop()                                   # b's heartbeats stop without a goodbye
    time.sleep(0.05)
    a.check()                                  # not stale yet
    time.sleep(0.3)
    with pytest.raises(RankLostError, match="no heartbeat"):
        a.check()

    class Boom:
        world_size, rank = 2, 0

        def all_reduce(self, x):
            raise TimeoutError("socket closed")

        def local_thing(self):
            return 7
    store2 = _FakeStore()
    m = HealthMonitor(store2, 0, 2)
    g = GuardedComm(Boom(), m)
    assert g.local_thing() == 7 and g.world_size == 2
    with pytest.raises(RankLostError, match="all_reduce failed"):
        g.all_reduce(None)
    assert store2.get("failed").decode().startswith("0: all_reduce failed")
    a.stop()
