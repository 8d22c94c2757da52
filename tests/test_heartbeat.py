"""
Failure detection on the host: a rank killed by SIGKILL between steps is named by the survivors' heartbeat
within a deadline (nobody enters a collective with it again, nobody hangs); an orderly departure reads as
"left"; a store that stops answering counts as a loss; the loss watch flags NaN at once and a sustained blow-up.
"""
import json
import os
import socket
import subprocess
import sys
import time

import pytest

from nanochat_b200.parallel.heartbeat import Heartbeat, LossWatch, RankLostError

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run_ranks(mode, out_dir, world=3, deadline=90):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()), WORLD_SIZE=str(world),
               OMP_NUM_THREADS="1")
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "_hb_worker.py"), mode, out_dir],
                              env=dict(env, RANK=str(r), LOCAL_RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(world)]
    t0 = time.time()
    outs = []
    for p in procs:
        try:
            outs.append(p.communicate(timeout=max(1, deadline - (time.time() - t0)))[0])
        except subprocess.TimeoutExpired:
            p.kill()                                     # the exact child this test started
            outs.append("TIMEOUT " + p.communicate()[0])
    return procs, outs


@pytest.mark.slow
def test_killed_rank_is_named_by_every_survivor_within_the_deadline(tmp_path):
    procs, outs = _run_ranks("kill", str(tmp_path))
    assert procs[2].returncode == -9                     # the victim really died by SIGKILL
    for r in (0, 1):
        assert procs[r].returncode == 0 and "TIMEOUT" not in outs[r], outs[r][-2000:]
        got = json.load(open(tmp_path / f"rank{r}.json"))
        assert got["outcome"].startswith("error: lost rank(s) [2]") and got["lost"] == [2], got
        assert got["steps"] == 3 and got["seconds"] < 30, got
    assert not (tmp_path / "rank2.json").exists()


@pytest.mark.slow
def test_orderly_departure_is_not_an_error(tmp_path):
    procs, outs = _run_ranks("leave", str(tmp_path))
    assert all(p.returncode == 0 for p in procs), [o[-1500:] for o in outs]
    got = [json.load(open(tmp_path / f"rank{r}.json"))["outcome"] for r in range(3)]
    assert got == ["peer left", "peer left", "left"]


class _FakeStore:
    """A dict with the TCP store's set / get / check; `broken` makes every call raise."""

    def __init__(self):
        self.d, self.broken = {}, False

    def _guard(self):
        if self.broken:
            raise ConnectionError("store down")

    def set(self, k, v):
        self._guard()
        self.d[k] = v.encode() if isinstance(v, str) else v

    def get(self, k):
        self._guard()
        return self.d[k]

    def check(self, keys):
        self._guard()
        return all(k in self.d for k in keys)


def test_silent_peer_and_broken_store_are_losses():
    store = _FakeStore()
    a = Heartbeat(store, 0, 2, interval=0.05, timeout=1.0)
    b = Heartbeat(store, 1, 2, interval=0.05, timeout=1.0)
    a.wait_for_peers(deadline=5)
    time.sleep(0.3)
    a.check(); b.check()                                 # both beating: healthy
    b.stop()                                             # rank 1 goes silent without saying so
    t0 = time.time()
    with pytest.raises(RankLostError, match=r"lost rank\(s\) \[1\].*no heartbeat"):
        while time.time() - t0 < 5:
            a.check()
            time.sleep(0.05)
    a.stop()
    store2 = _FakeStore()
    c = Heartbeat(store2, 1, 3, interval=0.05, timeout=1.0)
    store2.broken = True
    t0 = time.time()
    with pytest.raises(RankLostError, match="store unreachable") as e:
        while time.time() - t0 < 5:
            c.check()
            time.sleep(0.05)
    assert e.value.ranks == [0, 2]
    c.stop()
    with pytest.raises(RankLostError, match="never started"):
        Heartbeat(_FakeStore(), 0, 2, interval=0.05, timeout=1.0).wait_for_peers(deadline=0.3)


def test_loss_watch():
    w = LossWatch(factor=3.0, patience=3, warmup=5)
    for i in range(30):
        assert w.update(4.0 - 0.05 * i) is None
    assert w.update(50.0) is None and w.update(2.4) is None        # one bad batch is forgiven
    assert w.update(40.0) is None and w.update(45.0) is None
    assert "above 3x" in w.update(60.0)                            # three in a row are not
    assert "nan" in LossWatch().update(float("nan")) and "inf" in LossWatch().update(float("inf"))
    early = LossWatch(warmup=20)
    assert all(early.update(v) is None for v in (1.0, 100.0, 1.0, 100.0))     # the warm-up only feeds the average
