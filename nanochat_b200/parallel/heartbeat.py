"""
Host-side failure detection for multi-rank runs: a store-based heartbeat and a loss watch.

The reference has neither a watchdog nor elasticity: a rank that dies leaves the others inside their next
collective until the backend's timeout (minutes) ends it, and a diverged loss is only visible in the log
(reference: scripts/base_train.py:501 carries a note that loss-explosion detection is missing). Here every
rank learns of a lost peer on the host, BEFORE it launches the next step's kernels, so no device-side wait is
ever started against a peer that is gone:

* `Heartbeat` - a daemon thread per rank bumps a counter `hb/<rank>` in the job's key-value store (the TCP
  store `torch.distributed` already runs) every `interval` seconds and reads the peers' counters. A peer whose
  counter has not moved for `timeout` seconds is lost; so is everyone when the store itself stops answering
  (the rank that hosts it died). `check()` raises `RankLostError` naming the ranks; training loops call it
  between steps. A rank that stops in an orderly way calls `leave()`, which peers see as "left", not "lost".
* `LossWatch` - flags a non-finite loss at once and a loss above `factor` x its running average after
  `patience` consecutive steps.

Nothing here touches a GPU; the tests run it among gloo ranks on CPU with one rank killed by SIGKILL.
"""

import math
import threading
import time

import torch.distributed as dist


class RankLostError(RuntimeError):
    def __init__(self, ranks, reason):
        self.ranks = sorted(ranks)
        super().__init__(f"lost rank(s) {self.ranks}: {reason}")


def default_store():
    """The key-value store of the default process group (None when there is no group)."""
    if not (dist.is_available() and dist.is_initialized()):
        return None
    from torch.distributed import distributed_c10d
    return distributed_c10d._get_default_store()


class Heartbeat:
    def __init__(self, store, rank, world_size, interval=1.0, timeout=10.0, prefix="hb", start=True):
        assert timeout > 2 * interval, "the timeout must cover at least two beats"
        self.store, self.rank, self.world = store, rank, world_size
        self.interval, self.timeout, self.prefix = interval, timeout, prefix
        now = time.monotonic()
        self._last_value = {r: None for r in range(world_size) if r != rank}
        self._last_change = {r: now for r in self._last_value}
        self._left = set()
        self._lost = {}
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._beats = 0
        self._thread = None
        if start and world_size > 1:
            self.start()

    def _key(self, r):
        return f"{self.prefix}/{r}"

    # ------------------------------------------------------------------ the thread
    def start(self):
        self._beat()
        self._thread = threading.Thread(target=self._run, name="nanochat-heartbeat", daemon=True)
        self._thread.start()

    def _beat(self):
        self._beats += 1
        self.store.set(self._key(self.rank), str(self._beats))

    def _scan(self):
        now = time.monotonic()
        for r in self._last_value:
            if r in self._left or r in self._lost:
                continue
            key = self._key(r)
            value = self.store.get(key).decode() if self.store.check([key]) else None
            if value == "left":
                self._left.add(r)
            elif value is not None and value != self._last_value[r]:
                self._last_value[r], self._last_change[r] = value, now
            elif now - self._last_change[r] > self.timeout:
                with self._lock:
                    self._lost[r] = f"no heartbeat for {now - self._last_change[r]:.1f} s"

    def _run(self):
        while not self._stop.wait(self.interval):
            try:
                self._beat()
                self._scan()
            except Exception as e:  # the store is gone: the rank hosting it died (or the job is being torn down)
                if self._stop.is_set():
                    return
                with self._lock:
                    for r in self._last_value:
                        if r not in self._left:
                            self._lost.setdefault(r, f"store unreachable ({type(e).__name__})")
                return

    # ---------------------------------------------------------------------- the API
    def lost(self):
        with self._lock:
            return dict(self._lost)

    def departed(self):
        return set(self._left)

    def check(self):
        """Raise RankLostError if a peer was lost. Call between steps, before the step's first launch."""
        lost = self.lost()
        if lost:
            raise RankLostError(lost.keys(), "; ".join(f"rank {r}: {why}" for r, why in sorted(lost.items())))

    def wait_for_peers(self, deadline=30.0):
        """Block until every peer has beaten once (start-up skew), or raise RankLostError."""
        t0 = time.monotonic()
        while any(v is None for r, v in self._last_value.items() if r not in self._left):
            self.check()
            if time.monotonic() - t0 > deadline:
                missing = [r for r, v in self._last_value.items() if v is None]
                raise RankLostError(missing, f"never started within {deadline:.0f} s")
            time.sleep(min(0.05, self.interval))

    def leave(self):
        """Orderly departure: stop beating and tell the peers this rank left on purpose."""
        self.stop()
        try:
            self.store.set(self._key(self.rank), "left")
        except Exception:
            pass

    def stop(self):
        self._stop.set()
        if self._thread is not None and self._thread is not threading.current_thread():
            self._thread.join(timeout=2 * self.interval + 1)
            self._thread = None


class LossWatch:
    """Divergence detector for a training loss.

    `update(loss)` returns None while training looks healthy, else a short reason. A non-finite loss is
    reported at once; a loss above `factor` x the debiased running average only after `patience` consecutive
    steps (one bad batch is not a divergence). The first `warmup` steps only feed the average.
    """

    def __init__(self, factor=3.0, patience=5, warmup=20, beta=0.95):
        self.factor, self.patience, self.warmup, self.beta = factor, patience, warmup, beta
        self.ema, self.steps, self.strikes, self.accepted = 0.0, 0, 0, 0

    def update(self, loss):
        loss = float(loss)
        if not math.isfinite(loss):
            return f"loss is {loss}"
        self.steps += 1
        mean = self.ema / (1 - self.beta ** self.accepted) if self.accepted > 0 else loss
        if self.steps > self.warmup and loss > self.factor * mean:
            self.strikes += 1
            if self.strikes >= self.patience:
                return f"loss {loss:.4f} above {self.factor:g}x its running average {mean:.4f} for {self.strikes} steps"
            return None                      # do not let the spike into the average
        self.strikes = 0
        self.ema = self.beta * self.ema + (1 - self.beta) * loss
        self.accepted += 1
        return None
