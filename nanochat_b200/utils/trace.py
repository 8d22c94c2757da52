"""
Observability for training and serving runs: NVTX ranges, device-timed phases and a JSONL metrics file.

The reference reports one wall-clock `dt` per optimizer step and, optionally, wandb scalars
(reference: scripts/base_train.py:517-560). That number says nothing about where a step's time goes and,
on several GPUs, hides which rank was slow. Three small tools fill that in; all are inert unless asked for,
so the default step launches exactly the kernels it launched before.

* `nvtx(name)` - a range for a timeline profiler. Active only with `NANOCHAT_NVTX=1` on a CUDA build.
* `PhaseTimers` - CUDA events around named phases (forward / backward / optimizer ...) on the launching
  stream. Recording an event does not synchronise; `collect()` waits once for the last event, sums the
  intervals of each phase and reduces every phase as the MAX over ranks, which is the figure that bounds
  a data-parallel step. On CPU it falls back to the host clock. Enabled by `NANOCHAT_TRACE=1` or
  `PhaseTimers(enabled=True)`.
* `MetricsLog` - appends one JSON object per `log()` call to a file, flushed per line so a killed run
  keeps what it wrote. It has wandb's `log` / `finish` surface and can forward to a real wandb run.
"""

import contextlib
import json
import os
import time

import torch
import torch.distributed as dist


def _env_on(name):
    return os.environ.get(name, "0") not in ("", "0", "false", "False")


def nvtx_enabled():
    return _env_on("NANOCHAT_NVTX") and torch.cuda.is_available()


_NULL = contextlib.nullcontext()


@contextlib.contextmanager
def _nvtx_range(name):
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


def nvtx(name):
    """Context manager: an NVTX range named `name` when NANOCHAT_NVTX=1, nothing otherwise."""
    return _nvtx_range(name) if nvtx_enabled() else _NULL


class _Phase:
    __slots__ = ("timers", "name", "start")

    def __init__(self, timers, name):
        self.timers, self.name, self.start = timers, name, None

    def __enter__(self):
        t = self.timers
        if t.nvtx:
            torch.cuda.nvtx.range_push(self.name)
        if t.cuda:
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record()
        else:
            self.start = time.perf_counter()
        return self

    def __exit__(self, *exc):
        t = self.timers
        if t.cuda:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
        else:
            end = time.perf_counter()
        t._intervals.setdefault(self.name, []).append((self.start, end))
        if t.nvtx:
            torch.cuda.nvtx.range_pop()
        return False


class PhaseTimers:
    """Device-timed named phases of a step.

        timers = PhaseTimers()
        with timers.phase("forward"): loss = model(x, y)
        with timers.phase("backward"): loss.backward()
        with timers.phase("optimizer"): opt.step()
        ms = timers.collect()      # {"forward": .., "backward": .., "optimizer": ..}, max over ranks; resets

    A phase may be entered several times per step (gradient accumulation): its intervals are summed.
    """

    def __init__(self, enabled=None, device_type=None):
        self.enabled = _env_on("NANOCHAT_TRACE") if enabled is None else bool(enabled)
        if device_type is None:
            device_type = "cuda" if torch.cuda.is_available() else "cpu"
        self.cuda = device_type == "cuda"
        self.nvtx = nvtx_enabled() and self.cuda
        self._intervals = {}

    def phase(self, name):
        if not self.enabled:
            return _nvtx_range(name) if (self.nvtx) else _NULL
        return _Phase(self, name)

    def collect(self, reduce=True):
        """Milliseconds per phase since the last collect (max over ranks when a process group is up and
        `reduce`), in first-entered order. Empty when disabled."""
        if not self.enabled or not self._intervals:
            self._intervals = {}
            return {}
        names = list(self._intervals)
        if self.cuda:
            for iv in self._intervals.values():
                iv[-1][1].synchronize()          # the last event of each phase; earlier ones precede it in the stream
            ms = [sum(s.elapsed_time(e) for s, e in self._intervals[n]) for n in names]
        else:
            ms = [sum((e - s) * 1e3 for s, e in self._intervals[n]) for n in names]
        self._intervals = {}
        if reduce and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            # ranks enter the same phases in the same order (same program); reduce on the backend's device
            dev = "cuda" if (self.cuda and dist.get_backend() == "nccl") else "cpu"
            t = torch.tensor(ms, dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.tolist()
        return dict(zip(names, ms))


class MetricsLog:
    """JSONL metrics file with wandb's logging surface. `path=None` keeps it inert (non-master ranks)."""

    def __init__(self, path=None, forward_to=None, header=None):
        self.path, self.forward_to, self._f = path, forward_to, None
        if path is not None:
            os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
            self._f = open(path, "a", encoding="utf-8")
            if header is not None:
                self.log({"event": "run_start", **header})

    @staticmethod
    def _plain(v):
        if isinstance(v, torch.Tensor):
            return v.item() if v.numel() == 1 else v.tolist()
        if isinstance(v, dict):
            return {str(k): MetricsLog._plain(x) for k, x in v.items()}
        if isinstance(v, (list, tuple)):
            return [MetricsLog._plain(x) for x in v]
        if isinstance(v, (str, int, float, bool)) or v is None:
            return v
        try:
            return float(v)
        except (TypeError, ValueError):
            return str(v)

    def log(self, data, *args, **kwargs):
        if self.forward_to is not None and "event" not in data:
            self.forward_to.log(data, *args, **kwargs)
        if self._f is not None:
            rec = {"time": round(time.time(), 3)}
            rec.update(self._plain(data))
            self._f.write(json.dumps(rec, allow_nan=True) + "\n")
            self._f.flush()

    def finish(self):
        if self.forward_to is not None:
            self.forward_to.finish()
        if self._f is not None:
            self._f.close()
            self._f = None


def read_metrics(path):
    """The records of a metrics file; a torn last line (a run killed mid-write) is dropped."""
    out = []
    with open(path, encoding="utf-8") as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            try:
                out.append(json.loads(line))
            except json.JSONDecodeError:
                break
    return out
