"""
CPU tests of the observability tools: phase timers (single process and max-over-ranks under gloo), the JSONL
metrics file, and that the default training step records nothing.
"""
import json
import os
import subprocess
import sys
import time

import torch

from nanochat_b200.utils import trace

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_disabled_timers_are_inert(monkeypatch):
    monkeypatch.delenv("NANOCHAT_TRACE", raising=False)
    monkeypatch.delenv("NANOCHAT_NVTX", raising=False)
    t = trace.PhaseTimers()
    assert not t.enabled
    with t.phase("forward"):
        pass
    assert t.collect() == {} and t._intervals == {}
    with trace.nvtx("anything"):           # a no-op without NANOCHAT_NVTX=1 (and without CUDA)
        pass


def test_phase_intervals_are_summed_and_reset():
    t = trace.PhaseTimers(enabled=True, device_type="cpu")
    for _ in range(3):                      # three micro-steps
        with t.phase("forward"):
            time.sleep(0.01)
        with t.phase("backward"):
            time.sleep(0.02)
    with t.phase("optimizer"):
        time.sleep(0.005)
    ms = t.collect()
    assert list(ms) == ["forward", "backward", "optimizer"]
    assert 25 <= ms["forward"] < 5000 and 55 <= ms["backward"] < 5000 and 4 <= ms["optimizer"] < 5000
    assert ms["backward"] > 0 and ms["forward"] > 0
    assert t.collect() == {}                # collect resets


def test_env_switch_enables_timers(monkeypatch):
    monkeypatch.setenv("NANOCHAT_TRACE", "1")
    assert trace.PhaseTimers(device_type="cpu").enabled
    monkeypatch.setenv("NANOCHAT_TRACE", "0")
    assert not trace.PhaseTimers(device_type="cpu").enabled


def test_train_step_reports_phases_when_asked():
    from nanochat_b200.models.gpt import GPT, GPTConfig
    from nanochat_b200.train import TrainStep
    torch.manual_seed(0)
    cfg = GPTConfig(sequence_len=32, vocab_size=64, n_layer=2, n_head=2, n_kv_head=2, n_embd=32, window_pattern="L")
    model = GPT(cfg)
    model.init_weights()
    timers = trace.PhaseTimers(enabled=True, device_type="cpu")
    step = TrainStep(model, grad_accum=2, timers=timers)
    x = torch.randint(0, 64, (2, 32))
    loss = step.step(lambda i: (x, x))
    assert torch.isfinite(loss)
    ms = timers.collect()
    assert list(ms) == ["forward", "backward", "optimizer"] and all(v > 0 for v in ms.values())
    assert len(ms) == 3


def test_metrics_file_round_trip_and_torn_tail(tmp_path):
    class Sink:
        def __init__(self):
            self.got, self.done = [], False

        def log(self, data):
            self.got.append(data)

        def finish(self):
            self.done = True

    sink = Sink()
    path = str(tmp_path / "m" / "run.jsonl")
    log = trace.MetricsLog(path, forward_to=sink, header={"script": "t", "config": {"depth": 4}})
    log.log({"step": 0, "train/loss": torch.tensor(2.5), "vec": torch.arange(3), "obj": object})
    log.log({"step": 1, "train/loss": float("nan")})
    log.finish()
    assert sink.done and [d["step"] for d in sink.got] == [0, 1]       # the header is not forwarded
    with open(path, "a") as f:
        f.write('{"step": 2, "train/lo')                               # a run killed in mid-write
    recs = trace.read_metrics(path)
    assert [r.get("event") for r in recs] == ["run_start", None, None]
    assert recs[0]["config"] == {"depth": 4} and recs[1]["train/loss"] == 2.5 and recs[1]["vec"] == [0, 1, 2]
    assert recs[2]["train/loss"] != recs[2]["train/loss"]              # NaN survives
    assert all("time" in r for r in recs)
    inert = trace.MetricsLog(None)                                     # non-master ranks
    inert.log({"step": 3})
    inert.finish()


_WORKER = r"""
import os, sys, time
import torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from nanochat_b200.utils.trace import PhaseTimers
dist.init_process_group("gloo")
rank = dist.get_rank()
t = PhaseTimers(enabled=True, device_type="cpu")
with t.phase("forward"):
    time.sleep(0.15 if rank == 1 else 0.01)      # rank 1 is the slow one here
with t.phase("optimizer"):
    time.sleep(0.15 if rank == 0 else 0.01)      # rank 0 there
ms = t.collect()
assert ms["forward"] >= 140 and ms["optimizer"] >= 140, (rank, ms)
local = PhaseTimers(enabled=True, device_type="cpu")
with local.phase("forward"):
    time.sleep(0.01)
assert local.collect(reduce=False)["forward"] < 140
dist.destroy_process_group()
print("ok", rank)
"""


def test_phases_reduce_as_max_over_ranks(tmp_path):
    script = tmp_path / "w.py"
    script.write_text(_WORKER)
    import socket
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script), REPO], env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=120)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    json.dumps(outs)
