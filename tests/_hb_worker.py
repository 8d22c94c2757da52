"""Worker of tests/test_heartbeat.py: gloo ranks with a store heartbeat; one rank is killed or leaves."""
import json
import os
import signal
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from nanochat_b200.parallel.heartbeat import Heartbeat, RankLostError, default_store  # noqa: E402


def main():
    mode, out_dir = sys.argv[1], sys.argv[2]
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    hb = Heartbeat(default_store(), rank, world, interval=0.2, timeout=3.0)
    hb.wait_for_peers()
    victim = world - 1
    outcome = {"rank": rank, "steps": 0}
    t_lost = None
    try:
        for step in range(200):
            hb.check()                                   # before the step's collective
            if step == 3 and rank == victim:
                if mode == "kill":
                    os.kill(os.getpid(), signal.SIGKILL)  # dies between steps, nothing in flight
                hb.leave()                               # mode "leave": an orderly exit
                outcome["outcome"] = "left"
                break
            if step >= 3:
                if t_lost is None:
                    t_lost = time.monotonic()
                if mode == "leave" and victim in hb.departed():
                    outcome["outcome"] = "peer left"
                    break
                time.sleep(0.1)                          # survivors: host-side work only from here on
                continue
            t = torch.ones(4) * (rank + 1)
            dist.all_reduce(t)
            outcome["steps"] = step + 1
        else:
            outcome["outcome"] = "never noticed"
    except RankLostError as e:
        outcome["outcome"] = "error: " + str(e)
        outcome["lost"] = e.ranks
        outcome["seconds"] = time.monotonic() - t_lost if t_lost is not None else None
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump(outcome, f)
    hb.stop()
    os._exit(0)          # no destroy_process_group: it would wait for the rank that is gone


if __name__ == "__main__":
    main()
