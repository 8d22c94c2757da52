"""
CPU correctness configuration: tiny GPT d4 (4 layers, 256 wide, 2 heads x 128, vocabulary 32768, sequence 512,
global batch 8) in fp32 with Muon + AdamW for 20 steps on uniform-random token ids from a seed; prints the loss
trajectory as one JSON line.

    python baseline/config1_cpu.py --impl ours                       # one process
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 \
        baseline/config1_cpu.py --impl ours                          # two gloo ranks, 4 rows each
    python baseline/config1_cpu.py --impl reference                  # the reference's own code from baseline/_ref, eager

Every step draws one (8, 512) batch from the generator; with two ranks each takes its half of the rows, so the two
runs optimise the same objective. The reference creates no process group on CPU; its one-process run is the
comparison for both.
"""
import argparse
import json
import os
import sys

if "reference" in sys.argv:
    # the reference wraps its optimizer steps in torch.compile; "eager" means the same Python bodies, uncompiled
    os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--steps", type=int, default=20)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        from nanochat.gpt import GPT, GPTConfig
        assert world == 1
    else:
        sys.path.insert(0, ROOT)
        from nanochat_b200 import common
        from nanochat_b200.models.gpt import GPT, GPTConfig
        common.compute_init("cpu")
    torch.manual_seed(42)
    cfg = GPTConfig(sequence_len=512, vocab_size=32768, n_layer=4, n_head=2, n_kv_head=2, n_embd=256)
    with torch.device("meta"):
        model = GPT(cfg)
    model.to_empty(device="cpu")
    model.init_weights()
    opt = model.setup_optimizer(weight_decay=0.1)
    gen = torch.Generator().manual_seed(1234)
    rows = 8 // world
    losses = []
    for _ in range(args.steps):
        batch = torch.randint(0, cfg.vocab_size, (8, 513), generator=gen)
        mine = batch[rank * rows:(rank + 1) * rows]
        loss = model(mine[:, :-1].contiguous(), mine[:, 1:].contiguous())
        loss.backward()
        opt.step()
        model.zero_grad(set_to_none=True)
        if world > 1:
            import torch.distributed as dist
            t = loss.detach().clone()
            dist.all_reduce(t)
            losses.append((t / world).item())
        else:
            losses.append(loss.item())
    if rank == 0:
        print(json.dumps({"impl": args.impl, "world_size": world, "dtype": "fp32", "steps": args.steps,
                          "losses": [round(v, 6) for v in losses]}))
    if args.impl == "ours":
        from nanochat_b200 import common
        common.compute_cleanup()


if __name__ == "__main__":
    main()
