"""Worker for the multi-process CPU tests (launched by torch.distributed.run with the gloo backend)."""
import os
import sys
import json

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from nanochat_b200 import common                                     # noqa: E402
from nanochat_b200.models.gpt import GPT, GPTConfig                  # noqa: E402


def build():
    cfg = GPTConfig(sequence_len=64, vocab_size=512, n_layer=4, n_head=2, n_kv_head=2, n_embd=256)
    torch.manual_seed(42)
    model = GPT(cfg)
    model.init_weights()
    with torch.no_grad():
        for blk in model.transformer.h:
            blk.attn.c_proj.weight.normal_(0, 0.02)
            blk.mlp.c_proj.weight.normal_(0, 0.02)
    return model, cfg


def batch(cfg, step, shard):
    g = torch.Generator().manual_seed(1000 * step + shard)
    return (torch.randint(0, cfg.vocab_size, (2, 64), generator=g),
            torch.randint(0, cfg.vocab_size, (2, 64), generator=g))


def main():
    mode, out_path = sys.argv[1], sys.argv[2]
    steps = 3
    if mode == "train":
        _, rank, _, world, _ = common.compute_init("cpu", timeout_s=120)
        model, cfg = build()
        opt = model.setup_optimizer(weight_decay=0.1)
        losses = []
        for s in range(steps):
            x, y = batch(cfg, s, rank)
            loss = model(x, y)
            loss.backward()
            opt.step()
            model.zero_grad(set_to_none=True)
            losses.append(loss.item())
        if rank == 0:
            torch.save({"params": {k: v.clone() for k, v in model.state_dict().items()}, "losses": losses,
                        "world": world, "state_keys": sorted(opt.state_dict()["state"].keys())}, out_path)
        common.compute_cleanup()
    elif mode == "fail":
        # rank 1 dies between steps; rank 0 must get an error from its next collective, not hang
        import torch.distributed as dist
        _, rank, _, world, _ = common.compute_init("cpu", timeout_s=8)
        if rank == 1:
            os._exit(17)
        t = torch.ones(4)
        try:
            dist.all_reduce(t)
            outcome = "completed"
        except Exception as e:
            outcome = f"error:{type(e).__name__}"
        with open(out_path, "w") as f:
            json.dump({"outcome": outcome}, f)
        os._exit(0)


if __name__ == "__main__":
    main()
