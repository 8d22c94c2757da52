"""Multi-GPU worker (one process per GPU, NCCL): fused peer-to-peer optimizer step vs the NCCL path."""
import os
import sys
import json

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from nanochat_b200 import common                                     # noqa: E402
from nanochat_b200.models.gpt import GPT, GPTConfig                  # noqa: E402
from nanochat_b200.train import TrainStep                            # noqa: E402


def build(device):
    cfg = GPTConfig(sequence_len=256, vocab_size=2048, n_layer=4, n_head=2, n_kv_head=2, n_embd=256)
    torch.manual_seed(42)
    with torch.device("meta"):
        m = GPT(cfg)
    m.to_empty(device=device)
    m.init_weights()
    with torch.no_grad():
        for blk in m.transformer.h:
            blk.attn.c_proj.weight.normal_(0, 0.02)
            blk.mlp.c_proj.weight.normal_(0, 0.02)
        m.lm_head.weight.normal_(0, 0.05)
    return m, cfg


def main():
    out_path = sys.argv[1]
    _, rank, _, world, device = common.compute_init("cuda", timeout_s=120)
    from nanochat_b200 import ops
    from nanochat_b200.parallel.symm import SymmComm
    nat = ops.native_module()
    fused_model, cfg = build(device)
    nccl_model, _ = build(device)
    comm = SymmComm.create(fused_model)
    a = TrainStep(fused_model, grad_accum=2, comm=comm, weight_decay=0.1)
    b = TrainStep(nccl_model, grad_accum=2, weight_decay=0.1)      # default comm: torch.distributed (NCCL)
    gen = torch.Generator(device="cpu").manual_seed(100 + rank)
    losses, history = [], []
    for step in range(3):
        data = [(torch.randint(0, cfg.vocab_size, (2, 256), generator=gen).to(device),
                 torch.randint(0, cfg.vocab_size, (2, 256), generator=gen).to(device)) for _ in range(2)]
        history.append(data)
        la = a.step(lambda i: data[i])
        lb = b.step(lambda i: data[i])
        losses.append((la.item(), lb.item()))
    nat.check_status()
    comm.sync_masters()
    torch.cuda.synchronize()
    # oracle: the PyTorch reference bodies with NCCL collectives on the same data
    ops.set_kernel_mode("torch")
    oracle, _ = build(device)
    c = TrainStep(oracle, grad_accum=2, weight_decay=0.1, use_arena=False)
    for data in history:
        c.step(lambda i: data[i])
    ops.set_kernel_mode("native")

    def compare(model):
        bad = {}
        for (n, p), (_, q) in zip(model.named_parameters(), oracle.named_parameters()):
            d = (p.float() - q.float()).abs()
            tol = 3e-2 * q.float().abs().mean().item() + 2e-3
            frac = (d > tol).float().mean().item()
            if frac > 5e-3:
                bad[n] = (round(d.max().item(), 4), round(frac, 4))
        return dict(sorted(bad.items(), key=lambda kv: -kv[1][1])[:6])
    bad_fused, bad_nccl = compare(fused_model), compare(nccl_model)
    oracle_params = dict(oracle.named_parameters())
    shadow_err = 0.0
    for g in comm.arena.muon_groups:
        if g["shadow"] is None:
            continue
        names = [n for n, p in fused_model.named_parameters() if any(p is gp for gp in g["params"])]
        ref = torch.stack([oracle_params[n] for n in names]).float()
        shadow_err = max(shadow_err, ((g["shadow"].float() - ref).norm() / ref.norm()).item())
    for d in comm.arena.adamw_big:
        if d["shadow"] is not None:
            name = next(n for n, p in fused_model.named_parameters() if p is d["param"])
            ref = oracle_params[name].float()
            shadow_err = max(shadow_err, ((d["shadow"].float() - ref).norm() / ref.norm()).item())
    gathered = [None] * world
    dist.all_gather_object(gathered, {"rank": rank, "losses": losses, "shadow_err": shadow_err,
                                      "bad": bad_fused, "bad_nccl": bad_nccl})
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(gathered, f)
    dist.barrier()
    common.compute_cleanup()


if __name__ == "__main__":
    main()
