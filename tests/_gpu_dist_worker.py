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


# argv[2] (optional) = "layers,width": the default is a 4-layer 256-wide model; "26,128" has the Muon groups of the
# 26-layer flagship (104 / 26 / 26 matrices: uneven ownership, the last ranks own fewer or none) at toy width
LAYERS, WIDTH = (int(v) for v in (sys.argv[2] if len(sys.argv) > 2 else "4,256").split(","))


def build(device):
    cfg = GPTConfig(sequence_len=256, vocab_size=2048, n_layer=LAYERS, n_head=WIDTH // 128, n_kv_head=WIDTH // 128,
                    n_embd=WIDTH)
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
    # Small learning rates keep three steps in the regime where two implementations that differ by
    # rounding stay comparable element by element (at the training rates a +-lr sign flip of a
    # near-zero gradient is amplified by the following steps).
    hp = dict(weight_decay=0.1, embedding_lr=2e-3, unembedding_lr=4e-4, matrix_lr=2e-3, scalar_lr=5e-3)
    initial = {n: p.detach().float().clone() for n, p in fused_model.named_parameters()}
    a = TrainStep(fused_model, grad_accum=2, comm=comm, **hp)
    b = TrainStep(nccl_model, grad_accum=2, **hp)      # default comm: torch.distributed (NCCL)
    gen = torch.Generator(device="cpu").manual_seed(100 + rank)
    losses, history = [], []
    for step in range(3):
        data = [(torch.randint(0, cfg.vocab_size, (2, 256), generator=gen).to(device),
                 torch.randint(0, cfg.vocab_size, (2, 256), generator=gen).to(device)) for _ in range(2)]
        history.append(data)
        la = a.step(lambda i: data[i])
        lb = b.step(lambda i: data[i])
        losses.append((la.item(), lb.item()))
        if step == 0:
            # Sharp check of the scalars' gradient plumbing: both paths start from the same weights and data, so their
            # first Adam step (-lr * g / (|g| + eps)) may differ only where a gradient component is ~0.
            first_step_bad = {}
            for (n, p), (_, q) in zip(fused_model.named_parameters(), nccl_model.named_parameters()):
                if p.numel() < 64:
                    dp, dq = p.float() - initial[n], q.float() - initial[n]
                    frac = ((dp - dq).abs() > 0.05 * dq.abs() + 1e-7).float().mean().item()
                    if frac > 0.1 and p.numel() > 1 or frac > 0 and p.numel() == 1:
                        first_step_bad[n] = (round(frac, 4), dp.flatten()[:4].tolist(), dq.flatten()[:4].tolist())
    nat.check_status()
    comm.sync_masters()
    torch.cuda.synchronize()
    # oracle: the PyTorch reference bodies with NCCL collectives on the same data
    ops.set_kernel_mode("torch")
    oracle, _ = build(device)
    c = TrainStep(oracle, grad_accum=2, use_arena=False, **hp)
    for data in history:
        c.step(lambda i: data[i])
    ops.set_kernel_mode("native")

    def compare(model, other, rel, min_numel, truth=None):
        """Parameters whose update (value - initial value) disagrees with `other` on more than 2% of
        the elements; an element disagrees when it is off by more than rel x the mean |update|.
        Tensors under 64 elements (per-layer scalars) are judged against `truth` instead: their gradients are sums
        with heavy cancellation, an Adam step moves a parameter by about +-lr whatever the gradient's size, and after
        the first step (checked exactly above) any two implementations drift apart by whole steps. There an element
        disagrees when `model` is more than twice as far from `truth` as `other` is."""
        bad = {}
        truth_params = dict(truth.named_parameters()) if truth is not None else None
        for (n, p), (_, q) in zip(model.named_parameters(), other.named_parameters()):
            if p.numel() < min_numel:
                continue
            dp, dq = p.float() - initial[n], q.float() - initial[n]
            tol = rel * dq.abs().mean().item() + 1e-7
            if p.numel() < 64 and truth_params is not None:
                dt = truth_params[n].float() - initial[n]
                frac = ((dp - dt).abs() > 2 * (dq - dt).abs() + tol).float().mean().item()
                limit = 0.35 if p.numel() > 1 else 0.0
            else:
                frac = ((dp - dq).abs() > tol).float().mean().item()
                limit = 2e-2
            if frac > limit:
                bad[n] = (round((dp - dq).abs().max().item(), 5), round(frac, 4), round(dq.abs().mean().item(), 5))
        return dict(sorted(bad.items(), key=lambda kv: -kv[1][1])[:8])
    # same kernels, different collectives: only the summation order differs
    bad_pair = compare(fused_model, nccl_model, 0.25, 1, truth=oracle)
    bad_pair.update({f"first step: {n}": v for n, v in first_step_bad.items()})
    # against the PyTorch bodies: bf16 rounding differs everywhere, scalars (sums with heavy
    # cancellation) are left to the pairwise check
    bad_fused = compare(fused_model, oracle, 0.5, 64)
    bad_nccl = compare(nccl_model, oracle, 0.5, 64)
    oracle_params = dict(oracle.named_parameters())
    shadow_err = 0.0
    for g in comm.arena.muon_groups:
        if g["shadow"] is None or g["shape"][0] % 8 or g["shape"][1] % 8:
            continue        # the tiny value-embedding gate matrices are consumed from their fp32 masters
        name_of = {id(p): n for n, p in fused_model.named_parameters()}
        names = [name_of[id(gp)] for gp in g["params"]]          # the stack follows the group's order
        ref = torch.stack([oracle_params[n] for n in names]).float()
        shadow_err = max(shadow_err, ((g["shadow"].float() - ref).norm() / ref.norm()).item())
    for d in comm.arena.adamw_big:
        if d["shadow"] is not None:
            name = next(n for n, p in fused_model.named_parameters() if p is d["param"])
            ref = oracle_params[name].float()
            shadow_err = max(shadow_err, ((d["shadow"].float() - ref).norm() / ref.norm()).item())
    # the per-layer scalars' updates on all three paths, for inspection when the pairwise check complains
    scalars = {}
    for (n, p), (_, q), (_, o) in zip(fused_model.named_parameters(), nccl_model.named_parameters(),
                                      oracle.named_parameters()):
        if p.numel() < 64:
            scalars[n] = [[round(v, 6) for v in (t.float() - initial[n]).flatten().tolist()] for t in (p, q, o)]
    gathered = [None] * world
    dist.all_gather_object(gathered, {"rank": rank, "losses": losses, "shadow_err": shadow_err, "scalars": scalars,
                                      "bad": bad_fused, "bad_nccl": bad_nccl, "bad_pair": bad_pair})
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(gathered, f)
    dist.barrier()
    common.compute_cleanup()


if __name__ == "__main__":
    main()
