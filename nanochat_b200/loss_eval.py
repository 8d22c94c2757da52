"""
Bits per byte: a tokenizer-independent validation loss.

bpb = sum(nats of targets whose token has bytes > 0) / (ln 2 * sum(bytes of those targets)).
Special tokens carry 0 bytes in `token_bytes` and are skipped; targets < 0 (ignore_index) are
skipped without ever indexing `token_bytes` with them; sums are added across ranks; the result
is inf when no byte was counted (reference: nanochat/loss_eval.py:9-65).
"""

import math

import torch
import torch.distributed as dist


@torch.no_grad()
def evaluate_bpb(model, batches, steps, token_bytes):
    device = model.get_device()
    nats = torch.zeros((), dtype=torch.float32, device=device)
    nbytes = torch.zeros((), dtype=torch.int64, device=device)
    it = iter(batches)
    for _ in range(steps):
        x, y = next(it)
        loss = model(x, y, loss_reduction="none").view(-1)
        y = y.view(-1)
        valid = y >= 0
        per_tok = torch.where(valid, token_bytes[y.clamp_min(0)], torch.zeros_like(y, dtype=token_bytes.dtype))
        nats += (loss * (per_tok > 0)).sum()
        nbytes += per_tok.sum()
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(nats, op=dist.ReduceOp.SUM)
        dist.all_reduce(nbytes, op=dist.ReduceOp.SUM)
    total_bytes = nbytes.item()
    if total_bytes == 0:
        return float("inf")
    return nats.item() / (math.log(2) * total_bytes)


@torch.no_grad()
def evaluate_mean_loss(model, batches, steps):
    """Mean cross entropy per target token over `steps` batches of every rank (nats). The loaders' third item
    (their state), if present, is ignored."""
    device = model.get_device()
    total = torch.zeros((), dtype=torch.float64, device=device)
    count = torch.zeros((), dtype=torch.float64, device=device)
    it = iter(batches)
    for _ in range(steps):
        x, y = next(it)[:2]
        loss = model(x, y, loss_reduction="none").view(-1)
        valid = y.view(-1) >= 0
        total += (loss.double() * valid).sum()
        count += valid.sum()
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(total, op=dist.ReduceOp.SUM)
        dist.all_reduce(count, op=dist.ReduceOp.SUM)
    return (total / count.clamp_min(1)).item()
