"""
Depth-derived hyper-parameters and schedules of the pretraining / finetuning drivers.

Everything follows from `--depth` (reference: scripts/base_train.py:129-143,249-304,360-386):
  width      dim = ceil(depth * aspect_ratio / head_dim) * head_dim, heads = dim / head_dim
  horizon    target_tokens = ratio * (transformer matrices + lm_head parameters)
  batch      B = 2^round(log2(B_ref * (target_tokens / D_ref)^0.383)),  B_ref = 2^19 at d12
  lr scale   sqrt(B / B_ref) on every learning rate
  wd         wd_ref * sqrt(B / B_ref) * (D_ref / target_tokens)
"""

import math
from dataclasses import dataclass

B_REF = 2 ** 19


def model_dims(depth, aspect_ratio=64, head_dim=128):
    dim = -(-depth * aspect_ratio // head_dim) * head_dim
    return dim, dim // head_dim


def scaling_param_count(model):
    counts = model.num_scaling_params()
    return counts["transformer_matrices"] + counts["lm_head"]


@dataclass
class DerivedHParams:
    target_tokens: int
    d_ref: float
    total_batch_size: int
    batch_lr_scale: float
    weight_decay: float


def derive_hparams(scaling_params, ref_scaling_params, ratio, weight_decay, total_batch_size=-1):
    target_tokens = int(ratio * scaling_params)
    d_ref = ratio * ref_scaling_params
    if total_batch_size == -1:
        predicted = B_REF * (target_tokens / d_ref) ** 0.383
        total_batch_size = 2 ** round(math.log2(predicted))
    batch_ratio = total_batch_size / B_REF
    lr_scale = batch_ratio ** 0.5 if batch_ratio != 1.0 else 1.0
    wd = weight_decay * math.sqrt(total_batch_size / B_REF) * (d_ref / target_tokens)
    return DerivedHParams(target_tokens, d_ref, total_batch_size, lr_scale, wd)


def pretrain_lr_multiplier(it, num_iterations, warmup_steps=40, warmdown_ratio=0.65, final_lr_frac=0.05):
    """Linear warm-up over `warmup_steps`, flat, linear warm-down over the last `warmdown_ratio` to `final_lr_frac`."""
    warmdown_iters = round(warmdown_ratio * num_iterations)
    if it < warmup_steps:
        return (it + 1) / warmup_steps
    if it <= num_iterations - warmdown_iters:
        return 1.0
    progress = (num_iterations - it) / warmdown_iters
    return progress + (1 - progress) * final_lr_frac


def pretrain_muon_momentum(it, num_iterations, warmdown_ratio=0.65):
    """0.85 -> 0.97 over 400 steps, 0.97 -> 0.90 across the LR warm-down."""
    warmdown_iters = round(warmdown_ratio * num_iterations)
    start = num_iterations - warmdown_iters
    if it < 400:
        f = it / 400
        return (1 - f) * 0.85 + f * 0.97
    if it >= start:
        p = (it - start) / warmdown_iters
        return 0.97 * (1 - p) + 0.90 * p
    return 0.97


def pretrain_weight_decay(it, num_iterations, wd0):
    return wd0 * 0.5 * (1 + math.cos(math.pi * it / num_iterations))


def sft_lr_multiplier(progress, warmup_ratio=0.0, warmdown_ratio=0.5, final_lr_frac=0.0):
    """Same shape as pretraining but over progress in [0,1] (reference: scripts/chat_sft.py:307-315)."""
    if progress < warmup_ratio:
        return (progress + 1e-8) / warmup_ratio
    if progress <= 1.0 - warmdown_ratio:
        return 1.0
    decay = (progress - (1.0 - warmdown_ratio)) / warmdown_ratio
    return (1 - decay) + decay * final_lr_frac


def sft_muon_momentum(it):
    f = min(it / 300, 1)
    return (1 - f) * 0.85 + f * 0.95
