"""
Checkpoint files and directory conventions.

On-disk layout is the reference's, byte-compatible in both directions
(reference: nanochat/checkpoint_manager.py:41-73,117-193):

    <base>/{base,chatsft,chatrl}_checkpoints/<tag>/model_%06d.pt        state_dict (rank 0)
                                                   meta_%06d.json       indent=2 (rank 0)
                                                   optim_%06d_rank%d.pt optimizer.state_dict() (every rank)

Parameters that live as views inside fused buffers (parallel/arena.py) are saved
as ordinary per-parameter tensors because `state_dict()` walks the parameters,
and are re-packed after a load.

Robustness added on top of the reference behaviour: files are written to a
temporary name and renamed, and a truncated or unreadable checkpoint raises a
`CheckpointError` naming the file instead of surfacing a pickle error.
"""

import os
import re
import json
import logging

import torch

from nanochat_b200.common import get_base_dir, setup_default_logging

setup_default_logging()
logger = logging.getLogger(__name__)


class CheckpointError(RuntimeError):
    pass


def log0(message):
    if int(os.environ.get("RANK", 0)) == 0:
        logger.info(message)


def _patch_missing_config_keys(cfg):
    """Checkpoints older than sliding windows were trained with full context."""
    if "window_pattern" not in cfg:
        cfg["window_pattern"] = "L"
        log0("Patching missing window_pattern in model config to 'L'")


def _patch_missing_keys(model_data, model_config):
    """Old checkpoints lack the per-layer scalars: neutral values reproduce their function."""
    L = model_config.n_layer
    if "resid_lambdas" not in model_data:
        model_data["resid_lambdas"] = torch.ones(L)
        log0("Patching missing resid_lambdas in model data to 1.0")
    if "x0_lambdas" not in model_data:
        model_data["x0_lambdas"] = torch.zeros(L)
        log0("Patching missing x0_lambdas in model data to 0.0")


def _atomic_torch_save(obj, path):
    tmp = path + ".tmp"
    torch.save(obj, tmp)
    os.replace(tmp, path)


def _safe_torch_load(path, device):
    if not os.path.exists(path):
        raise CheckpointError(f"checkpoint file missing: {path}")
    try:
        return torch.load(path, map_location=device)
    except Exception as e:
        raise CheckpointError(f"checkpoint file unreadable (truncated or corrupt): {path}: {e}") from e


def save_checkpoint(checkpoint_dir, step, model_data, optimizer_data, meta_data, rank=0):
    if rank == 0:
        os.makedirs(checkpoint_dir, exist_ok=True)
        model_path = os.path.join(checkpoint_dir, f"model_{step:06d}.pt")
        _atomic_torch_save(model_data, model_path)
        logger.info(f"Saved model parameters to: {model_path}")
        meta_path = os.path.join(checkpoint_dir, f"meta_{step:06d}.json")
        with open(meta_path + ".tmp", "w", encoding="utf-8") as f:
            json.dump(meta_data, f, indent=2)
        os.replace(meta_path + ".tmp", meta_path)
        logger.info(f"Saved metadata to: {meta_path}")
    if optimizer_data is not None:
        os.makedirs(checkpoint_dir, exist_ok=True)
        optim_path = os.path.join(checkpoint_dir, f"optim_{step:06d}_rank{rank:d}.pt")
        _atomic_torch_save(optimizer_data, optim_path)
        logger.info(f"Saved optimizer state to: {optim_path}")


def load_checkpoint(checkpoint_dir, step, device, load_optimizer=False, rank=0):
    model_data = _safe_torch_load(os.path.join(checkpoint_dir, f"model_{step:06d}.pt"), device)
    optimizer_data = None
    if load_optimizer:
        optimizer_data = _safe_torch_load(os.path.join(checkpoint_dir, f"optim_{step:06d}_rank{rank:d}.pt"), device)
    meta_path = os.path.join(checkpoint_dir, f"meta_{step:06d}.json")
    if not os.path.exists(meta_path):
        raise CheckpointError(f"checkpoint file missing: {meta_path}")
    with open(meta_path, "r", encoding="utf-8") as f:
        meta_data = json.load(f)
    return model_data, optimizer_data, meta_data


def build_model(checkpoint_dir, step, device, phase):
    """(model, tokenizer, meta) from a checkpoint; the model is plain (no wrappers)."""
    from nanochat_b200.models.gpt import GPT, GPTConfig
    from nanochat_b200.tokenizer import get_tokenizer
    assert phase in ("train", "eval"), f"Invalid phase: {phase}"
    if not isinstance(device, torch.device):
        device = torch.device(device)
    model_data, _, meta_data = load_checkpoint(checkpoint_dir, step, device, load_optimizer=False)
    if device.type in ("cpu", "mps"):
        model_data = {k: (v.float() if v.dtype == torch.bfloat16 else v) for k, v in model_data.items()}
    model_data = {k.removeprefix("_orig_mod."): v for k, v in model_data.items()}
    cfg_kwargs = meta_data["model_config"]
    _patch_missing_config_keys(cfg_kwargs)
    log0(f"Building model with config: {cfg_kwargs}")
    config = GPTConfig(**cfg_kwargs)
    _patch_missing_keys(model_data, config)
    with torch.device("meta"):
        model = GPT(config)
    model.to_empty(device=device)
    model.init_weights()  # builds the rotary tables; parameter values are overwritten next
    model.load_state_dict(model_data, strict=True, assign=True)
    model.eval() if phase == "eval" else model.train()
    tokenizer = get_tokenizer()
    assert tokenizer.get_vocab_size() == cfg_kwargs["vocab_size"], (
        f"Tokenizer vocab size {tokenizer.get_vocab_size()} does not match model config vocab size {cfg_kwargs['vocab_size']}")
    return model, tokenizer, meta_data


def find_largest_model(checkpoints_dir):
    """Guess the model tag: the deepest d<N>, else the most recently touched directory."""
    tags = [f for f in os.listdir(checkpoints_dir) if os.path.isdir(os.path.join(checkpoints_dir, f))]
    if not tags:
        raise FileNotFoundError(f"No checkpoints found in {checkpoints_dir}")
    depth_tags = []
    for t in tags:
        m = re.match(r"d(\d+)", t)
        if m:
            depth_tags.append((int(m.group(1)), t))
    if depth_tags:
        return max(depth_tags)[1]
    return max(tags, key=lambda t: os.path.getmtime(os.path.join(checkpoints_dir, t)))


def find_last_step(checkpoint_dir):
    steps = [int(m.group(1)) for f in os.listdir(checkpoint_dir) if (m := re.search(r"model_(\d+)\.pt$", f))]
    if not steps:
        raise FileNotFoundError(f"No checkpoints found in {checkpoint_dir}")
    return max(steps)


_SOURCE_DIRS = {"base": "base_checkpoints", "sft": "chatsft_checkpoints", "rl": "chatrl_checkpoints"}


def load_model_from_dir(checkpoints_dir, device, phase, model_tag=None, step=None):
    if model_tag is None:
        model_tag = find_largest_model(checkpoints_dir)
        log0(f"No model tag provided, guessing model tag: {model_tag}")
    checkpoint_dir = os.path.join(checkpoints_dir, model_tag)
    if step is None:
        step = find_last_step(checkpoint_dir)
    log0(f"Loading model from {checkpoint_dir} with step {step}")
    return build_model(checkpoint_dir, step, device, phase)


def load_model(source, *args, **kwargs):
    checkpoints_dir = os.path.join(get_base_dir(), _SOURCE_DIRS[source])
    return load_model_from_dir(checkpoints_dir, *args, **kwargs)


def optimizer_shard_count(checkpoint_dir, step):
    """How many ranks saved optimizer shards at `step` (the world size of the run that wrote the checkpoint)."""
    prefix = f"optim_{step:06d}_rank"
    return sum(1 for f in os.listdir(checkpoint_dir) if f.startswith(prefix) and f.endswith(".pt"))


def load_optimizer_state(source, device, rank, model_tag=None, step=None, world_size=None):
    """This rank's optimizer shard only, or None when the file does not exist. The state is sharded by rank, so
    shards written by a run of another world size do not fit: with `world_size` given, every rank sees the same
    mismatch in the directory listing and gets None (a fresh optimizer) instead of a shape error on some ranks."""
    checkpoints_dir = os.path.join(get_base_dir(), _SOURCE_DIRS[source])
    if model_tag is None:
        model_tag = find_largest_model(checkpoints_dir)
    checkpoint_dir = os.path.join(checkpoints_dir, model_tag)
    if step is None:
        step = find_last_step(checkpoint_dir)
    path = os.path.join(checkpoint_dir, f"optim_{step:06d}_rank{rank:d}.pt")
    if world_size is not None:
        saved = optimizer_shard_count(checkpoint_dir, step)
        if saved != world_size and saved > 0:
            log0(f"Optimizer checkpoint at {checkpoint_dir} step {step} was written by {saved} rank(s); this run has "
                 f"{world_size}: not loading it")
            return None
    if not os.path.exists(path):
        log0(f"Optimizer checkpoint not found: {path}")
        return None
    log0(f"Loading optimizer state from {path}")
    return _safe_torch_load(path, device)
