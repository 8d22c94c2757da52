"""
Pretrain a base model.

    python -m scripts.base_train --depth 12
    torchrun --nproc_per_node=8 -m scripts.base_train -- --depth 26 --fp8
    # CPU smoke run
    python -m scripts.base_train --depth=4 --max-seq-len=512 --device-batch-size=1 --eval-tokens=512 \
        --core-metric-every=-1 --total-batch-size=512 --num-iterations=20

`--depth` is the only dial: width, heads, token horizon, batch size, learning rates and weight
decay are derived from it (nanochat_b200/schedules.py). Flags, log lines and checkpoint
metadata follow the reference driver (scripts/base_train.py) so its sweep scripts keep working.
Extra flags: --synthetic-data (uniform-random tokens, no corpus/tokenizer needed),
--comm {auto,nccl,fused} (optimizer collectives), --kernels {native,torch}.
"""
import os
os.environ.setdefault("PYTORCH_ALLOC_CONF", "expandable_segments:True")
import gc
import json
import time
import argparse
from dataclasses import asdict
from contextlib import contextmanager

import torch

from nanochat_b200 import common, ops
from nanochat_b200.common import (compute_init, compute_cleanup, print0, DummyWandb, print_banner, get_base_dir,
                                  autodetect_device_type, get_peak_flops)
from nanochat_b200.models.gpt import GPT, GPTConfig
from nanochat_b200 import schedules
from nanochat_b200.checkpoint_manager import (save_checkpoint, load_checkpoint, optimizer_shard_count,
                                               CheckpointError)
from nanochat_b200.loss_eval import evaluate_bpb, evaluate_mean_loss
from nanochat_b200.engine import Engine
from nanochat_b200.utils.trace import MetricsLog, PhaseTimers

print_banner()

parser = argparse.ArgumentParser(description="Pretrain base model")
parser.add_argument("--run", type=str, default="dummy", help="wandb run name ('dummy' disables wandb logging)")
parser.add_argument("--device-type", type=str, default="", help="cuda|cpu (empty = autodetect)")
parser.add_argument("--fp8", action="store_true", help="block-scaled FP8 linear layers")
parser.add_argument("--fp8-recipe", type=str, default="tensorwise", choices=["rowwise", "tensorwise", "mxfp8"])
parser.add_argument("--depth", type=int, default=20)
parser.add_argument("--aspect-ratio", type=int, default=64)
parser.add_argument("--head-dim", type=int, default=128)
parser.add_argument("--max-seq-len", type=int, default=2048)
parser.add_argument("--window-pattern", type=str, default="SSSL")
parser.add_argument("--num-iterations", type=int, default=-1)
parser.add_argument("--target-flops", type=float, default=-1.0)
parser.add_argument("--target-param-data-ratio", type=float, default=12)
parser.add_argument("--device-batch-size", type=int, default=32)
parser.add_argument("--total-batch-size", type=int, default=-1)
parser.add_argument("--embedding-lr", type=float, default=0.3)
parser.add_argument("--unembedding-lr", type=float, default=0.008)
parser.add_argument("--weight-decay", type=float, default=0.28)
parser.add_argument("--matrix-lr", type=float, default=0.02)
parser.add_argument("--scalar-lr", type=float, default=0.5)
parser.add_argument("--warmup-steps", type=int, default=40)
parser.add_argument("--warmdown-ratio", type=float, default=0.65)
parser.add_argument("--final-lr-frac", type=float, default=0.05)
parser.add_argument("--resume-from-step", type=int, default=-1)
parser.add_argument("--eval-every", type=int, default=250)
parser.add_argument("--eval-tokens", type=int, default=80 * 524288)
parser.add_argument("--core-metric-every", type=int, default=2000)
parser.add_argument("--core-metric-max-per-task", type=int, default=500)
parser.add_argument("--sample-every", type=int, default=2000)
parser.add_argument("--save-every", type=int, default=-1)
parser.add_argument("--log-every", type=int, default=100, help="steps between metric records (wandb and the metrics file)")
parser.add_argument("--heartbeat-timeout", type=float, default=0.0,
                    help="seconds without a peer's heartbeat before the run stops with an error (0 = no heartbeat)")
parser.add_argument("--abort-on-divergence", action="store_true",
                    help="stop when the loss is non-finite or stays above 3x its running average")
parser.add_argument("--metrics-file", type=str, default=None,
                    help="JSONL metrics file (default: <base_dir>/metrics/base_train_<model tag>.jsonl; '' disables)")
parser.add_argument("--model-tag", type=str, default=None)
# additions of this framework
parser.add_argument("--synthetic-data", action="store_true", help="uniform-random tokens instead of the corpus")
parser.add_argument("--vocab-size", type=int, default=32768, help="vocabulary size with --synthetic-data")
parser.add_argument("--synthetic-cycle", type=int, default=0,
                    help="with --synthetic-data: repeat the first N batches forever (0 = fresh random batches)")
parser.add_argument("--no-final-save", action="store_true", help="do not write the checkpoint of the last step (timing runs)")
parser.add_argument("--comm", type=str, default="auto", choices=["auto", "nccl", "fused"],
                    help="optimizer collectives: torch.distributed or fused peer-to-peer kernels")
parser.add_argument("--kernels", type=str, default="native", choices=["native", "torch"])
args = parser.parse_args()
user_config = vars(args).copy()

ops.set_kernel_mode(args.kernels)
device_type = autodetect_device_type() if args.device_type == "" else args.device_type
ddp, ddp_rank, ddp_local_rank, ddp_world_size, device = compute_init(device_type)
master_process = ddp_rank == 0
synchronize = torch.cuda.synchronize if device_type == "cuda" else lambda: None
get_max_memory = torch.cuda.max_memory_allocated if device_type == "cuda" else lambda: 0
if device_type == "cuda":
    gpu_name = torch.cuda.get_device_name(0)
    gpu_peak_flops = get_peak_flops(gpu_name)
    print0(f"GPU: {gpu_name} | Peak FLOPS (BF16): {gpu_peak_flops:.2e}")
else:
    gpu_peak_flops = float("inf")
print0(f"COMPUTE_DTYPE: {common.COMPUTE_DTYPE} ({common.COMPUTE_DTYPE_REASON})")

use_dummy_wandb = args.run == "dummy" or not master_process
if use_dummy_wandb:
    wandb_run = DummyWandb()
else:
    import wandb
    wandb_run = wandb.init(project="nanochat", name=args.run, config=user_config)

# ---------------------------------------------------------------- tokenizer / vocabulary
if args.synthetic_data:
    tokenizer, token_bytes, vocab_size = None, None, args.vocab_size
else:
    from nanochat_b200.tokenizer import get_tokenizer, get_token_bytes
    tokenizer = get_tokenizer()
    token_bytes = get_token_bytes(device=device)
    vocab_size = tokenizer.get_vocab_size()
print0(f"Vocab size: {vocab_size:,}")


def build_model_meta(depth):
    dim, heads = schedules.model_dims(depth, args.aspect_ratio, args.head_dim)
    cfg = GPTConfig(sequence_len=args.max_seq_len, vocab_size=vocab_size, n_layer=depth, n_head=heads,
                    n_kv_head=heads, n_embd=dim, window_pattern=args.window_pattern)
    with torch.device("meta"):
        return GPT(cfg)


model = build_model_meta(args.depth)
model_config_kwargs = asdict(model.config)
print0(f"Model config:\n{json.dumps(model_config_kwargs, indent=2)}")
model.to_empty(device=device)
model.init_weights()

base_dir = get_base_dir()
checkpoint_dir = os.path.join(base_dir, "base_checkpoints", args.model_tag if args.model_tag else f"d{args.depth}")
# every metric record also goes to a JSONL file on the master rank (one object per line, flushed per line)
metrics_path = args.metrics_file
if metrics_path is None:
    metrics_path = os.path.join(base_dir, "metrics", f"base_train_{args.model_tag if args.model_tag else f'd{args.depth}'}.jsonl")
wandb_run = MetricsLog(metrics_path if (master_process and metrics_path) else None, forward_to=wandb_run,
                       header={"script": "base_train", "config": user_config, "world_size": ddp_world_size})
timers = PhaseTimers(device_type=device_type)
# host-side failure detection (both off by default): a lost rank is reported before the next step is launched
from nanochat_b200.parallel.heartbeat import Heartbeat, LossWatch, default_store
heartbeat = None
if args.heartbeat_timeout > 0 and ddp_world_size > 1:
    heartbeat = Heartbeat(default_store(), ddp_rank, ddp_world_size, interval=min(1.0, args.heartbeat_timeout / 4),
                          timeout=args.heartbeat_timeout)
    heartbeat.wait_for_peers()
loss_watch = LossWatch() if args.abort_on_divergence else None
resuming = args.resume_from_step != -1
if resuming:
    print0(f"Resuming optimization from step {args.resume_from_step}")
    saved_ranks = optimizer_shard_count(checkpoint_dir, args.resume_from_step)
    if saved_ranks not in (0, ddp_world_size):
        raise CheckpointError(f"{checkpoint_dir} step {args.resume_from_step} was written by {saved_ranks} rank(s); the "
                              f"optimizer state is sharded by rank, so resume with {saved_ranks} rank(s), not {ddp_world_size}")
    model_data, optimizer_data, meta_data = load_checkpoint(checkpoint_dir, args.resume_from_step, device,
                                                            load_optimizer=True, rank=ddp_rank)
    model.load_state_dict(model_data, strict=True, assign=True)
    del model_data

# ---------------------------------------------------------------------------------- fp8
if args.fp8:
    if device_type != "cuda":
        print0("Warning: FP8 training requires CUDA, ignoring --fp8 flag")
    else:
        from nanochat_b200.fp8 import Float8LinearConfig, convert_to_float8_training, default_fp8_filter
        n_linear = sum(1 for m in model.modules() if isinstance(m, torch.nn.Linear))
        convert_to_float8_training(model, config=Float8LinearConfig.from_recipe_name(args.fp8_recipe),
                                   module_filter_fn=default_fp8_filter)
        n_fp8 = sum(1 for m in model.modules() if "Float8" in type(m).__name__)
        print0(f"✓ FP8 training enabled ({args.fp8_recipe} scaling) - converted {n_fp8}/{n_linear} linear layers, "
               f"skipped {n_linear - n_fp8} (too small)")


@contextmanager
def disable_fp8(m):
    """Evaluation always runs the bf16 linears (reference: scripts/base_train.py:195-240)."""
    from nanochat_b200.fp8 import fp8_disabled
    with fp8_disabled(m):
        yield


orig_model = model   # no tracing compiler: the training module is also the evaluation module

# ---------------------------------------------------------------- scaling-law hyper-parameters
param_counts = model.num_scaling_params()
print0("Parameter counts:")
for key, value in param_counts.items():
    print0(f"{key:24s}: {value:,}")
num_flops_per_token = model.estimate_flops()
print0(f"Estimated FLOPs per token: {num_flops_per_token:e}")
num_scaling_params = schedules.scaling_param_count(model)
hp = schedules.derive_hparams(num_scaling_params, schedules.scaling_param_count(build_model_meta(12)),
                              args.target_param_data_ratio, args.weight_decay, args.total_batch_size)
total_batch_size = hp.total_batch_size
if args.total_batch_size == -1:
    print0(f"Auto-computed optimal batch size: {total_batch_size:,} tokens")
if hp.batch_lr_scale != 1.0:
    print0(f"Scaling LRs by {hp.batch_lr_scale:.4f} for batch size {total_batch_size:,} (reference: {schedules.B_REF:,})")
if hp.weight_decay != args.weight_decay:
    print0(f"Scaling weight decay from {args.weight_decay:.6f} to {hp.weight_decay:.6f} for depth {args.depth}")

# ----------------------------------------------------------------------------- optimizer
# The step itself (micro-batches, sharded update, gradient reset) is train.TrainStep: the same object the
# benchmark times. It builds the parameter arena on the native path and picks the optimizer collectives.
from nanochat_b200.train import TrainStep
scaler = torch.amp.GradScaler() if common.COMPUTE_DTYPE == torch.float16 else None
if scaler is not None:
    print0("GradScaler enabled for fp16 training")
trainer = TrainStep(
    model, comm=args.comm if ddp_world_size > 1 else None, scaler=scaler, timers=timers, log=print0,
    unembedding_lr=args.unembedding_lr * hp.batch_lr_scale, embedding_lr=args.embedding_lr * hp.batch_lr_scale,
    scalar_lr=args.scalar_lr * hp.batch_lr_scale, matrix_lr=args.matrix_lr * hp.batch_lr_scale,
    weight_decay=hp.weight_decay)
optimizer = trainer.optimizer
if ddp_world_size > 1:
    print0(f"Optimizer collectives: {trainer.comm_name}")
if resuming:
    optimizer.load_state_dict(optimizer_data)
    del optimizer_data

# ----------------------------------------------------------------------------------- data
if args.synthetic_data:
    from nanochat_b200.dataloader import synthetic_token_loader
    train_loader = synthetic_token_loader(args.device_batch_size, args.max_seq_len, vocab_size, device=device,
                                          cycle=args.synthetic_cycle)
    build_val_loader = None
    # a fixed stream of random tokens whose mean loss a reloaded checkpoint must reproduce: held out for fresh random
    # batches, the repeated training batches themselves when the stream cycles (then the loss is seen to fall)
    build_synthetic_val = lambda: synthetic_token_loader(
        args.device_batch_size, args.max_seq_len, vocab_size, device=device, cycle=args.synthetic_cycle,
        seed=0 if args.synthetic_cycle > 0 else 4321)
else:
    from nanochat_b200.dataloader import (tokenizing_distributed_data_loader_bos_bestfit,
                                          tokenizing_distributed_data_loader_with_state_bos_bestfit)
    resume_state = None if not resuming else meta_data["dataloader_state_dict"]
    train_loader = tokenizing_distributed_data_loader_with_state_bos_bestfit(
        tokenizer, args.device_batch_size, args.max_seq_len, split="train", device=device,
        resume_state_dict=resume_state)
    build_val_loader = lambda: tokenizing_distributed_data_loader_bos_bestfit(
        tokenizer, args.device_batch_size, args.max_seq_len, split="val", device=device)
x, y, dataloader_state_dict = next(train_loader)


def current_batch(_micro_step):
    return x, y


def advance_batch(_micro_step):
    """Runs once a micro-batch's backward is queued: host-side packing of the next batch overlaps the GPU work."""
    global x, y, dataloader_state_dict
    x, y, dataloader_state_dict = next(train_loader)


# ------------------------------------------------------------------------------- horizon
assert args.num_iterations > 0 or args.target_param_data_ratio > 0 or args.target_flops > 0
if args.num_iterations > 0:
    num_iterations = args.num_iterations
    print0(f"Using user-provided number of iterations: {num_iterations:,}")
elif args.target_flops > 0:
    num_iterations = round(args.target_flops / (num_flops_per_token * total_batch_size))
    print0(f"Calculated number of iterations from target FLOPs: {num_iterations:,}")
else:
    num_iterations = hp.target_tokens // total_batch_size
    print0(f"Calculated number of iterations from target data:param ratio: {num_iterations:,}")
total_tokens = total_batch_size * num_iterations
print0(f"Total number of training tokens: {total_tokens:,}")
print0(f"Tokens : Scaling params ratio: {total_tokens / num_scaling_params:.2f}")
print0(f"Total training FLOPs estimate: {num_flops_per_token * total_tokens:e}")

if not resuming:
    step, val_bpb, min_val_bpb, smooth_train_loss, total_training_time = 0, None, float("inf"), 0, 0
else:
    step = meta_data["step"]
    val_bpb = meta_data["val_bpb"]
    loop_state = meta_data["loop_state"]
    min_val_bpb = loop_state["min_val_bpb"]
    smooth_train_loss = loop_state["smooth_train_loss"]
    total_training_time = loop_state["total_training_time"]

tokens_per_fwdbwd = args.device_batch_size * args.max_seq_len
world_tokens_per_fwdbwd = tokens_per_fwdbwd * ddp_world_size
assert total_batch_size % world_tokens_per_fwdbwd == 0, (
    f"total_batch_size ({total_batch_size}) must be a multiple of {world_tokens_per_fwdbwd}.")
grad_accum_steps = total_batch_size // world_tokens_per_fwdbwd
print0(f"Tokens / micro-batch / rank: {args.device_batch_size} x {args.max_seq_len} = {tokens_per_fwdbwd:,}")
print0(f"Tokens / micro-batch: {world_tokens_per_fwdbwd:,}")
print0(f"Total batch size {total_batch_size:,} => gradient accumulation steps: {grad_accum_steps}")
trainer.grad_accum = grad_accum_steps

# ---------------------------------------------------------------------------------- loop
while True:
    last_step = step == num_iterations
    if heartbeat is not None:
        heartbeat.check()                  # raises RankLostError: no collective is started against a dead peer
    flops_so_far = num_flops_per_token * total_batch_size * step

    if build_val_loader is not None and args.eval_every > 0 and (last_step or step % args.eval_every == 0):
        model.eval()
        eval_steps = args.eval_tokens // (args.device_batch_size * args.max_seq_len * ddp_world_size)
        with disable_fp8(model):
            val_bpb = evaluate_bpb(model, build_val_loader(), eval_steps, token_bytes)
        print0(f"Step {step:05d} | Validation bpb: {val_bpb:.6f}")
        min_val_bpb = min(min_val_bpb, val_bpb)
        wandb_run.log({"step": step, "total_training_flops": flops_so_far,
                       "total_training_time": total_training_time, "val/bpb": val_bpb})
        model.train()

    if args.synthetic_data and args.eval_every > 0 and (last_step or step % args.eval_every == 0):
        model.eval()
        eval_steps = max(1, min(4, args.eval_tokens // (args.device_batch_size * args.max_seq_len * ddp_world_size)))
        with disable_fp8(model):
            val_loss = evaluate_mean_loss(model, build_synthetic_val(), eval_steps)
        print0(f"Step {step:05d} | Validation loss: {val_loss:.6f}")
        wandb_run.log({"step": step, "total_training_flops": flops_so_far,
                       "total_training_time": total_training_time, "val/loss": val_loss})
        model.train()

    if tokenizer is not None and args.core_metric_every > 0 and (
            last_step or (step > 0 and step % args.core_metric_every == 0)):
        from scripts.base_eval import evaluate_core
        model.eval()
        with disable_fp8(orig_model):
            results = evaluate_core(orig_model, tokenizer, device, max_per_task=args.core_metric_max_per_task)
        print0(f"Step {step:05d} | CORE metric: {results['core_metric']:.4f}")
        wandb_run.log({"step": step, "total_training_flops": flops_so_far, "core_metric": results["core_metric"],
                       "centered_results": results["centered_results"]})
        model.train()

    if tokenizer is not None and args.sample_every > 0 and master_process and (
            last_step or (step > 0 and step % args.sample_every == 0)):
        from scripts.base_eval import SAMPLE_PROMPTS
        model.eval()
        engine = Engine(orig_model, tokenizer)
        for prompt in SAMPLE_PROMPTS:
            with disable_fp8(orig_model):
                sample, _ = engine.generate_batch(tokenizer(prompt, prepend="<|bos|>"), num_samples=1,
                                                  max_tokens=16, temperature=0)
            print0(tokenizer.decode(sample[0]))
        model.train()

    if (last_step and not args.no_final_save) or (step > 0 and step != args.resume_from_step and args.save_every > 0
                                                  and step % args.save_every == 0):
        save_checkpoint(checkpoint_dir, step, trainer.model_state_dict(), optimizer.state_dict(), {
            "step": step, "val_bpb": val_bpb, "model_config": model_config_kwargs, "user_config": user_config,
            "device_batch_size": args.device_batch_size, "max_seq_len": args.max_seq_len,
            "total_batch_size": total_batch_size, "dataloader_state_dict": dataloader_state_dict,
            "loop_state": {"min_val_bpb": min_val_bpb, "smooth_train_loss": smooth_train_loss,
                           "total_training_time": total_training_time},
        }, rank=ddp_rank)

    if last_step:
        break

    # ------------------------------------------------------------------ one optimizer step
    synchronize()
    t0 = time.time()
    lrm = schedules.pretrain_lr_multiplier(step, num_iterations, args.warmup_steps, args.warmdown_ratio,
                                           args.final_lr_frac)
    muon_momentum = schedules.pretrain_muon_momentum(step, num_iterations, args.warmdown_ratio)
    muon_weight_decay = schedules.pretrain_weight_decay(step, num_iterations, hp.weight_decay)
    for group in optimizer.param_groups:
        group["lr"] = group["initial_lr"] * lrm
        if group["kind"] == "muon":
            group["momentum"] = muon_momentum
            group["weight_decay"] = muon_weight_decay
    train_loss = trainer.step(current_batch, after_backward=advance_batch)
    train_loss_f = train_loss.item()
    synchronize()
    dt = time.time() - t0
    phase_ms = timers.collect()            # {} unless NANOCHAT_TRACE=1; device time per phase, max over ranks
    if loss_watch is not None:
        why = loss_watch.update(train_loss_f)
        if why is not None:                # every rank sees its own shard's loss; any rank may raise
            raise RuntimeError(f"training diverged at step {step}: {why}")

    ema_beta = 0.9
    smooth_train_loss = ema_beta * smooth_train_loss + (1 - ema_beta) * train_loss_f
    debiased_smooth_loss = smooth_train_loss / (1 - ema_beta ** (step + 1))
    pct_done = 100 * step / num_iterations
    tok_per_sec = int(total_batch_size / dt)
    mfu = 100 * num_flops_per_token * total_batch_size / dt / (gpu_peak_flops * ddp_world_size)
    if step > 10:
        total_training_time += dt
    steps_done = step - 10
    eta_str = ""
    if steps_done > 0:
        eta_str = f" | eta: {(num_iterations - step) * total_training_time / steps_done / 60:.1f}m"
    epoch = f"{dataloader_state_dict['epoch']} pq: {dataloader_state_dict['pq_idx']} rg: {dataloader_state_dict['rg_idx']}"
    print0(f"step {step:05d}/{num_iterations:05d} ({pct_done:.2f}%) | loss: {debiased_smooth_loss:.6f} | lrm: {lrm:.2f} | "
           f"dt: {dt * 1000:.2f}ms | tok/sec: {tok_per_sec:,} | bf16_mfu: {mfu:.2f} | epoch: {epoch} | "
           f"total time: {total_training_time/60:.2f}m{eta_str}")
    if phase_ms:
        print0("    phases (device ms, max over ranks): " + " | ".join(f"{k}: {v:.2f}" for k, v in phase_ms.items()))
    if step % args.log_every == 0:
        wandb_run.log({"step": step, "total_training_flops": flops_so_far,
                       "total_training_time": total_training_time, "train/loss": debiased_smooth_loss,
                       "train/lrm": lrm, "train/dt": dt, "train/tok_per_sec": tok_per_sec, "train/mfu": mfu,
                       "train/epoch": epoch, **{f"train/{k}_ms": v for k, v in phase_ms.items()}})

    first_step_of_run = (step == 0) or (resuming and step == args.resume_from_step)
    step += 1
    # the cyclic GC costs ~0.5 s per scan on a large module graph: freeze what exists, then switch it off
    if first_step_of_run:
        gc.collect()
        gc.freeze()
        gc.disable()
    elif step % 5000 == 0:
        gc.collect()

if device_type == "cuda" and ops.get_kernel_mode() == "native":
    nat = ops.native_module()
    nat.check_status()                     # raises if any kernel gave up on a bounded wait during the run
    print0(f"Native kernels: {nat.launch_count():,} launches | fp8 layer passes: {nat.stats['fp8_layer_forward']:,} | "
           f"bf16 layer passes: {nat.stats['bf16_layer_forward']:,} | fused QKV: {nat.stats['fused_qkv_forward']:,}")
print0(f"Peak memory usage: {get_max_memory() / 1024 / 1024:.2f}MiB")
print0(f"Total training time: {total_training_time/60:.2f}m")
if val_bpb is not None:
    print0(f"Minimum validation bpb: {min_val_bpb:.6f}")
wandb_run.finish()
if heartbeat is not None:
    heartbeat.leave()
compute_cleanup()
