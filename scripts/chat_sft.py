"""
Supervised finetuning of a pretrained base model on a mixture of chat tasks.

    python -m scripts.chat_sft
    torchrun --nproc_per_node=8 -m scripts.chat_sft -- --device-batch-size 16

Unset batch / learning-rate flags inherit the values stored with the pretraining checkpoint;
the optimizer is warm-started from the pretraining shard of this rank (momentum buffers) with
fresh learning rates; data are best-fit packed conversations with assistant-only loss
(nanochat_b200/sft_data.py); the LR schedule runs over consumed-data progress
(reference: scripts/chat_sft.py). `--synthetic-data` trains on generated conversations
(lengths U[64,2048], Bernoulli(0.5) turn masks) from random-init weights of `--depth`.
"""
import os
os.environ.setdefault("PYTORCH_ALLOC_CONF", "expandable_segments:True")
import gc
import time
import argparse

import torch
import torch.distributed as dist

from nanochat_b200 import common, schedules
from nanochat_b200.common import (compute_init, compute_cleanup, print0, DummyWandb, get_base_dir,
                                  autodetect_device_type, get_peak_flops, is_ddp_initialized)
from nanochat_b200.checkpoint_manager import save_checkpoint, load_model, load_optimizer_state
from nanochat_b200.loss_eval import evaluate_bpb
from nanochat_b200.sft_data import SFTState, sft_batches, synthetic_conversations

parser = argparse.ArgumentParser(description="Supervised fine-tuning (SFT) the model")
parser.add_argument("--run", type=str, default="dummy")
parser.add_argument("--device-type", type=str, default="")
parser.add_argument("--model-tag", type=str, default=None)
parser.add_argument("--model-step", type=int, default=None)
parser.add_argument("--load-optimizer", type=int, default=1)
parser.add_argument("--num-iterations", type=int, default=-1)
parser.add_argument("--max-seq-len", type=int, default=None)
parser.add_argument("--device-batch-size", type=int, default=None)
parser.add_argument("--total-batch-size", type=int, default=None)
parser.add_argument("--embedding-lr", type=float, default=None)
parser.add_argument("--unembedding-lr", type=float, default=None)
parser.add_argument("--matrix-lr", type=float, default=None)
parser.add_argument("--init-lr-frac", type=float, default=0.8)
parser.add_argument("--warmup-ratio", type=float, default=0.0)
parser.add_argument("--warmdown-ratio", type=float, default=0.5)
parser.add_argument("--final-lr-frac", type=float, default=0.0)
parser.add_argument("--eval-every", type=int, default=200)
parser.add_argument("--metrics-file", type=str, default=None,
                    help="JSONL metrics file (default: <base_dir>/metrics/chat_sft.jsonl; '' disables)")
parser.add_argument("--eval-tokens", type=int, default=40 * 524288)
parser.add_argument("--chatcore-every", type=int, default=200)
parser.add_argument("--chatcore-max-cat", type=int, default=-1)
parser.add_argument("--chatcore-max-sample", type=int, default=24)
parser.add_argument("--mmlu-epochs", type=int, default=3)
parser.add_argument("--gsm8k-epochs", type=int, default=4)
parser.add_argument("--synthetic-data", action="store_true")
parser.add_argument("--depth", type=int, default=32, help="model depth with --synthetic-data")
parser.add_argument("--comm", type=str, default="auto", choices=["auto", "nccl", "fused"],
                    help="optimizer collectives: torch.distributed or fused peer-to-peer kernels")
args = parser.parse_args()
user_config = vars(args).copy()

device_type = autodetect_device_type() if args.device_type == "" else args.device_type
ddp, ddp_rank, ddp_local_rank, ddp_world_size, device = compute_init(device_type)
master_process = ddp_rank == 0
print0(f"COMPUTE_DTYPE: {common.COMPUTE_DTYPE} ({common.COMPUTE_DTYPE_REASON})")
synchronize = torch.cuda.synchronize if device_type == "cuda" else lambda: None
get_max_memory = torch.cuda.max_memory_allocated if device_type == "cuda" else lambda: 0
gpu_peak_flops = get_peak_flops(torch.cuda.get_device_name(0)) if device_type == "cuda" else float("inf")
if args.run == "dummy" or not master_process:
    wandb_run = DummyWandb()
else:
    import wandb
    wandb_run = wandb.init(project="nanochat-sft", name=args.run, config=user_config)
# metric records also go to a JSONL file on the master rank
from nanochat_b200.utils.trace import MetricsLog
metrics_path = os.path.join(get_base_dir(), "metrics", "chat_sft.jsonl") if args.metrics_file is None else args.metrics_file
wandb_run = MetricsLog(metrics_path if (master_process and metrics_path) else None, forward_to=wandb_run,
                       header={"script": "chat_sft", "config": user_config, "world_size": ddp_world_size})

if args.synthetic_data:
    from nanochat_b200.models.gpt import GPT, GPTConfig
    dim, heads = schedules.model_dims(args.depth)
    cfg = GPTConfig(sequence_len=args.max_seq_len or 2048, vocab_size=32768, n_layer=args.depth, n_head=heads,
                    n_kv_head=heads, n_embd=dim)
    with torch.device("meta"):
        model = GPT(cfg)
    model.to_empty(device=device)
    model.init_weights()
    tokenizer, meta = None, {}
else:
    model, tokenizer, meta = load_model("base", device, phase="train", model_tag=args.model_tag, step=args.model_step)

pretrain_cfg = meta.get("user_config", {})
for name, fallback, source in (("max_seq_len", 2048, meta), ("device_batch_size", 32, meta),
                               ("total_batch_size", 524288, meta), ("embedding_lr", 0.3, pretrain_cfg),
                               ("unembedding_lr", 0.004, pretrain_cfg), ("matrix_lr", 0.02, pretrain_cfg)):
    given, stored = getattr(args, name), source.get(name)
    if given is None:
        setattr(args, name, stored if stored is not None else fallback)
        print0(f"Inherited {name}={getattr(args, name)} from pretrained checkpoint")
    elif stored is not None and given != stored:
        print0(f"NOTE: --{name.replace('_', '-')}={given} overrides pretrained value of {stored}")
    else:
        print0(f"Using {name}={given}")

orig_model = model
depth = model.config.n_layer
num_flops_per_token = model.estimate_flops()
tokens_per_fwdbwd = args.device_batch_size * args.max_seq_len
world_tokens_per_fwdbwd = tokens_per_fwdbwd * ddp_world_size
assert args.total_batch_size % world_tokens_per_fwdbwd == 0, (
    f"total_batch_size ({args.total_batch_size}) must be a multiple of {world_tokens_per_fwdbwd}.")
grad_accum_steps = args.total_batch_size // world_tokens_per_fwdbwd
print0(f"Tokens / micro-batch / rank: {args.device_batch_size} x {args.max_seq_len} = {tokens_per_fwdbwd:,}")
print0(f"Tokens / micro-batch: {world_tokens_per_fwdbwd:,}")
print0(f"Total batch size {args.total_batch_size:,} => gradient accumulation steps: {grad_accum_steps}")

# pretraining ends with weight decay annealed to zero, so SFT continues without it. The step (micro-batches,
# sharded update, gradient reset) is train.TrainStep, the object pretraining and the benchmark use.
from nanochat_b200.train import TrainStep
scaler = torch.amp.GradScaler() if common.COMPUTE_DTYPE == torch.float16 else None
trainer = TrainStep(model, grad_accum=grad_accum_steps, comm=args.comm if ddp_world_size > 1 else None, scaler=scaler,
                    log=print0, unembedding_lr=args.unembedding_lr, embedding_lr=args.embedding_lr,
                    matrix_lr=args.matrix_lr, weight_decay=0.0)
optimizer = trainer.optimizer
if ddp_world_size > 1:
    print0(f"Optimizer collectives: {trainer.comm_name}")
if args.load_optimizer and not args.synthetic_data:
    shard = load_optimizer_state("base", device, rank=ddp_rank, model_tag=args.model_tag, step=args.model_step,
                                 world_size=ddp_world_size)
    if shard is not None:
        fresh_lrs = [g["lr"] for g in optimizer.param_groups]
        optimizer.load_state_dict(shard)      # also brings back the (annealed) pretraining LRs ...
        for g, lr in zip(optimizer.param_groups, fresh_lrs):
            g["lr"] = lr                      # ... which are replaced by the SFT ones
        del shard
        print0("Loaded optimizer state from pretrained checkpoint (momentum buffers only, LRs reset)")
    else:
        print0("WARNING: optimizer checkpoint not found, starting with fresh optimizer (slightly worse)")
for g in optimizer.param_groups:
    g["lr"] *= args.init_lr_frac
    g["initial_lr"] = g["lr"]

# --------------------------------------------------------------------------------- data
if args.synthetic_data:
    train_dataset = synthetic_conversations(20000, 32768, max_len=args.max_seq_len, seed=ddp_rank)
    val_dataset = synthetic_conversations(512, 32768, max_len=args.max_seq_len, seed=10_000 + ddp_rank)
    render, bos = (lambda item: item), 0
    token_bytes = None
else:
    from nanochat_b200.tokenizer import get_token_bytes
    from tasks.common import TaskMixture
    from tasks.gsm8k import GSM8K
    from tasks.mmlu import MMLU
    from tasks.smoltalk import SmolTalk
    token_bytes = get_token_bytes(device=device)
    train_dataset = TaskMixture([SmolTalk(split="train"),
                                 *[MMLU(subset="all", split="auxiliary_train") for _ in range(args.mmlu_epochs)],
                                 *[GSM8K(subset="main", split="train") for _ in range(args.gsm8k_epochs)]])
    print0(f"Training mixture: {len(train_dataset):,} rows (MMLU x{args.mmlu_epochs}, GSM8K x{args.gsm8k_epochs})")
    val_dataset = TaskMixture([SmolTalk(split="test"), MMLU(subset="all", split="test", stop=5200),
                               GSM8K(subset="main", split="test", stop=420)])
    render, bos = tokenizer.render_conversation, tokenizer.get_bos_token_id()

state = SFTState()
train_loader = sft_batches(train_dataset, render, bos, args.device_batch_size, args.max_seq_len, ddp_rank,
                           ddp_world_size, device, num_iterations=args.num_iterations, state=state)
build_val_loader = lambda: sft_batches(val_dataset, render, bos, args.device_batch_size, args.max_seq_len,
                                       ddp_rank, ddp_world_size, device, track_progress=False)

# --------------------------------------------------------------------------------- loop
x, y = next(train_loader)
progress, step, lrm = 0.0, 0, 1.0


def current_batch(_micro_step):
    return x, y


def advance_batch(_micro_step):
    """Runs once a micro-batch's backward is queued: packing the next batch overlaps the GPU work."""
    global x, y, progress
    x, y = next(train_loader)
    progress = max(progress, state.approx_progress)


def set_schedules():
    """The learning-rate schedule runs over consumed-data progress, known once the step's batches are drawn."""
    global lrm
    lrm = schedules.sft_lr_multiplier(progress, args.warmup_ratio, args.warmdown_ratio, args.final_lr_frac)
    for g in optimizer.param_groups:
        g["lr"] = g["initial_lr"] * lrm
        if g["kind"] == "muon":
            g["momentum"] = schedules.sft_muon_momentum(step)


min_val_bpb, val_bpb = float("inf"), None
smooth_train_loss, ema_beta, total_training_time = 0.0, 0.9, 0.0
while True:
    flops_so_far = num_flops_per_token * args.total_batch_size * step
    last_step = state.last_step
    if ddp and is_ddp_initialized():        # ranks run out of data at slightly different times: agree
        flag = torch.tensor(int(last_step), dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        last_step = bool(flag.item())

    if token_bytes is not None and (last_step or (args.eval_every > 0 and step % args.eval_every == 0)):
        model.eval()
        eval_steps = args.eval_tokens // (args.device_batch_size * args.max_seq_len * ddp_world_size)
        val_bpb = evaluate_bpb(model, build_val_loader(), eval_steps, token_bytes)
        print0(f"Step {step:05d} | Validation bpb: {val_bpb:.4f}")
        min_val_bpb = min(min_val_bpb, val_bpb)
        wandb_run.log({"step": step, "total_training_flops": flops_so_far,
                       "total_training_time": total_training_time, "val/bpb": val_bpb})
        model.train()

    if tokenizer is not None and args.chatcore_every > 0 and (
            last_step or (step > 0 and step % args.chatcore_every == 0)):
        from nanochat_b200.engine import Engine
        from scripts.chat_eval import run_chat_eval, chatcore, ALL_TASKS, CATEGORICAL_TASKS
        model.eval()
        engine = Engine(orig_model, tokenizer)
        task_results = {}
        for name in ALL_TASKS:
            limit = args.chatcore_max_cat if name in CATEGORICAL_TASKS else args.chatcore_max_sample
            task_results[name] = run_chat_eval(name, orig_model, tokenizer, engine, batch_size=args.device_batch_size,
                                               max_problems=None if limit < 0 else limit)
            print0(f"  {name}: {100 * task_results[name]:.2f}%")
        cc, cc_cat = chatcore(task_results), chatcore(task_results, sorted(CATEGORICAL_TASKS))
        print0(f"Step {step:05d} | ChatCORE: {cc:.4f} | ChatCORE_cat: {cc_cat:.4f}")
        wandb_run.log({"step": step, "total_training_flops": flops_so_far, "chatcore_metric": cc,
                       "chatcore_cat": cc_cat, **{f"chatcore/{k}": v for k, v in task_results.items()}})
        model.train()

    if last_step and not args.synthetic_data:
        model_state = trainer.model_state_dict()      # collective: every rank's parameters made current first
        out_dir = os.path.join(get_base_dir(), "chatsft_checkpoints", args.model_tag if args.model_tag else f"d{depth}")
        save_checkpoint(out_dir, step, model_state, optimizer.state_dict(), {
            "step": step, "val_bpb": val_bpb,
            "model_config": {"sequence_len": args.max_seq_len, "vocab_size": tokenizer.get_vocab_size(),
                             "n_layer": depth, "n_head": model.config.n_head, "n_kv_head": model.config.n_kv_head,
                             "n_embd": model.config.n_embd, "window_pattern": model.config.window_pattern},
            "user_config": user_config}, rank=ddp_rank)
    if last_step:
        break

    synchronize()
    t0 = time.time()
    train_loss = trainer.step(current_batch, after_backward=advance_batch, before_update=set_schedules)
    synchronize()
    dt = time.time() - t0
    step += 1

    smooth_train_loss = ema_beta * smooth_train_loss + (1 - ema_beta) * train_loss.item()
    debiased = smooth_train_loss / (1 - ema_beta ** (step + 1))
    tok_per_sec = int(args.total_batch_size / dt)
    mfu = 100 * num_flops_per_token * args.total_batch_size / dt / (gpu_peak_flops * ddp_world_size)
    if step > 10:
        total_training_time += dt
    print0(f"step {step:05d} ({100 * progress:.2f}%) | loss: {debiased:.6f} | lrm: {lrm:.2f} | dt: {dt * 1000:.2f}ms | "
           f"tok/sec: {tok_per_sec:,} | mfu: {mfu:.2f} | epoch: {state.current_epoch} | "
           f"total time: {total_training_time/60:.2f}m")
    if step % 10 == 0:
        wandb_run.log({"step": step, "total_training_flops": flops_so_far, "total_training_time": total_training_time,
                       "train/loss": debiased, "train/lrm": lrm, "train/dt": dt, "train/tok_per_sec": tok_per_sec,
                       "train/mfu": mfu, "train/epoch": state.current_epoch})
    if step == 1:
        gc.collect()
        gc.freeze()
        gc.disable()
    elif step % 5000 == 0:
        gc.collect()

from nanochat_b200 import ops
if device_type == "cuda" and ops.get_kernel_mode() == "native":
    ops.native_module().check_status()     # raises if any kernel gave up on a bounded wait during the run
print0(f"Peak memory usage: {get_max_memory() / 1024 / 1024:.2f}MiB")
print0(f"Total training time: {total_training_time/60:.2f}m")
print0(f"Minimum validation bpb: {min_val_bpb:.4f}")
wandb_run.finish()
compute_cleanup()
