"""
Reinforcement learning on GSM8K: on-policy REINFORCE with a mean baseline ("GRPO" without the
trust region, KL term, z-scoring or length normalisation by sequence).

    python -m scripts.chat_rl
    torchrun --nproc_per_node=8 -m scripts.chat_rl -- --run default

Per training example: sample `num_samples` completions with the Engine (tool use included),
reward = exact final-answer match, advantage = reward - mean reward, loss =
-sum(logp * advantage) over sampled tokens / (valid tokens x passes x examples per rank).
Forced (tool-output) and prompt tokens carry no loss (reference: scripts/chat_rl.py).
"""
import os
import argparse
import itertools

import torch
import torch.distributed as dist

from nanochat_b200.common import (compute_init, compute_cleanup, print0, get_base_dir, DummyWandb,
                                  autodetect_device_type)
from nanochat_b200.checkpoint_manager import save_checkpoint, load_model
from nanochat_b200.engine import Engine
from tasks.gsm8k import GSM8K

parser = argparse.ArgumentParser(description="Reinforcement learning on GSM8K")
parser.add_argument("--run", type=str, default="dummy")
parser.add_argument("--device-type", type=str, default="")
parser.add_argument("--model-tag", type=str, default=None)
parser.add_argument("--model-step", type=int, default=None)
parser.add_argument("--num-epochs", type=int, default=1)
parser.add_argument("--device-batch-size", type=int, default=8)
parser.add_argument("--examples-per-step", type=int, default=16)
parser.add_argument("--num-samples", type=int, default=16)
parser.add_argument("--max-new-tokens", type=int, default=256)
parser.add_argument("--temperature", type=float, default=1.0)
parser.add_argument("--top-k", type=int, default=50)
parser.add_argument("--embedding-lr", type=float, default=0.2)
parser.add_argument("--unembedding-lr", type=float, default=0.004)
parser.add_argument("--matrix-lr", type=float, default=0.02)
parser.add_argument("--weight-decay", type=float, default=0.0)
parser.add_argument("--init-lr-frac", type=float, default=0.05)
parser.add_argument("--eval-every", type=int, default=60)
parser.add_argument("--eval-examples", type=int, default=400)
parser.add_argument("--save-every", type=int, default=60)
parser.add_argument("--comm", type=str, default="auto", choices=["auto", "nccl", "fused"],
                    help="optimizer collectives: torch.distributed or fused peer-to-peer kernels")
args = parser.parse_args()
user_config = vars(args).copy()

device_type = autodetect_device_type() if args.device_type == "" else args.device_type
ddp, ddp_rank, ddp_local_rank, ddp_world_size, device = compute_init(device_type)
master_process = ddp_rank == 0
if args.run == "dummy" or not master_process:
    wandb_run = DummyWandb()
else:
    import wandb
    wandb_run = wandb.init(project="nanochat-rl", name=args.run, config=user_config)

model, tokenizer, meta = load_model("sft", device, phase="eval", model_tag=args.model_tag, step=args.model_step)
engine = Engine(model, tokenizer)
train_task = GSM8K(subset="main", split="train")
val_task = GSM8K(subset="main", split="test")
num_steps = (len(train_task) // args.examples_per_step) * args.num_epochs
print0(f"Calculated number of steps: {num_steps}")
step = 0


@torch.no_grad()
def rollouts():
    """Yields, per training example of this rank: (sequences, inputs, targets, rewards, advantages)."""
    pad = tokenizer.encode_special("<|assistant_end|>")     # padding only; never enters the loss
    for idx in itertools.cycle(range(ddp_rank, len(train_task), ddp_world_size)):
        conv = train_task[idx]
        prompt = tokenizer.render_for_completion(conv)
        model.eval()
        seqs, masks = [], []
        for k in range(args.num_samples // args.device_batch_size):
            seed = hash((step, idx, k)) & 0x7FFFFFFF
            s, m = engine.generate_batch(prompt, num_samples=args.device_batch_size, max_tokens=args.max_new_tokens,
                                         temperature=args.temperature, top_k=args.top_k, seed=seed)
            seqs += s
            masks += m
        rewards = torch.tensor([train_task.reward(conv, tokenizer.decode(s[len(prompt):])) for s in seqs],
                               dtype=torch.float, device=device)
        width = max(len(s) for s in seqs)
        ids = torch.tensor([s + [pad] * (width - len(s)) for s in seqs], dtype=torch.long, device=device)
        keep = torch.tensor([m + [0] * (width - len(m)) for m in masks], dtype=torch.long, device=device)
        targets = ids[:, 1:].clone()
        targets[keep[:, 1:] == 0] = -1      # prompt, forced tool output and padding carry no loss
        yield seqs, ids[:, :-1], targets, rewards, rewards - rewards.mean()


def run_gsm8k_eval(task, max_examples=None, num_samples=1, max_completion_tokens=256, temperature=0.0, top_k=50):
    """Yields {'idx', 'outcomes': [{'is_correct'}...]} for this rank's share; the caller reduces."""
    limit = len(task) if max_examples is None else min(max_examples, len(task))
    assert num_samples <= args.device_batch_size
    for idx in range(ddp_rank, limit, ddp_world_size):
        conv = task[idx]
        prompt = tokenizer.render_for_completion(conv)
        seqs, _ = engine.generate_batch(prompt, num_samples=num_samples, max_tokens=max_completion_tokens,
                                        temperature=temperature, top_k=top_k)
        yield {"idx": idx, "outcomes": [{"is_correct": task.evaluate(conv, tokenizer.decode(s[len(prompt):]))}
                                        for s in seqs]}


# the update (sharded optimizer step, gradient reset, consistent checkpoints) is train.TrainStep, as in pretraining
from nanochat_b200.train import TrainStep
trainer = TrainStep(model, comm=args.comm if ddp_world_size > 1 else None, log=print0,
                    unembedding_lr=args.unembedding_lr, embedding_lr=args.embedding_lr,
                    matrix_lr=args.matrix_lr, weight_decay=args.weight_decay)
optimizer = trainer.optimizer
for g in optimizer.param_groups:
    g["lr"] *= args.init_lr_frac
    g["initial_lr"] = g["lr"]
print0(f"Total sequences per step: {args.examples_per_step * args.num_samples}")
assert args.examples_per_step % ddp_world_size == 0, "Desired examples per step must be divisible by the number of ranks"
examples_per_rank = args.examples_per_step // ddp_world_size
print0(f"Calculated examples per rank: {examples_per_rank}")

batches = rollouts()
for step in range(num_steps):
    if step % args.eval_every == 0:
        model.eval()
        K = args.device_batch_size
        records = list(run_gsm8k_eval(val_task, num_samples=K, max_examples=args.eval_examples, temperature=1.0))
        passk = torch.tensor([sum(any(o["is_correct"] for o in r["outcomes"][:k]) for r in records)
                              for k in range(1, K + 1)], dtype=torch.float, device=device)
        count = torch.tensor(len(records), dtype=torch.long, device=device)
        if ddp and dist.is_initialized():
            dist.all_reduce(count, op=dist.ReduceOp.SUM)
            dist.all_reduce(passk, op=dist.ReduceOp.SUM)
        passk = passk / count.item()
        print0(f"Step {step} | " + ", ".join(f"Pass@{k}: {passk[k - 1].item():.4f}" for k in range(1, K + 1)))
        wandb_run.log({"step": step, **{f"pass@{k}": passk[k - 1].item() for k in range(1, K + 1)}})

    reward_means, lengths = [], []
    for example_step in range(examples_per_rank):
        seqs, inputs_all, targets_all, rewards_all, adv_all = next(batches)
        model.train()
        assert inputs_all.size(0) % args.device_batch_size == 0
        passes = inputs_all.size(0) // args.device_batch_size
        for p in range(passes):
            sl = slice(p * args.device_batch_size, (p + 1) * args.device_batch_size)
            inputs, targets, adv = inputs_all[sl], targets_all[sl], adv_all[sl]
            logp = -model(inputs, targets, loss_reduction="none").view_as(inputs)
            valid = (targets >= 0).sum().clamp(min=1)
            loss = -(logp * adv.unsqueeze(-1)).sum() / (valid * passes * examples_per_rank)
            trainer.backward(loss)
            print0(f"Step {step}/{num_steps} | Example step {example_step} | Pass {p} | loss: {loss.item():.6f} | "
                   f"Average reward: {rewards_all[sl].mean().item()}")
        reward_means.append(rewards_all.mean().item())
        lengths += [len(s) for s in seqs]

    mean_reward = sum(reward_means) / len(reward_means)
    mean_len = sum(lengths) / len(lengths)
    if ddp and dist.is_initialized():
        t = torch.tensor([mean_reward, mean_len], dtype=torch.float, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        mean_reward, mean_len = (t / ddp_world_size).tolist()
    print0(f"Step {step}/{num_steps} | Average reward: {mean_reward} | Average sequence length: {mean_len:.2f}")
    wandb_run.log({"step": step, "reward": mean_reward, "sequence_length": mean_len})

    lrm = 1.0 - step / num_steps
    for g in optimizer.param_groups:
        g["lr"] = g["initial_lr"] * lrm
    trainer.optimizer_step()
    wandb_run.log({"step": step, "lrm": lrm})

    saving = (step > 0 and step % args.save_every == 0) or step == num_steps - 1
    model_state = trainer.model_state_dict() if saving else None      # collective: every rank takes part
    if master_process and saving:
        out_dir = os.path.join(get_base_dir(), "chatrl_checkpoints",
                               args.model_tag if args.model_tag else f"d{model.config.n_layer}")
        save_checkpoint(out_dir, step, model_state, None, {"model_config": dict(model.config.__dict__)})
        print(f"Saved model checkpoint to {out_dir}")

batches.close()          # the rollout generator holds a no_grad context: close it before the interpreter tears torch down
wandb_run.finish()
compute_cleanup()
