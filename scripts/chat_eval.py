"""
Evaluate a chat model on ARC-Easy, ARC-Challenge, MMLU (categorical) and GSM8K, HumanEval
(generative); ChatCORE is the mean baseline-centred accuracy over all five.

    python -m scripts.chat_eval -i sft -a ARC-Easy
    torchrun --nproc_per_node=8 -m scripts.chat_eval -- -i sft

Categorical tasks are scored without sampling: one batched forward, then the argmax over the
logits of the answer-letter tokens at the last prompt position. Generative tasks sample
`num_samples` completions per problem and pass if any of them passes
(reference: scripts/chat_eval.py:28-176).
"""
import argparse

import torch
import torch.distributed as dist

from nanochat_b200.common import compute_init, compute_cleanup, get_dist_info, print0, autodetect_device_type

ALL_TASKS = ["ARC-Easy", "ARC-Challenge", "MMLU", "GSM8K", "HumanEval"]
CATEGORICAL_TASKS = {"ARC-Easy", "ARC-Challenge", "MMLU"}
BASELINE_ACCURACY = {"ARC-Easy": 0.25, "ARC-Challenge": 0.25, "MMLU": 0.25, "GSM8K": 0.0, "HumanEval": 0.0}


def _sum_over_ranks(values, device):
    t = torch.tensor(values, dtype=torch.long, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return t.tolist()


def run_generative_eval(task, tokenizer, model, engine, num_samples, max_new_tokens, temperature, top_k,
                        max_problems=None):
    ddp, rank, _, world = get_dist_info()
    n = len(task) if max_problems is None else min(len(task), max_problems)
    passed = total = 0
    for i in range(rank, n, world):
        conv = task[i]
        prompt = tokenizer.render_for_completion(conv)
        outs, _ = engine.generate_batch(prompt, num_samples=num_samples, max_tokens=max_new_tokens,
                                        temperature=temperature, top_k=top_k)
        texts = [tokenizer.decode(o[len(prompt):]) for o in outs]
        passed += int(any(task.evaluate(conv, t) for t in texts))
        total += 1
        print(f"\r\033[KRank {rank} | {passed}/{total} ({100 * passed / total:.2f}%)", end="", flush=True)
    print()
    if ddp and dist.is_initialized():
        passed, total = _sum_over_ranks([passed, total], model.get_device())
    print0("=" * 50)
    print0(f"Final: {passed}/{total} ({100 * passed / total:.2f}%)")
    return passed / total


def run_categorical_eval(task, tokenizer, model, batch_size, max_problems=None):
    ddp, rank, _, world = get_dist_info()
    device = model.get_device()
    pad = tokenizer.get_bos_token_id()
    n = len(task) if max_problems is None else min(len(task), max_problems)
    n_batches = -(-n // batch_size)
    letter_id = {}
    passed = total = 0
    for bi in range(rank, n_batches, world):
        convs = [task[j] for j in range(bi * batch_size, min((bi + 1) * batch_size, n))]
        prompts = [tokenizer.render_for_completion(c) for c in convs]
        width = max(len(p) for p in prompts)
        answer_pos = [len(p) - 1 for p in prompts]
        ids = torch.tensor([p + [pad] * (width - len(p)) for p in prompts], dtype=torch.long, device=device)
        with torch.no_grad():
            logits = model(ids)
        for row, conv in enumerate(convs):
            choices = []
            for letter in conv["letters"]:
                if letter not in letter_id:
                    enc = tokenizer.encode(letter)
                    assert len(enc) == 1, "Each letter must be a single token"
                    letter_id[letter] = enc[0]
                choices.append(letter_id[letter])
            pick = logits[row, answer_pos[row], choices].argmax(dim=-1).item()
            passed += int(task.evaluate(conv, conv["letters"][pick]))
            total += 1
    if ddp and dist.is_initialized():
        passed, total = _sum_over_ranks([passed, total], device)
    print0(f"Final: {passed}/{total} ({100 * passed / total:.2f}%)")
    return passed / total


def _make_task(name):
    from tasks.humaneval import HumanEval
    from tasks.mmlu import MMLU
    from tasks.arc import ARC
    from tasks.gsm8k import GSM8K
    return {
        "HumanEval": lambda: HumanEval(),
        "MMLU": lambda: MMLU(subset="all", split="test"),
        "ARC-Easy": lambda: ARC(subset="ARC-Easy", split="test"),
        "ARC-Challenge": lambda: ARC(subset="ARC-Challenge", split="test"),
        "GSM8K": lambda: GSM8K(subset="main", split="test"),
    }[name]()


def run_chat_eval(task_name, model, tokenizer, engine, batch_size=1, num_samples=1, max_new_tokens=512,
                  temperature=0.0, top_k=50, max_problems=None):
    task = _make_task(task_name)
    if task.eval_type == "generative":
        return run_generative_eval(task, tokenizer, model, engine, num_samples, max_new_tokens, temperature,
                                   top_k, max_problems=max_problems)
    if task.eval_type == "categorical":
        return run_categorical_eval(task, tokenizer, model, batch_size, max_problems=max_problems)
    raise ValueError(f"Unsupported task evaluation type: {task.eval_type}")


def chatcore(results, tasks=ALL_TASKS):
    return sum((results[t] - BASELINE_ACCURACY[t]) / (1.0 - BASELINE_ACCURACY[t]) for t in tasks) / len(tasks)


if __name__ == "__main__":
    from nanochat_b200.checkpoint_manager import load_model
    from nanochat_b200.engine import Engine
    ap = argparse.ArgumentParser()
    ap.add_argument("-i", "--source", type=str, required=True, help="sft|rl")
    ap.add_argument("-a", "--task-name", type=str, default=None, help="task names separated by | (default: all)")
    ap.add_argument("-t", "--temperature", type=float, default=0.0)
    ap.add_argument("-m", "--max-new-tokens", type=int, default=512)
    ap.add_argument("-n", "--num-samples", type=int, default=1)
    ap.add_argument("-k", "--top-k", type=int, default=50)
    ap.add_argument("-b", "--batch-size", type=int, default=8)
    ap.add_argument("-g", "--model-tag", type=str, default=None)
    ap.add_argument("-s", "--step", type=int, default=None)
    ap.add_argument("-x", "--max-problems", type=int, default=None)
    ap.add_argument("--device-type", type=str, default="", choices=["cuda", "cpu", "mps", ""])
    args = ap.parse_args()
    device_type = autodetect_device_type() if args.device_type == "" else args.device_type
    _, _, _, _, device = compute_init(device_type)
    model, tokenizer, meta = load_model(args.source, device, phase="eval", model_tag=args.model_tag, step=args.step)
    engine = Engine(model, tokenizer)
    names = ALL_TASKS if args.task_name is None else args.task_name.split("|")
    results = {}
    for name in names:
        results[name] = run_chat_eval(name, model, tokenizer, engine, batch_size=args.batch_size,
                                      num_samples=args.num_samples, max_new_tokens=args.max_new_tokens,
                                      temperature=args.temperature, top_k=args.top_k,
                                      max_problems=args.max_problems)
        print0(f"{name} accuracy: {100 * results[name]:.2f}%")
    if all(t in results for t in ALL_TASKS):
        print0(f"ChatCORE metric: {chatcore(results):.4f}")
    compute_cleanup()
