"""
Evaluate a base model: CORE (in-context accuracy), bits per byte on train/val, and samples.

    python -m scripts.base_eval --model-tag d24 --device-batch-size 16 --max-per-task 100
    torchrun --nproc_per_node=8 -m scripts.base_eval --model-tag d24

`--eval` takes a comma-separated subset of core,bpb,sample (reference: scripts/base_eval.py).
"""
import os
import csv
import json
import time
import random
import shutil
import zipfile
import tempfile
import argparse


from nanochat_b200.common import (compute_init, compute_cleanup, print0, get_base_dir, autodetect_device_type,
                                  download_file_with_lock)
from nanochat_b200.core_eval import evaluate_task

EVAL_BUNDLE_URL = "https://karpathy-public.s3.us-west-2.amazonaws.com/eval_bundle.zip"

SAMPLE_PROMPTS = [
    "The capital of France is",
    "The chemical symbol of gold is",
    "If yesterday was Friday, then tomorrow will be",
    "The opposite of hot is",
    "The planets of the solar system are:",
    "My favorite color is",
    "If 5*x + 3 = 13, then x is",
]


def place_eval_bundle(zip_path):
    target = os.path.join(get_base_dir(), "eval_bundle")
    with tempfile.TemporaryDirectory() as tmp:
        with zipfile.ZipFile(zip_path, "r") as z:
            z.extractall(tmp)
        shutil.move(os.path.join(tmp, "eval_bundle"), target)
    print0(f"Placed eval_bundle directory at {target}")


def evaluate_core(model, tokenizer, device, max_per_task=-1):
    """Runs every task of the bundle's core.yaml; returns accuracies, centred accuracies and their mean."""
    import yaml
    bundle = os.path.join(get_base_dir(), "eval_bundle")
    if not os.path.exists(bundle):
        download_file_with_lock(EVAL_BUNDLE_URL, "eval_bundle.zip", postprocess_fn=place_eval_bundle)
    with open(os.path.join(bundle, "core.yaml"), encoding="utf-8") as f:
        tasks = yaml.safe_load(f)["icl_tasks"]
    baselines = {}
    with open(os.path.join(bundle, "eval_meta_data.csv"), encoding="utf-8") as f:
        for row in csv.DictReader(f):
            baselines[row["Eval Task"]] = float(row["Random baseline"])
    results, centered = {}, {}
    for task in tasks:
        t0 = time.time()
        label = task["label"]
        meta = {"task_type": task["icl_task_type"], "dataset_uri": task["dataset_uri"],
                "num_fewshot": task["num_fewshot"][0],
                "continuation_delimiter": task.get("continuation_delimiter", " ")}
        print0(f"Evaluating: {label} ({meta['num_fewshot']}-shot, type: {meta['task_type']})... ", end="")
        with open(os.path.join(bundle, "eval_data", meta["dataset_uri"]), encoding="utf-8") as f:
            data = [json.loads(line.strip()) for line in f]
        random.Random(1337).shuffle(data)          # fixed order so --max-per-task takes a stable subset
        if max_per_task > 0:
            data = data[:max_per_task]
        acc = evaluate_task(model, tokenizer, data, device, meta)
        base = 0.01 * baselines[label]
        results[label] = acc
        centered[label] = (acc - base) / (1.0 - base)
        print0(f"accuracy: {acc:.4f} | centered: {centered[label]:.4f} | time: {time.time() - t0:.2f}s")
    return {"results": results, "centered_results": centered,
            "core_metric": sum(centered.values()) / len(centered)}


def main():
    from nanochat_b200.tokenizer import get_token_bytes
    from nanochat_b200.checkpoint_manager import load_model
    from nanochat_b200.dataloader import tokenizing_distributed_data_loader_bos_bestfit
    from nanochat_b200.loss_eval import evaluate_bpb
    from nanochat_b200.engine import Engine
    ap = argparse.ArgumentParser(description="Base model evaluation")
    ap.add_argument("--eval", type=str, default="core,bpb,sample")
    ap.add_argument("--model-tag", type=str, default=None)
    ap.add_argument("--step", type=int, default=None)
    ap.add_argument("--max-per-task", type=int, default=-1)
    ap.add_argument("--device-batch-size", type=int, default=32)
    ap.add_argument("--split-tokens", type=int, default=40 * 524288)
    ap.add_argument("--device-type", type=str, default="")
    args = ap.parse_args()
    modes = {m.strip() for m in args.eval.split(",")}
    if modes - {"core", "bpb", "sample"}:
        ap.error(f"Invalid eval modes: {modes - {'core', 'bpb', 'sample'}}")
    device_type = autodetect_device_type() if args.device_type == "" else args.device_type
    _, rank, _, world, device = compute_init(device_type)
    model, tokenizer, meta = load_model("base", device, phase="eval", model_tag=args.model_tag, step=args.step)
    seq_len = meta["model_config"]["sequence_len"]
    print0(f"Evaluating model: base_model (step {meta['step']})")
    print0(f"Eval modes: {', '.join(sorted(modes))}")

    if "sample" in modes and rank == 0:
        print0("\n" + "=" * 80 + "\nModel Samples\n" + "=" * 80)
        engine = Engine(model, tokenizer)
        print0("\nConditioned samples:")
        for prompt in SAMPLE_PROMPTS:
            out, _ = engine.generate_batch(tokenizer(prompt, prepend="<|bos|>"), num_samples=1, max_tokens=16,
                                           temperature=0)
            print0("-" * 80 + "\n" + tokenizer.decode(out[0]))
        print0("\nUnconditioned samples:")
        outs, _ = engine.generate_batch(tokenizer("", prepend="<|bos|>"), num_samples=8, max_tokens=128,
                                        temperature=1.0)
        for o in outs:
            print0("-" * 80 + "\n" + tokenizer.decode(o))

    if "bpb" in modes:
        print0("\n" + "=" * 80 + "\nBPB Evaluation\n" + "=" * 80)
        token_bytes = get_token_bytes(device=device)
        per_step = args.device_batch_size * seq_len * world
        if args.split_tokens % per_step != 0:
            args.split_tokens = (args.split_tokens // per_step) * per_step
            print0(f"Adjusted split_tokens to {args.split_tokens} (must be divisible by {per_step})")
        for split in ("train", "val"):
            loader = tokenizing_distributed_data_loader_bos_bestfit(tokenizer, args.device_batch_size, seq_len,
                                                                    split, device=device)
            print0(f"{split} bpb: {evaluate_bpb(model, loader, args.split_tokens // per_step, token_bytes):.6f}")

    if "core" in modes:
        print0("\n" + "=" * 80 + "\nCORE Evaluation\n" + "=" * 80)
        core = evaluate_core(model, tokenizer, device, max_per_task=args.max_per_task)
        if rank == 0:
            path = os.path.join(get_base_dir(), "base_eval", f"base_model_{meta['step']:06d}.csv")
            os.makedirs(os.path.dirname(path), exist_ok=True)
            with open(path, "w", encoding="utf-8", newline="") as f:
                f.write(f"{'Task':<35}, {'Accuracy':<10}, {'Centered':<10}\n")
                for label, acc in core["results"].items():
                    f.write(f"{label:<35}, {acc:<10.6f}, {core['centered_results'][label]:<10.6f}\n")
                f.write(f"{'CORE':<35}, {'':<10}, {core['core_metric']:<10.6f}\n")
            print0(f"\nResults written to: {path}")
            print0(f"CORE metric: {core['core_metric']:.4f}")
    compute_cleanup()


if __name__ == "__main__":
    main()
