"""
The whole pipeline on CPU at toy size, through the entry points a user runs: synthetic corpus shards -> tokenizer
training -> pretraining (with validation bpb and a checkpoint) -> resume from that checkpoint -> base evaluation ->
one-shot chat -> SFT on synthetic conversations. Every stage is a subprocess with its own interpreter, as in the
run scripts.
"""
import os
import random
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.slow


def _run(base_dir, *args, timeout=600, extra_env=None):
    env = dict(os.environ, NANOCHAT_BASE_DIR=base_dir, OMP_NUM_THREADS="4", WANDB_MODE="disabled")
    env.update(extra_env or {})
    r = subprocess.run([sys.executable, "-m", *args], cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, (args, r.stdout[-1500:], r.stderr[-3000:])
    return r.stdout + r.stderr


def test_toy_pipeline_end_to_end(tmp_path):
    import pyarrow as pa
    import pyarrow.parquet as pq
    base = str(tmp_path / "nanochat")
    data = os.path.join(base, "base_data_climbmix")
    os.makedirs(data)
    rnd = random.Random(0)
    words = ("the quick brown fox jumps over lazy dog and then runs far away from home while it rains hard on every "
             "street of town").split()
    for i in range(3):                                       # the last shard is the validation split
        docs = [" ".join(rnd.choice(words) for _ in range(rnd.randint(30, 200))) + "." for _ in range(600)]
        pq.write_table(pa.table({"text": docs}), os.path.join(data, f"shard_{i:05d}.parquet"), row_group_size=100)

    out = _run(base, "scripts.tok_train", "--max-chars=300000", "--vocab-size=512")
    assert os.path.exists(os.path.join(base, "tokenizer", "tokenizer.pkl"))
    assert os.path.exists(os.path.join(base, "tokenizer", "token_bytes.pt"))
    out = _run(base, "scripts.tok_eval")           # the comparison vocabularies need a network: reported, not fatal
    assert re.search(r"Ours: \d+", out) and "GPT-2" in out

    train_args = ["scripts.base_train", "--depth=2", "--head-dim=64", "--window-pattern=L", "--max-seq-len=64",
                  "--device-batch-size=4", "--total-batch-size=512", "--eval-tokens=1024", "--core-metric-every=-1",
                  "--sample-every=-1", "--device-type=cpu"]
    out = _run(base, *train_args, "--num-iterations=4", "--eval-every=2", "--log-every=2",
               extra_env={"NANOCHAT_TRACE": "1"})
    bpbs = [float(x) for x in re.findall(r"Validation bpb: ([0-9.]+)", out)]
    assert len(bpbs) == 3 and bpbs[-1] < bpbs[0], bpbs       # it learns, even in four steps
    # the lines the sweep scripts (runs/miniseries.sh, runs/scaling_laws.sh) scrape out of the log
    for pattern in (r"^total +: [\d,]+$", r"^transformer_matrices +: [\d,]+$", r"^lm_head +: [\d,]+$",
                    r"number of iterations.*: [\d,]+$", r"Total batch size [\d,]+", r"Validation bpb: [\d.]+$"):
        assert re.search(pattern, out, re.M), pattern
    assert re.search(r"phases \(device ms, max over ranks\): forward: [0-9.]+ \| backward: [0-9.]+ \| optimizer:", out)
    from nanochat_b200.utils.trace import read_metrics
    recs = read_metrics(os.path.join(base, "metrics", "base_train_d2.jsonl"))
    assert recs[0]["event"] == "run_start" and recs[0]["config"]["depth"] == 2
    train = [r for r in recs if "train/loss" in r]
    assert [r["step"] for r in train] == [0, 2] and all(r["train/forward_ms"] > 0 for r in train)
    assert any("val/bpb" in r for r in recs)
    ck = os.path.join(base, "base_checkpoints", "d2")
    assert sorted(os.listdir(ck)) == ["meta_000004.json", "model_000004.pt", "optim_000004_rank0.pt"]

    _write_eval_bundle(base)
    resume_args = [a for a in train_args if not a.startswith("--core-metric-every")]
    out = _run(base, *resume_args, "--num-iterations=6", "--eval-every=-1", "--resume-from-step=4",
               "--core-metric-every=5", "--core-metric-max-per-task=4")
    assert "Resuming optimization from step 4" in out and "step 00005/00006" in out and "step 00003/" not in out
    assert len(re.findall(r"CORE metric: -?[0-9.]+", out)) == 2          # at step 5 and at the last step

    out = _run(base, "scripts.base_eval", "--eval", "core,bpb,sample", "--device-batch-size=2", "--split-tokens=1024",
               "--max-per-task=5", "--device-type=cpu")
    assert re.search(r"val bpb: [0-9.]+", out)
    assert len(re.findall(r"accuracy: [0-9.]+ \| centered: -?[0-9.]+", out)) == 3
    assert re.search(r"CORE metric: -?[0-9.]+$", out, re.M)          # the line the sweep scripts scrape
    assert os.path.exists(os.path.join(base, "base_eval", "base_model_000006.csv"))

    out = _run(base, "scripts.chat_cli", "-i", "base", "-p", "the quick", "-t", "0.0", "--device-type=cpu")
    assert "Assistant:" in out

    out = _run(base, "scripts.chat_sft", "--synthetic-data", "--depth=2", "--num-iterations=3", "--max-seq-len=64",
               "--device-batch-size=2", "--total-batch-size=256", "--eval-every=-1", "--chatcore-every=-1",
               "--device-type=cpu")
    assert re.search(r"step 0000\d .*loss: [0-9.]+", out)

    # the real finetuning path: base checkpoint + optimizer warm start + task mixture, with the task datasets
    # placed in the local cache (no network); then task evaluation and RL on the finetuned model
    _write_task_data(base)
    out = _run(base, "scripts.chat_sft", "--num-iterations=3", "--device-batch-size=2", "--total-batch-size=256",
               "--eval-every=2", "--eval-tokens=256", "--chatcore-every=-1", "--device-type=cpu")
    assert "Inherited max_seq_len=64" in out and "Loaded optimizer state from pretrained checkpoint" in out
    assert re.search(r"Training mixture: \d+ rows", out) and re.search(r"step 0000\d .*loss: [0-9.]+", out)
    assert os.path.isdir(os.path.join(base, "chatsft_checkpoints", "d2"))
    out = _run(base, "scripts.chat_eval", "-i", "sft", "-x", "4", "-m", "8", "-b", "2", "--device-type=cpu")   # all tasks
    for name in ("ARC-Easy", "ARC-Challenge", "MMLU", "GSM8K", "HumanEval"):
        assert re.search(name + r" accuracy: [0-9.]+%", out), name
    assert re.search(r"ChatCORE metric: -?[0-9.]+", out)
    out = _run(base, "scripts.chat_rl", "--num-samples=2", "--device-batch-size=2", "--examples-per-step=2",
               "--max-new-tokens=8", "--eval-examples=2", "--eval-every=2", "--save-every=2", "--device-type=cpu")
    assert "Calculated number of steps: 4" in out and re.search(r"Step 0 \| Pass@1: [0-9.]+, Pass@2: [0-9.]+", out)
    assert re.search(r"Step 3/4 \|", out) or re.search(r"[Ss]tep 3", out)
    rl = os.path.join(base, "chatrl_checkpoints", "d2")
    assert any(f.startswith("model_") for f in os.listdir(rl))
    out = _run(base, "scripts.chat_cli", "-i", "rl", "-p", "2+2?", "-t", "0.0", "--device-type=cpu")
    assert "Assistant:" in out


def _write_eval_bundle(base):
    """A three-task stand-in for the CORE bundle (one task of each type), where `scripts.base_eval` looks for it."""
    import json
    d = os.path.join(base, "eval_bundle")
    os.makedirs(os.path.join(d, "eval_data"), exist_ok=True)
    tasks = [("toy_mc", "multiple_choice", 2, 25.0), ("toy_schema", "schema", 0, 50.0), ("toy_lm", "language_modeling", 1, 0.0)]
    with open(os.path.join(d, "core.yaml"), "w") as f:
        f.write("icl_tasks:\n")
        for label, kind, shots, _ in tasks:
            f.write(f"- label: {label}\n  dataset_uri: {label}.jsonl\n  num_fewshot: [{shots}]\n  icl_task_type: {kind}\n")
            if kind == "language_modeling":
                f.write("  continuation_delimiter: ' '\n")
    with open(os.path.join(d, "eval_meta_data.csv"), "w") as f:
        f.write("Eval Task,Task Category,Task Type,#shots,#datapoints,Random baseline,Centered Metric?\n")
        for label, kind, shots, base_acc in tasks:
            f.write(f"{label},toy,{kind},{shots},8,{base_acc},\n")
    rows = {
        "toy_mc": [{"query": f"the quick fox number {i} jumps", "choices": ["over", "far", "home", "rains"], "gold": i % 4}
                   for i in range(8)],
        "toy_schema": [{"context_options": [f"the dog {i}", f"the fox {i}"], "continuation": "runs far away", "gold": i % 2}
                       for i in range(8)],
        "toy_lm": [{"context": f"it rains hard on every street {i}", "continuation": "of town"} for i in range(8)],
    }
    for label, items in rows.items():
        with open(os.path.join(d, "eval_data", f"{label}.jsonl"), "w") as f:
            f.write("\n".join(json.dumps(r) for r in items) + "\n")


def _write_task_data(base):
    """Tiny stand-ins for the hub datasets, in the cache layout `tasks.common.load_hub_dataset` reads."""
    import json
    import pyarrow as pa
    import pyarrow.parquet as pq

    def put(repo, subset, split, table):
        d = os.path.join(base, "task_data", repo.replace("/", "--"), subset, split)
        os.makedirs(d, exist_ok=True)
        pq.write_table(table, os.path.join(d, "00000.parquet"))
        with open(os.path.join(d, "manifest.json"), "w") as f:
            json.dump(["00000.parquet"], f)

    def gsm(n, off):
        return pa.Table.from_pydict({
            "question": [f"What is {i + off} plus {i}?" for i in range(n)],
            "answer": [f"Add them: <<{i + off}+{i}={2 * i + off}>>{2 * i + off}\n#### {2 * i + off}" for i in range(n)]})
    talk = pa.Table.from_pylist([
        {"messages": ([{"role": "system", "content": "Be brief."}] if i % 3 == 0 else []) + [
            {"role": "user", "content": f"Say the number {i}."}, {"role": "assistant", "content": f"The number is {i}."},
            {"role": "user", "content": "Again?"}, {"role": "assistant", "content": f"{i}"}]}
        for i in range(40)])
    put("HuggingFaceTB/smol-smoltalk", "default", "train", talk)
    put("HuggingFaceTB/smol-smoltalk", "default", "test", talk.slice(0, 12))
    mmlu = pa.Table.from_pylist([
        {"question": f"Pick option {i % 4}.", "subject": "toy", "choices": ["zero", "one", "two", "three"], "answer": i % 4}
        for i in range(24)])
    put("cais/mmlu", "all", "auxiliary_train", mmlu)
    put("cais/mmlu", "all", "test", mmlu.slice(0, 8))
    put("openai/gsm8k", "main", "train", gsm(8, 1))
    put("openai/gsm8k", "main", "test", gsm(4, 3))
    arc = pa.Table.from_pylist([
        {"id": str(i), "question": f"Which is letter {'ABCD'[i % 4]}?",
         "choices": {"text": ["a", "b", "c", "d"], "label": ["A", "B", "C", "D"]}, "answerKey": "ABCD"[i % 4]}
        for i in range(6)])
    for split in ("train", "validation", "test"):
        put("allenai/ai2_arc", "ARC-Easy", split, arc)
        put("allenai/ai2_arc", "ARC-Challenge", split, arc)
    he = pa.Table.from_pylist([
        {"task_id": f"Toy/{i}", "prompt": f"def add{i}(a, b):\n    \"\"\"Return a + b + {i}.\"\"\"\n",
         "canonical_solution": f"    return a + b + {i}\n", "entry_point": f"add{i}",
         "test": f"def check(f):\n    assert f(1, 2) == {3 + i}\n"} for i in range(4)])
    put("openai/openai_humaneval", "openai_humaneval", "test", he)

