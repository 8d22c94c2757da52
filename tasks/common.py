"""
Task plumbing: a Task is an indexable view over a dataset of conversations (plus an
optional scorer); mixtures and sequences compose tasks for finetuning.

Behaviour mirrors the reference (tasks/common.py): `HubDataset.shuffle(seed)` is exactly
`numpy.random.default_rng(seed).permutation(n)` (what HuggingFace `datasets` does, so row
order matches runs made with that library); `load_hub_dataset` reads the hub's parquet
export into `<base>/task_data/<repo--id>/<subset>/<split>/` once, guarded by a file lock;
`Task` slicing uses ceil-division length; `TaskMixture` interleaves with a seed-42 shuffle.
"""

import os
import json
import random
import urllib.request

import numpy as np
import pyarrow as pa
import pyarrow.parquet as pq

from nanochat_b200.common import get_base_dir


class HubDataset:
    """A pyarrow table with lazy dict rows and an optional row permutation."""

    def __init__(self, table, permutation=None):
        self.table = table
        self.permutation = permutation

    def __len__(self):
        return self.table.num_rows

    def shuffle(self, seed):
        return HubDataset(self.table, np.random.default_rng(seed).permutation(len(self)))

    def __getitem__(self, index):
        row = index if self.permutation is None else int(self.permutation[index])
        return {name: self.table[name][row].as_py() for name in self.table.column_names}


def load_hub_dataset(repo_id, subset="default", split="train"):
    """Download (once) and open the parquet export of a hub dataset split."""
    from filelock import FileLock
    shard_dir = os.path.join(get_base_dir(), "task_data", repo_id.replace("/", "--"), subset, split)
    manifest = os.path.join(shard_dir, "manifest.json")
    if not os.path.exists(manifest):
        os.makedirs(shard_dir, exist_ok=True)
        with FileLock(manifest + ".lock"):
            if not os.path.exists(manifest):   # we hold the lock and nobody finished before us
                api = f"https://huggingface.co/api/datasets/{repo_id}/parquet/{subset}/{split}"
                with urllib.request.urlopen(api) as resp:
                    urls = json.loads(resp.read())
                names = []
                for i, url in enumerate(urls):
                    name = f"{i:05d}.parquet"
                    print(f"Downloading {url} ...")
                    with urllib.request.urlopen(url) as resp:
                        blob = resp.read()
                    with open(os.path.join(shard_dir, name), "wb") as f:
                        f.write(blob)
                    names.append(name)
                with open(manifest, "w") as f:
                    json.dump(names, f)
    with open(manifest) as f:
        names = json.load(f)
    return HubDataset(pa.concat_tables([pq.read_table(os.path.join(shard_dir, n)) for n in names]))


class Task:
    """Indexable view `[start:stop:step]` over `num_examples()` conversations."""

    def __init__(self, start=0, stop=None, step=1):
        assert start >= 0, f"Start must be non-negative, got {start}"
        assert stop is None or stop >= start, f"Stop should be greater than or equal to start, got {stop} and {start}"
        assert step >= 1, f"Step must be strictly positive, got {step}"
        self.start, self.stop, self.step = start, stop, step

    @property
    def eval_type(self):
        raise NotImplementedError

    def num_examples(self):
        raise NotImplementedError

    def get_example(self, index):
        raise NotImplementedError

    def evaluate(self, problem, completion):
        raise NotImplementedError

    def __len__(self):
        # a stop beyond the data (a fixed evaluation budget on a smaller dataset) ends at the data
        stop = self.num_examples() if self.stop is None else min(self.stop, self.num_examples())
        n = -(-(stop - self.start) // self.step)
        assert n >= 0, f"Negative number of examples???: {n}"
        return n

    def __getitem__(self, index: int):
        assert isinstance(index, int), f"Index must be an integer, got {type(index)}"
        return self.get_example(self.start + index * self.step)


class TaskMixture(Task):
    """Union of tasks in a fixed pseudo-random order; list a task twice to oversample it."""

    def __init__(self, tasks, **kwargs):
        super().__init__(**kwargs)
        self.tasks = tasks
        self.lengths = [len(t) for t in tasks]
        self.num_conversations = sum(self.lengths)
        self.index_map = [(ti, li) for ti, n in enumerate(self.lengths) for li in range(n)]
        random.Random(42).shuffle(self.index_map)

    def num_examples(self):
        return self.num_conversations

    def get_example(self, index):
        assert 0 <= index < self.num_conversations, (
            f"Index {index} out of range for mixture with {self.num_conversations} conversations")
        ti, li = self.index_map[index]
        return self.tasks[ti][li]


class TaskSequence(Task):
    """Tasks back to back (a curriculum)."""

    def __init__(self, tasks, **kwargs):
        super().__init__(**kwargs)
        self.tasks = tasks
        self.lengths = [len(t) for t in tasks]
        self.num_conversations = sum(self.lengths)

    def num_examples(self):
        return self.num_conversations

    def get_example(self, index):
        assert 0 <= index < self.num_conversations, (
            f"Index {index} out of range for sequence with {self.num_conversations} conversations")
        for task, n in zip(self.tasks, self.lengths):
            if index < n:
                return task[index]
            index -= n


def render_mc(question, letters, choices):
    """Multiple-choice prompt. The letter follows '=' with no space so the prompt contains the very
    token ("A", not " A") the assistant must answer with; small models are sensitive to that."""
    lines = [f"Multiple Choice question: {question}\n"]
    lines += [f"- {choice}={letter}\n" for letter, choice in zip(letters, choices)]
    lines.append("\nRespond only with the letter of the correct answer.")
    return "".join(lines)


if __name__ == "__main__":
    from tasks.mmlu import MMLU
    full = MMLU(subset="all", split="auxiliary_train")
    part = MMLU(subset="all", split="auxiliary_train", start=5, stop=10)
    print("MMLU:", len(full), "slice:", len(part), "match:", full[5] == part[0])
