"""Task containers: slicing views, mixtures, the parquet-backed dataset wrapper (no network)."""
import numpy as np
import pyarrow as pa

from tasks.common import Task, TaskMixture, TaskSequence, HubDataset, render_mc


class Toy(Task):
    def __init__(self, n=10, tag="a", **kw):
        super().__init__(**kw)
        self.n, self.tag = n, tag

    def num_examples(self):
        return self.n

    def get_example(self, index):
        return {"i": index, "tag": self.tag}


def test_full_and_sliced_views():
    assert len(Toy(10)) == 10 and Toy(10)[9] == {"i": 9, "tag": "a"}
    t = Toy(10, start=5, stop=10)
    assert len(t) == 5 and t[0]["i"] == 5
    t = Toy(10, start=0, stop=10, step=3)
    assert len(t) == 4 and [t[i]["i"] for i in range(4)] == [0, 3, 6, 9]
    assert len(Toy(10, stop=5200)) == 10 and len(Toy(10, start=4, stop=5200, step=2)) == 3      # stop ends at the data


def test_mixture_is_a_deterministic_interleaved_permutation():
    mk = lambda: TaskMixture([Toy(3, "a"), Toy(5, "b")])
    ex = [mk()[i] for i in range(8)]
    assert sorted((e["tag"], e["i"]) for e in ex) == [("a", i) for i in range(3)] + [("b", i) for i in range(5)]
    assert ex == [mk()[i] for i in range(8)]
    assert [e["tag"] for e in ex] != ["a"] * 3 + ["b"] * 5
    assert len(TaskMixture([Toy(3), Toy(3)])) == 6


def test_sequence_keeps_order():
    seq = TaskSequence([Toy(2, "a"), Toy(3, "b")])
    assert [seq[i]["tag"] for i in range(5)] == ["a", "a", "b", "b", "b"]


def test_hub_dataset_rows_and_numpy_shuffle():
    table = pa.table({"x": list(range(100)), "y": [str(i) for i in range(100)]})
    ds = HubDataset(table)
    assert len(ds) == 100 and ds[7] == {"x": 7, "y": "7"}
    perm = np.random.default_rng(42).permutation(100)
    sh = ds.shuffle(seed=42)
    assert [sh[i]["x"] for i in range(100)] == [int(p) for p in perm]
    assert ds[0]["x"] == 0


def test_render_mc_binds_letter_without_space():
    q = render_mc("What is 1+1?", ("A", "B"), ("1", "2"))
    assert "=A\n" in q and "=B\n" in q


def test_gsm8k_parsing_helpers():
    from tasks.gsm8k import extract_answer
    assert extract_answer("so the total is\n#### 1,234") == "1234"
    assert extract_answer("no marker") is None
