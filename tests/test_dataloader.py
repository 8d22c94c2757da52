"""Best-fit packing (C++ vs Python oracle) and the parquet -> batch pipeline on a tiny local corpus."""
import os
import random

import pyarrow as pa
import pyarrow.parquet as pq
import pytest
import torch

from nanochat_b200 import dataloader as dl


def _docs(seed, n, lo=2, hi=300):
    rng = random.Random(seed)
    return [[rng.randrange(1000) for _ in range(rng.randint(lo, hi))] for _ in range(n)]


def test_cpp_packer_matches_python_oracle():
    tok = pytest.importorskip("nanochat_b200.utils.build").load_tokenizer_extension()
    cap, buf = 129, 50
    feed_a, feed_b = iter(_docs(1, 5000)), iter(_docs(1, 5000))
    pool = []
    packer = tok.BestFitPacker(cap, buf)
    refill_py = lambda: pool.extend(next(feed_a) for _ in range(7))
    refill_cpp = lambda: packer.add_documents([next(feed_b) for _ in range(7)])
    for _ in range(5):
        want = dl.pack_rows_python(pool, 8, cap, refill_py, buf)
        got = torch.from_numpy(packer.pack(8, refill_cpp))
        assert torch.equal(want, got)


def test_rows_start_documents_and_are_full():
    cap, buf = 65, 20
    bos = 999999
    feed = iter([[bos] + d for d in _docs(2, 3000, 1, 200)])
    pool = []
    rows = dl.pack_rows_python(pool, 16, cap, lambda: pool.append(next(feed)), buf)
    assert rows.shape == (16, cap) and (rows[:, 0] == bos).all()


class _ByteTok:
    def get_bos_token_id(self):
        return 256

    def encode(self, texts, prepend=None, num_threads=1):
        return [([prepend] if prepend is not None else []) + list(t.encode()) for t in texts]


def test_loader_shapes_shift_and_resume_state(tmp_path, monkeypatch):
    monkeypatch.setenv("NANOCHAT_BASE_DIR", str(tmp_path))
    d = tmp_path / "base_data_climbmix"
    os.makedirs(d)
    rng = random.Random(0)
    for shard in range(3):
        texts = ["".join(rng.choice("abcdefgh ") for _ in range(rng.randint(5, 120))) for _ in range(64)]
        pq.write_table(pa.table({"text": texts}), d / f"shard_{shard:05d}.parquet", row_group_size=16)
    loader = dl.tokenizing_distributed_data_loader_with_state_bos_bestfit(
        _ByteTok(), B=4, T=32, split="train", device="cpu", buffer_size=16, tokenizer_batch_size=8)
    x, y, state = next(loader)
    assert x.shape == (4, 32) and y.shape == (4, 32) and x.dtype == torch.long
    assert torch.equal(x[:, 1:], y[:, :-1]) and (x[:, 0] == 256).all()
    assert set(state) == {"pq_idx", "rg_idx", "epoch"} and state["epoch"] == 1
    for _ in range(40):                      # runs past the two training shards -> next epoch
        x, y, state = next(loader)
    assert state["epoch"] >= 2
    val = dl.tokenizing_distributed_data_loader_bos_bestfit(_ByteTok(), 2, 16, "val", device="cpu", buffer_size=8)
    vx, vy = next(val)
    assert vx.shape == (2, 16)
    resumed = dl._document_batches("train", {"pq_idx": 1, "rg_idx": 1, "epoch": 3}, 8)
    _, (pq_idx, rg_idx, epoch) = next(resumed)
    assert (pq_idx, rg_idx, epoch) == (1, 2, 3)


def test_repackaged_corpus_is_read_back_by_the_loader(tmp_path, monkeypatch):
    """Local files -> shards -> the loader's row-group iterator: nothing lost, last shard is validation."""
    import json
    import pyarrow.parquet as pq
    from scripts import repackage_data as rp
    from nanochat_b200 import dataset
    src = tmp_path / "src"
    src.mkdir()
    docs_txt = [f"line document {i} " + "x" * (i % 50) for i in range(700)]
    (src / "a.txt").write_text("\n".join(docs_txt) + "\n\n")
    docs_jsonl = [f"json document {i}\nwith a second line" for i in range(300)]
    (src / "b.jsonl").write_text("\n".join(json.dumps({"text": d, "other": i}) for i, d in enumerate(docs_jsonl)))
    base = tmp_path / "base"
    monkeypatch.setenv("NANOCHAT_BASE_DIR", str(base))
    out = dataset.data_dir()
    m = rp.repackage([str(src)], out, chars_per_shard=6000, row_group_size=64, seed=1, shuffle_buffer=256, log=lambda s: None)
    assert m["documents"] == 1000 and len(m["shards"]) >= 3 and m["validation_shard"] == m["shards"][-1]["file"]
    for s in m["shards"][:-1]:
        assert s["documents"] % 64 == 0 and s["characters"] >= 6000
    assert pq.ParquetFile(os.path.join(out, "shard_00000.parquet")).metadata.row_group(0).num_rows == 64
    train = [d for batch in dataset.parquets_iter_batched("train") for d in batch]
    val = [d for batch in dataset.parquets_iter_batched("val") for d in batch]
    assert sorted(train + val) == sorted(docs_txt + docs_jsonl) and len(val) == m["shards"][-1]["documents"]
    assert train[:50] != (docs_txt + docs_jsonl)[:50]                      # shuffled
    two = [d for r in range(2) for batch in dataset.parquets_iter_batched("train", start=r, step=2) for d in batch]
    assert sorted(two) == sorted(train)                                    # rank striding covers every row group once
    again = tmp_path / "again"
    m2 = rp.repackage([str(src)], str(again), chars_per_shard=6000, row_group_size=64, seed=1, shuffle_buffer=256,
                      log=lambda s: None)
    assert m2["shards"] == m["shards"]                                     # same seed, same shards
    with pytest.raises(FileExistsError):
        rp.repackage([str(src)], out, log=lambda s: None)


_EXIT_WORKER = r"""
import os, random, sys
sys.path.insert(0, sys.argv[1])
os.environ["NANOCHAT_BASE_DIR"] = sys.argv[2]
import pyarrow as pa, pyarrow.parquet as pq
from nanochat_b200 import dataset, dataloader as dl
from nanochat_b200.tokenizer import BPETokenizer
rnd = random.Random(0)
words = [("w%d" % i) * rnd.randint(1, 3) for i in range(400)]
os.makedirs(dataset.data_dir())
for s in range(2):
    docs = [" ".join(rnd.choice(words) for _ in range(rnd.randint(200, 900))) for _ in range(800)]
    pq.write_table(pa.table({"text": docs}), os.path.join(dataset.data_dir(), "shard_%05d.parquet" % s), row_group_size=128)
tok = BPETokenizer.train_from_iterator((d for b in dataset.parquets_iter_batched("train") for d in b), 600)
loader = dl.tokenizing_distributed_data_loader_with_state_bos_bestfit(tok, 8, 512, "train", device="cpu")
for _ in range(int(sys.argv[3])):
    x, y, state = next(loader)
assert x.shape == (8, 512)
print("leaving with the loader alive")
# no close(), no del: the interpreter exits while the producer thread is busy tokenising
"""


@pytest.mark.parametrize("batches", [1, 7, 20])
def test_process_exits_cleanly_with_a_live_loader(tmp_path, batches):
    import subprocess
    import sys
    script = tmp_path / "w.py"
    script.write_text(_EXIT_WORKER)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, str(script), root, str(tmp_path / "base"), str(batches)], capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 0 and "leaving with the loader alive" in r.stdout, (r.returncode, r.stderr[-2000:])
    assert "terminate called" not in r.stderr, r.stderr[-2000:]
