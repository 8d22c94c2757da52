"""
Repackage a local text corpus into the shard format the pretraining loader reads.

The reference documents how its hosted corpus was produced (reference: dev/repackage_data_reference.py:78-104:
shuffle, `text` column, row groups of 1024 documents, zstd level 3, about 250 M characters per shard) but the
script only works against a dataset hub. This tool does the same job for files you already have, so the whole
pipeline runs without a network:

    python -m scripts.repackage_data corpus_dir/ more.jsonl --out-dir ~/.cache/nanochat/base_data_climbmix

Inputs (files or directories, searched recursively): `.txt` (one document per line, or the whole file as one
document with --whole-files), `.jsonl` (one object per line, the document in --text-key), `.parquet` (the
document column named --text-key). Documents are shuffled with a seeded buffer (memory stays bounded on
corpora larger than RAM), cut into shards of --chars-per-shard characters whose document count is a multiple of
the row-group size, and written as `shard_%05d.parquet`. The last shard written is the validation split, as
everywhere else in this code base; unlike the reference script, the documents left over at the end are kept
(they form that last shard). A `manifest.json` records what was written.
"""

import argparse
import json
import os
import random
import sys
import time

import pyarrow as pa
import pyarrow.parquet as pq

ROW_GROUP_SIZE = 1024
CHARS_PER_SHARD = 250_000_000


def find_inputs(paths):
    out = []
    for p in paths:
        if os.path.isdir(p):
            for root, _, names in sorted(os.walk(p)):
                out += [os.path.join(root, n) for n in sorted(names) if n.endswith((".txt", ".jsonl", ".parquet"))]
        elif os.path.exists(p):
            out.append(p)
        else:
            raise FileNotFoundError(p)
    return out


def iter_documents(paths, text_key="text", whole_files=False):
    """Every non-empty document of the inputs, in file order."""
    for path in paths:
        if path.endswith(".parquet"):
            pf = pq.ParquetFile(path)
            for rg in range(pf.num_row_groups):
                for doc in pf.read_row_group(rg, columns=[text_key]).column(text_key).to_pylist():
                    if doc:
                        yield doc
        elif path.endswith(".jsonl"):
            with open(path, encoding="utf-8") as f:
                for line in f:
                    line = line.strip()
                    if line:
                        doc = json.loads(line).get(text_key)
                        if doc:
                            yield doc
        elif whole_files:
            with open(path, encoding="utf-8", errors="replace") as f:
                doc = f.read()
            if doc.strip():
                yield doc
        else:
            with open(path, encoding="utf-8", errors="replace") as f:
                for line in f:
                    line = line.rstrip("\n")
                    if line.strip():
                        yield line


def shuffled(docs, buffer_size, seed):
    """Seeded streaming shuffle: fill a buffer, then swap every arrival with a random resident. With a buffer
    at least as large as the corpus this is a uniform permutation."""
    rng = random.Random(seed)
    buf = []
    for doc in docs:
        if len(buf) < buffer_size:
            buf.append(doc)
            continue
        i = rng.randrange(buffer_size)
        buf[i], doc = doc, buf[i]
        yield doc
    rng.shuffle(buf)
    yield from buf


def write_shard(out_dir, index, docs, row_group_size):
    path = os.path.join(out_dir, f"shard_{index:05d}.parquet")
    tmp = path + ".tmp"
    pq.write_table(pa.Table.from_pydict({"text": docs}), tmp, row_group_size=row_group_size, use_dictionary=False,
                   compression="zstd", compression_level=3, write_statistics=False)
    os.replace(tmp, path)
    return path


def repackage(inputs, out_dir, chars_per_shard=CHARS_PER_SHARD, row_group_size=ROW_GROUP_SIZE, seed=42,
              shuffle_buffer=1_000_000, text_key="text", whole_files=False, log=print):
    """Returns the manifest (also written to `<out_dir>/manifest.json`)."""
    os.makedirs(out_dir, exist_ok=True)
    existing = [n for n in os.listdir(out_dir) if n.endswith(".parquet")]
    if existing:
        raise FileExistsError(f"{out_dir} already holds {len(existing)} shards; choose an empty directory")
    files = find_inputs(inputs)
    docs = iter_documents(files, text_key, whole_files)
    if shuffle_buffer > 0:
        docs = shuffled(docs, shuffle_buffer, seed)
    shards, cur, cur_chars, t0 = [], [], 0, time.time()

    def flush():
        nonlocal cur, cur_chars, t0
        path = write_shard(out_dir, len(shards), cur, row_group_size)
        shards.append({"file": os.path.basename(path), "documents": len(cur), "characters": cur_chars})
        log(f"Wrote {path}. #documents: {len(cur)} | #characters: {cur_chars} | time: {time.time() - t0:.2f}s")
        cur, cur_chars, t0 = [], 0, time.time()

    for doc in docs:
        cur.append(doc)
        cur_chars += len(doc)
        if cur_chars >= chars_per_shard and len(cur) % row_group_size == 0:
            flush()
    if cur:
        flush()                      # the remainder: kept, and as the last shard it is the validation split
    if len(shards) < 2:
        log("WARNING: fewer than two shards were written; the loader needs at least one training shard and the "
            "validation shard (lower --chars-per-shard)")
    manifest = {"inputs": files, "seed": seed, "shuffle_buffer": shuffle_buffer, "row_group_size": row_group_size,
                "chars_per_shard": chars_per_shard, "shards": shards,
                "documents": sum(s["documents"] for s in shards), "characters": sum(s["characters"] for s in shards),
                "validation_shard": shards[-1]["file"] if shards else None}
    with open(os.path.join(out_dir, "manifest.json"), "w") as f:
        json.dump(manifest, f, indent=2)
    return manifest


def main(argv=None):
    from nanochat_b200.dataset import data_dir
    ap = argparse.ArgumentParser(description="Repackage local text into pretraining shards")
    ap.add_argument("inputs", nargs="+", help="files or directories (.txt, .jsonl, .parquet)")
    ap.add_argument("--out-dir", default=None, help="default: the directory the pretraining loader reads")
    ap.add_argument("--chars-per-shard", type=int, default=CHARS_PER_SHARD)
    ap.add_argument("--row-group-size", type=int, default=ROW_GROUP_SIZE)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--shuffle-buffer", type=int, default=1_000_000, help="documents held for the shuffle (0 = keep order)")
    ap.add_argument("--text-key", default="text")
    ap.add_argument("--whole-files", action="store_true", help="a .txt file is one document, not one per line")
    args = ap.parse_args(argv)
    m = repackage(args.inputs, args.out_dir or data_dir(), args.chars_per_shard, args.row_group_size, args.seed,
                  args.shuffle_buffer, args.text_key, args.whole_files)
    print(f"{len(m['shards'])} shards, {m['documents']:,} documents, {m['characters']:,} characters; "
          f"validation shard: {m['validation_shard']}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
