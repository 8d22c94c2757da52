"""
Pretraining corpus: ClimbMix-400B repackaged as parquet shards `shard_%05d.parquet` with one
`text` column; the highest-numbered shard is the validation split.

  python -m nanochat_b200.dataset -n 170        # fetch 170 training shards + the validation shard

Listing, row-group iteration and the download policy (temp file + rename, five attempts with
exponential back-off, a worker pool) follow the reference (nanochat/dataset.py:23-160).
"""

import os
import time
import argparse

import pyarrow.parquet as pq

from nanochat_b200.common import get_base_dir

BASE_URL = "https://huggingface.co/datasets/karpathy/climbmix-400b-shuffle/resolve/main"
MAX_SHARD = 6542   # index of the last shard (the validation shard)


def __getattr__(name):
    """`DATA_DIR` and `base_dir` of the reference's module, resolved on access so that NANOCHAT_BASE_DIR set after the
    import is honoured."""
    if name == "DATA_DIR":
        return data_dir()
    if name == "base_dir":
        return get_base_dir()
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def index_to_filename(index):
    return f"shard_{index:05d}.parquet"


def data_dir():
    return os.path.join(get_base_dir(), "base_data_climbmix")


_default_data_dir = data_dir


def list_parquet_files(data_dir=None, warn_on_legacy=False):
    """Sorted full paths of the shards on disk. Falls back to the older `base_data` directory when the
    ClimbMix directory does not exist."""
    d = _default_data_dir() if data_dir is None else data_dir      # the parameter keeps the reference's name
    if not os.path.exists(d):
        if warn_on_legacy:
            print(f"WARNING: {d} not found; run `python -m nanochat_b200.dataset -n 170` and re-train the "
                  "tokenizer. Falling back to the legacy base_data directory.")
        d = os.path.join(get_base_dir(), "base_data")
    names = sorted(f for f in os.listdir(d) if f.endswith(".parquet") and not f.endswith(".tmp"))
    return [os.path.join(d, f) for f in names]


def parquets_iter_batched(split, start=0, step=1):
    """Yields lists of documents, one list per parquet row group; `start`/`step` stride row groups
    (rank / world size under data parallelism)."""
    assert split in ("train", "val"), "split must be 'train' or 'val'"
    paths = list_parquet_files()
    paths = paths[:-1] if split == "train" else paths[-1:]
    for path in paths:
        pf = pq.ParquetFile(path)
        for rg in range(start, pf.num_row_groups, step):
            yield pf.read_row_group(rg).column("text").to_pylist()


def download_single_file(index, max_attempts=5):
    """Fetch one shard; True on success (or if it is already there)."""
    import requests
    target = os.path.join(data_dir(), index_to_filename(index))
    if os.path.exists(target):
        print(f"Skipping {target} (already exists)")
        return True
    url = f"{BASE_URL}/{index_to_filename(index)}"
    print(f"Downloading {index_to_filename(index)}...")
    for attempt in range(1, max_attempts + 1):
        tmp = target + ".tmp"
        try:
            with requests.get(url, stream=True, timeout=30) as resp:
                resp.raise_for_status()
                with open(tmp, "wb") as f:
                    for chunk in resp.iter_content(chunk_size=1 << 20):
                        if chunk:
                            f.write(chunk)
            os.rename(tmp, target)
            print(f"Successfully downloaded {index_to_filename(index)}")
            return True
        except (requests.RequestException, IOError) as e:
            print(f"Attempt {attempt}/{max_attempts} failed for {index_to_filename(index)}: {e}")
            for leftover in (tmp, target):
                try:
                    os.remove(leftover)
                except OSError:
                    pass
            if attempt < max_attempts:
                time.sleep(2 ** attempt)
    print(f"Failed to download {index_to_filename(index)} after {max_attempts} attempts")
    return False


if __name__ == "__main__":
    from multiprocessing import Pool
    ap = argparse.ArgumentParser(description="Download pretraining dataset shards")
    ap.add_argument("-n", "--num-files", type=int, default=-1, help="number of train shards (-1 = all)")
    ap.add_argument("-w", "--num-workers", type=int, default=4)
    args = ap.parse_args()
    os.makedirs(data_dir(), exist_ok=True)
    n_train = MAX_SHARD if args.num_files == -1 else min(args.num_files, MAX_SHARD)
    ids = list(range(n_train)) + [MAX_SHARD]
    print(f"Downloading {len(ids)} shards using {args.num_workers} workers into {data_dir()}")
    with Pool(processes=args.num_workers) as pool:
        ok = pool.map(download_single_file, ids)
    print(f"Done! Downloaded: {sum(ok)}/{len(ids)} shards to {data_dir()}")
