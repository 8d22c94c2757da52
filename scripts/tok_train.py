"""
Train the BPE tokenizer on the pretraining corpus and cache the per-token byte lengths.

    python -m scripts.tok_train --max-chars 2000000000 --vocab-size 32768

Writes <base>/tokenizer/tokenizer.pkl and token_bytes.pt (int32, 0 for special tokens), the two
files every other stage reads (reference: scripts/tok_train.py).
"""
import os
import time
import argparse

import torch

from nanochat_b200.common import get_base_dir
from nanochat_b200.dataset import parquets_iter_batched
from nanochat_b200.tokenizer import BPETokenizer


def token_byte_lengths(tokenizer):
    """int32 (vocab,) tensor: UTF-8 byte length of every ordinary token, 0 for special tokens."""
    special = {tokenizer.encode_special(s) for s in tokenizer.get_special_tokens()}
    lengths = [0 if t in special else len(tokenizer.decode_single_token_bytes(t))
               for t in range(tokenizer.get_vocab_size())]
    return torch.tensor(lengths, dtype=torch.int32, device="cpu")


def main():
    ap = argparse.ArgumentParser(description="Train a BPE tokenizer")
    ap.add_argument("--max-chars", type=int, default=2_000_000_000, help="characters of text to train on")
    ap.add_argument("--doc-cap", type=int, default=10_000, help="characters kept per document")
    ap.add_argument("--vocab-size", type=int, default=32768)
    args = ap.parse_args()
    print(f"max_chars: {args.max_chars:,}")
    print(f"doc_cap: {args.doc_cap:,}")
    print(f"vocab_size: {args.vocab_size:,}")

    def texts():
        seen = 0
        for batch in parquets_iter_batched(split="train"):
            for doc in batch:
                doc = doc[:args.doc_cap]
                seen += len(doc)
                yield doc
                if seen > args.max_chars:
                    return

    t0 = time.time()
    tokenizer = BPETokenizer.train_from_iterator(texts(), args.vocab_size)
    print(f"Training time: {time.time() - t0:.2f}s")
    tok_dir = os.path.join(get_base_dir(), "tokenizer")
    tokenizer.save(tok_dir)

    probe = "Hello world! This is a test.\nNumbers: 123, 4567, 89\nContractions: I'm, you're, it's\n" \
            "Special chars: @#$%^&*()\nUnicode: 你好世界 🌍"
    assert tokenizer.decode(tokenizer.encode(probe)) == probe, "tokenizer does not round-trip"

    path = os.path.join(tok_dir, "token_bytes.pt")
    with open(path, "wb") as f:
        torch.save(token_byte_lengths(tokenizer), f)
    print(f"Saved token_bytes to {path}")


if __name__ == "__main__":
    main()
