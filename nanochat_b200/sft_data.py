"""
SFT batches: rendered conversations packed best-fit into rows of T+1 tokens, padded (never
cropped) when nothing fits, with the assistant-only loss mask folded into the targets.

Rules (reference: scripts/chat_sft.py:180-298): a buffer of 100 rendered conversations; each
row repeatedly takes the largest conversation that fits; when none fits the rest of the row is
filled with BOS tokens whose targets are -1; targets are also -1 wherever the render mask of
the TARGET token is 0; inputs are int32, targets int64. Conversations are dealt to ranks
round-robin (`cursor = rank, rank + world, ...`); progress is measured in conversations
actually placed, so the epoch ends when the data has been consumed, not when it was fetched.

`synthetic_conversations` provides the benchmark stand-in for a chat dataset: lengths uniform in
[64, 2048] with a Bernoulli(0.5) loss mask per turn.
"""

import random

import torch


class SFTState:
    """Progress shared between the generator and the training loop."""

    def __init__(self):
        self.last_step = False
        self.approx_progress = 0.0
        self.current_epoch = 1


def sft_batches(dataset, render, bos_token, B, T, rank=0, world=1, device="cpu", num_iterations=-1,
                state=None, track_progress=True, buffer_size=100):
    """Yields (inputs int32 (B,T), targets int64 (B,T)) forever. `render(conversation)` -> (ids, mask)."""
    n = len(dataset)
    assert n > 0
    cap = T + 1
    pool = []                 # (ids, mask)
    cursor = rank
    consumed = rank
    epoch = 1
    it = 0
    use_cuda = torch.device(device).type == "cuda"

    def refill():
        nonlocal cursor, epoch
        while len(pool) < buffer_size:
            pool.append(render(dataset[cursor]))
            cursor += world
            if cursor >= n:
                cursor %= n
                epoch += 1

    while True:
        rows, masks, content = [], [], []
        for _ in range(B):
            row, mrow = [], []
            filled = cap
            while len(row) < cap:
                if len(pool) < buffer_size:
                    refill()
                room = cap - len(row)
                best, best_len = -1, 0
                for i, (ids, _) in enumerate(pool):
                    if best_len < len(ids) <= room:
                        best, best_len = i, len(ids)
                if best < 0:
                    filled = len(row)
                    row += [bos_token] * room
                    mrow += [0] * room
                    break
                ids, m = pool.pop(best)
                row += ids
                mrow += m
                consumed += world
            rows.append(row[:cap])
            masks.append(mrow[:cap])
            content.append(filled)
        it += 1
        if state is not None and track_progress:
            if 0 < num_iterations <= it:
                state.last_step = True
            state.current_epoch = epoch
            state.approx_progress = it / num_iterations if num_iterations > 0 else consumed / n
            if consumed >= n:
                state.last_step = True
        batch = torch.tensor(rows, dtype=torch.long)
        mask = torch.tensor(masks, dtype=torch.int8)
        targets = batch[:, 1:].clone()
        targets[mask[:, 1:] == 0] = -1
        for r, c in enumerate(content):
            if c < cap:
                targets[r, max(c - 1, 0):] = -1
        inputs = batch[:, :-1].to(torch.int32)
        if use_cuda:
            inputs, targets = inputs.pin_memory(), targets.pin_memory()
        yield (inputs.to(device, non_blocking=use_cuda).contiguous(),
               targets.to(device, non_blocking=use_cuda).contiguous())


class synthetic_conversations:
    """Indexable set of pre-rendered (ids, mask) pairs: total length U[64, max_len], turns of 8..256
    tokens alternating user/assistant, each assistant turn supervised with probability 0.5."""

    def __init__(self, count, vocab_size, max_len=2048, seed=0, bos_token=0):
        rng = random.Random(seed)
        self.items = []
        for _ in range(count):
            total = rng.randint(64, max_len)
            ids, mask = [bos_token], [0]
            assistant = False
            while len(ids) < total:
                turn = min(rng.randint(8, 256), total - len(ids))
                supervised = 1 if (assistant and rng.random() < 0.5) else 0
                ids += [rng.randrange(1, vocab_size) for _ in range(turn)]
                mask += [supervised] * turn
                assistant = not assistant
            self.items.append((ids, mask))

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        return self.items[i]
