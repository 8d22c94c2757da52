"""
Pretraining data pipeline: parquet row groups -> tokenised documents -> BOS-aligned best-fit
packed rows -> pinned staging -> one asynchronous host-to-device copy per batch.

Packing rule (reference: nanochat/dataloader.py:74-161): every row of T+1 tokens starts a
document (hence with BOS); repeatedly place the LARGEST buffered document that still fits;
when none fits, crop the SHORTEST buffered document to fill the row exactly. No padding, about
a third of the tokens are lost to cropping at T=2048. Row groups are strided over ranks
(`rg = rank, rank + world, ...`) and the position (pq_idx, rg_idx, epoch) is reported with each
batch so training can resume approximately where it stopped.

B200-native differences: the packer is C++ (`_tok.pack_rows`, a length-indexed pool instead of
a Python scan per placement), batches are prepared by a background thread into a ring of pinned
buffers, and the H2D copy is issued on a side stream so it overlaps the previous step's
kernels; the consumer only waits on an event.
"""

import threading
import atexit
import queue

import torch
import pyarrow.parquet as pq

from nanochat_b200.common import get_dist_info
from nanochat_b200.dataset import list_parquet_files


def _document_batches(split, resume_state_dict, tokenizer_batch_size):
    """Infinite stream of (list of texts, (pq_idx, rg_idx, epoch)) for this rank."""
    _, rank, _, world = get_dist_info()
    paths = list_parquet_files(warn_on_legacy=(rank == 0 and split == "train"))
    assert len(paths) != 0, "No dataset parquet files found, did you run dataset.py?"
    paths = paths[:-1] if split == "train" else paths[-1:]
    resume_pq = resume_state_dict["pq_idx"] if resume_state_dict is not None else 0
    resume_rg = resume_state_dict["rg_idx"] if resume_state_dict is not None else None
    epoch = resume_state_dict.get("epoch", 1) if resume_state_dict is not None else 1
    first_pass = True
    while True:
        pq_idx = resume_pq if first_pass else 0
        while pq_idx < len(paths):
            pf = pq.ParquetFile(paths[pq_idx])
            if first_pass and resume_rg is not None and pq_idx == resume_pq:
                # continue with the stripe after the one that was in flight when the state was saved
                rg_idx = (resume_rg // world + 1) * world + rank
                if rg_idx >= pf.num_row_groups:
                    pq_idx += 1
                    continue
                resume_rg = None
            else:
                rg_idx = rank
            while rg_idx < pf.num_row_groups:
                texts = pf.read_row_group(rg_idx).column("text").to_pylist()
                for i in range(0, len(texts), tokenizer_batch_size):
                    yield texts[i:i + tokenizer_batch_size], (pq_idx, rg_idx, epoch)
                rg_idx += world
            pq_idx += 1
        first_pass = False
        epoch += 1


def pack_rows_python(doc_buffer, num_rows, row_capacity, refill, buffer_size):
    """Best-fit-crop packing in plain Python (oracle for the C++ packer). Mutates doc_buffer."""
    rows = torch.empty((num_rows, row_capacity), dtype=torch.long)
    for r in range(num_rows):
        pos = 0
        while pos < row_capacity:
            while len(doc_buffer) < buffer_size:
                refill()
            room = row_capacity - pos
            best, best_len = -1, 0
            for i, doc in enumerate(doc_buffer):
                n = len(doc)
                if n <= room and n > best_len:
                    best, best_len = i, n
            if best >= 0:
                doc = doc_buffer.pop(best)
                rows[r, pos:pos + len(doc)] = torch.tensor(doc, dtype=torch.long)
                pos += len(doc)
            else:
                shortest = min(range(len(doc_buffer)), key=lambda i: len(doc_buffer[i]))
                doc = doc_buffer.pop(shortest)
                rows[r, pos:] = torch.tensor(doc[:room], dtype=torch.long)
                pos = row_capacity
    return rows


def _cpp_packer():
    try:
        from nanochat_b200.utils.build import load_tokenizer_extension
        return load_tokenizer_extension()
    except Exception:
        return None


def tokenizing_distributed_data_loader_with_state_bos_bestfit(
        tokenizer, B, T, split, tokenizer_threads=4, tokenizer_batch_size=128, device="cuda",
        resume_state_dict=None, buffer_size=1000, prefetch=2):
    """Yields (inputs (B,T) int64, targets (B,T) int64, state_dict) forever."""
    assert split in ("train", "val"), "split must be 'train' or 'val'"
    row_capacity = T + 1
    batches = _document_batches(split, resume_state_dict, tokenizer_batch_size)
    bos = tokenizer.get_bos_token_id()
    state = {"pq_idx": 0, "rg_idx": 0, "epoch": 1}
    doc_buffer = []
    cpp = _cpp_packer()
    packer = cpp.BestFitPacker(row_capacity, buffer_size) if cpp is not None else None

    def refill():
        texts, (state["pq_idx"], state["rg_idx"], state["epoch"]) = next(batches)
        docs = tokenizer.encode(texts, prepend=bos, num_threads=tokenizer_threads)
        if packer is not None:
            packer.add_documents(docs)
        else:
            doc_buffer.extend(docs)

    use_cuda = torch.device(device).type == "cuda"
    n_slots = prefetch + 1
    pinned = [torch.empty(2 * B * T, dtype=torch.long, pin_memory=use_cuda) for _ in range(n_slots)]
    on_dev = [torch.empty(2 * B * T, dtype=torch.long, device=device) for _ in range(n_slots)]
    copy_stream = torch.cuda.Stream() if use_cuda else None
    # released[slot]: recorded on the consumer's stream when it is done issuing work on that slot's batch. Host-side
    # queue order alone does not stop a later copy from overwriting a batch whose kernels are still queued (the
    # embedding backward reads the token ids last), so the copy stream waits for this event before it refills a slot.
    released = [None] * n_slots

    def build(slot):
        if packer is not None:
            while packer.needs_documents():
                refill()
            rows = torch.from_numpy(packer.pack(B, refill))
        else:
            rows = pack_rows_python(doc_buffer, B, row_capacity, refill, buffer_size)
        host = pinned[slot]
        host[:B * T].view(B, T).copy_(rows[:, :-1])
        host[B * T:].view(B, T).copy_(rows[:, 1:])
        return dict(state)

    ready = queue.Queue(maxsize=prefetch)
    free = queue.Queue()
    for s in range(n_slots):
        free.put(s)
    stop = threading.Event()

    def hand_over(item):
        while not stop.is_set():
            try:
                ready.put(item, timeout=0.2)
                return
            except queue.Full:
                continue

    def worker():
        try:
            while not stop.is_set():
                slot = free.get()
                if slot is None:
                    return
                snapshot = build(slot)
                hand_over((slot, snapshot, None))
        except BaseException as e:   # surface loader failures in the training thread
            hand_over((None, None, e))

    thread = threading.Thread(target=worker, daemon=True)
    thread.start()

    def shutdown():
        """Stop the producer and wait for it: a daemon thread that is inside the C++ tokenizer when the interpreter
        finalises is unwound through frames that own running std::threads, which aborts the process."""
        if stop.is_set():
            return
        stop.set()
        free.put(None)
        thread.join(timeout=30)
        live = _live_loaders              # None once the module has been torn down at interpreter exit
        if live is not None and shutdown in live:
            live.remove(shutdown)

    _live_loaders.append(shutdown)
    try:
        previous = None
        while True:
            slot, snapshot, err = ready.get()
            if err is not None:
                raise err
            dst = on_dev[slot]
            if use_cuda:
                if released[slot] is not None:
                    copy_stream.wait_event(released[slot])
                with torch.cuda.stream(copy_stream):
                    dst.copy_(pinned[slot], non_blocking=True)
                    done = torch.cuda.Event()
                    done.record(copy_stream)
                torch.cuda.current_stream().wait_event(done)
                done.synchronize()          # the pinned slot may be refilled once the copy has landed
            else:
                dst.copy_(pinned[slot])
            if previous is not None:
                if use_cuda:                # everything the consumer queued on the previous batch is ahead of this mark
                    released[previous] = torch.cuda.Event()
                    released[previous].record(torch.cuda.current_stream())
                free.put(previous)          # the consumer is done with the batch handed out before this one
            previous = slot
            yield dst[:B * T].view(B, T), dst[B * T:].view(B, T), snapshot
    finally:
        shutdown()


_live_loaders = []


@atexit.register
def _stop_loaders_at_exit():
    for shutdown in list(_live_loaders):
        shutdown()


def tokenizing_distributed_data_loader_bos_bestfit(*args, **kwargs):
    for inputs, targets, _ in tokenizing_distributed_data_loader_with_state_bos_bestfit(*args, **kwargs):
        yield inputs, targets


def synthetic_token_loader(B, T, vocab_size, device="cuda", seed=0, cycle=0):
    """Uniform-random token batches of the training shape (for benchmarks without a corpus). `cycle` > 0 repeats
    the first `cycle` batches forever (a memorisable stream: tests use it to see the loss fall)."""
    _, rank, _, _ = get_dist_info()
    gen = torch.Generator(device="cpu").manual_seed(seed + rank)
    state = {"pq_idx": 0, "rg_idx": 0, "epoch": 1}
    use_cuda = torch.device(device).type == "cuda"
    kept = []
    i = 0
    while True:
        if cycle > 0 and len(kept) == cycle:
            rows = kept[i % cycle]
        else:
            rows = torch.randint(0, vocab_size, (B, T + 1), generator=gen, dtype=torch.long)
            if use_cuda:
                rows = rows.pin_memory()
            if cycle > 0:
                kept.append(rows)
        i += 1
        dev_rows = rows.to(device, non_blocking=use_cuda)
        yield dev_rows[:, :-1].contiguous(), dev_rows[:, 1:].contiguous(), state
