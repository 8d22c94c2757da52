"""
CORE metric (DCLM, arXiv:2406.11794): in-context evaluation of a base model on multiple-choice,
schema and language-modelling tasks.

Scoring rules follow the reference (nanochat/core_eval.py): few-shot examples are drawn with
`random.Random(1234 + idx)` from the other items; multiple-choice prompts share a prefix and
are scored by the lowest mean loss over the differing continuation; schema prompts share a
suffix (the continuation) and are scored the same way over that suffix; language-modelling
items count as correct when the argmax prediction reproduces every continuation token.
Examples are strided over ranks and the per-example results are summed across ranks.

Prompts are assembled with plain string formatting (the layouts are fixed: few-shot blocks
separated by a blank line), and the model is asked for per-position losses and argmax through
`forward_model`, which works with any callable returning (B, T, V) logits.
"""

import random

import torch
import torch.distributed as dist
import torch.nn.functional as F


def render_prompts_mc(item, continuation_delimiter, fewshot_examples=None):
    """One prompt per choice: shared few-shot block and query, differing answer."""
    shots = "".join(f"{ex['query']}{continuation_delimiter}{ex['choices'][ex['gold']]}\n\n"
                    for ex in (fewshot_examples or []))
    return [f"{shots}{item['query']}{continuation_delimiter}{choice}" for choice in item["choices"]]


def render_prompts_schema(item, continuation_delimiter, fewshot_examples=None):
    """One prompt per context option: differing context, shared continuation."""
    shots = "".join(f"{ex['context_options'][ex['gold']]}{continuation_delimiter}{ex['continuation']}\n\n"
                    for ex in (fewshot_examples or []))
    return [f"{shots}{ctx}{continuation_delimiter}{item['continuation']}" for ctx in item["context_options"]]


def render_prompts_lm(item, continuation_delimiter, fewshot_examples=None):
    """[prompt without continuation, prompt with continuation]; contexts are whitespace-trimmed so the
    first is a clean token prefix of the second."""
    shots = "".join(f"{str(ex['context']).strip()}{continuation_delimiter}{ex['continuation']}\n\n"
                    for ex in (fewshot_examples or []))
    stem = f"{shots}{str(item['context']).strip()}{continuation_delimiter}"
    return [stem.strip(), f"{stem}{item['continuation']}"]


def find_common_length(token_sequences, direction="left"):
    """Length of the common prefix ('left') or suffix ('right') of several token lists."""
    shortest = min(len(s) for s in token_sequences)
    first = token_sequences[0]
    for n in range(shortest):
        pos = n if direction == "left" else -1 - n
        if any(s[pos] != first[pos] for s in token_sequences):
            return n
    return shortest


def stack_sequences(tokens, pad_token_id):
    width = max(len(t) for t in tokens)
    out = torch.full((len(tokens), width), pad_token_id, dtype=torch.long)
    for i, t in enumerate(tokens):
        out[i, :len(t)] = torch.tensor(t, dtype=torch.long)
    return out


def batch_sequences_mc(tokenizer, prompts):
    tokens = tokenizer(prompts, prepend=tokenizer.get_bos_token_id())
    start = find_common_length(tokens, "left")
    return tokens, [start] * len(prompts), [len(t) for t in tokens]


def batch_sequences_schema(tokenizer, prompts):
    tokens = tokenizer(prompts, prepend=tokenizer.get_bos_token_id())
    suffix = find_common_length(tokens, "right")
    ends = [len(t) for t in tokens]
    return tokens, [e - suffix for e in ends], ends


def batch_sequences_lm(tokenizer, prompts):
    without, with_c = tokenizer(prompts, prepend=tokenizer.get_bos_token_id())
    assert len(without) < len(with_c) and without == with_c[:len(without)], (
        "prompt without is supposed to be a prefix of prompt with")
    return [with_c], [len(without)], [len(with_c)]


@torch.no_grad()
def forward_model(model, input_ids):
    """(B,T) ids -> ((B,T) next-token losses with NaN in the last column, (B,T) argmax predictions)."""
    B, T = input_ids.shape
    logits = model(input_ids)
    targets = torch.roll(input_ids, shifts=-1, dims=1)
    losses = F.cross_entropy(logits.view(B * T, -1), targets.view(B * T), reduction="none").view(B, T)
    losses[:, -1] = float("nan")
    return losses, logits.argmax(dim=-1)


_RENDER = {
    "multiple_choice": (render_prompts_mc, batch_sequences_mc),
    "schema": (render_prompts_schema, batch_sequences_schema),
    "language_modeling": (render_prompts_lm, batch_sequences_lm),
}


@torch.no_grad()
def evaluate_example(idx, model, tokenizer, data, device, task_meta):
    item = data[idx]
    kind = task_meta["task_type"]
    if kind not in _RENDER:
        raise ValueError(f"Unsupported task type: {kind}")
    shots = []
    if task_meta["num_fewshot"] > 0:
        others = [i for i in range(len(data)) if i != idx]
        shots = [data[i] for i in random.Random(1234 + idx).sample(others, task_meta["num_fewshot"])]
    render, batch = _RENDER[kind]
    tokens, starts, ends = batch(tokenizer, render(item, task_meta["continuation_delimiter"], shots))
    limit = getattr(model, "max_seq_len", None)
    if limit is not None:
        # keep the tail of over-long sequences and shift the scoring span with it
        clipped = []
        for t, s, e in zip(tokens, starts, ends):
            cut = max(0, len(t) - limit)
            assert s - cut >= 0 and e - cut >= 0, "scoring span fell off the truncated sequence"
            clipped.append((t[cut:], s - cut, e - cut))
        tokens, starts, ends = map(list, zip(*clipped))
    input_ids = stack_sequences(tokens, tokenizer.get_bos_token_id()).to(device)
    losses, predictions = forward_model(model, input_ids)
    if kind == "language_modeling":
        s, e = starts[0], ends[0]
        return torch.all(predictions[0, s - 1:e - 1] == input_ids[0, s:e]).item()
    means = [losses[i, s - 1:e - 1].mean().item() for i, (s, e) in enumerate(zip(starts, ends))]
    return means.index(min(means)) == item["gold"]


def evaluate_task(model, tokenizer, data, device, task_meta):
    """Accuracy over `data`; examples are dealt round-robin to ranks and summed back."""
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    correct = torch.zeros(len(data), dtype=torch.float32, device=device)
    for idx in range(rank, len(data), world):
        correct[idx] = float(evaluate_example(idx, model, tokenizer, data, device, task_meta))
    if world > 1:
        dist.barrier()
        dist.all_reduce(correct, op=dist.ReduceOp.SUM)
    return correct.mean().item()
