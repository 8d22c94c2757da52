"""
Inference engine: KV cache, batched sampling and the tool-use state machine.

Behavioural contract (reference: nanochat/engine.py):
  * `KVCache` holds (n_layers, B, T, H, D) key/value tensors plus per-row lengths
    (engine.py:82-137); `prefill(other)` copies a batch-1 prompt cache into every
    row of a wider cache.
  * `Engine.generate` prefills the prompt once at batch 1, forks the cache to
    `num_samples` rows, samples every row's first token independently, then decodes
    in lock-step, yielding `(token_column, token_masks)` per step (mask 1 = sampled,
    0 = forced). Rows finish on <|assistant_end|> or <|bos|> (engine.py:176-275).
  * Between <|python_start|> and <|python_end|> the row's tokens are collected,
    decoded and handed to `use_calculator`; a result is force-fed back as
    <|output_start|> result <|output_end|> (engine.py:252-267).

B200-native differences: the cache position is mirrored on the host so a decode
step never calls `.item()`; on CUDA the per-token forward of a `GPT` is replayed
from a captured CUDA graph whose positions live in device memory (see
`runtime.DecodeGraph`), and weights are consumed from bf16 shadows instead of
being re-cast from fp32 every token. On that path the cache is paged
(`PagedKVCache`): the prompt is prefilled straight into pages that every sample
row's page table points at, so forking N samples copies at most one partial page
per row instead of the whole prompt, and N samples hold the prompt once.
"""

import signal
import warnings
from collections import deque
from contextlib import contextmanager

import torch

from nanochat_b200 import common
from nanochat_b200 import ops


# ----------------------------------------------------------------------------
# calculator tool

@contextmanager
def timeout(duration, formula):
    def on_alarm(signum, frame):
        raise Exception(f"'{formula}': timed out after {duration} seconds")
    signal.signal(signal.SIGALRM, on_alarm)
    signal.alarm(duration)
    try:
        yield
    finally:
        signal.alarm(0)


def eval_with_timeout(formula, max_time=3):
    try:
        with timeout(max_time, formula):
            with warnings.catch_warnings():
                warnings.simplefilter("ignore", SyntaxWarning)
                return eval(formula, {"__builtins__": {}}, {})
    except Exception:
        signal.alarm(0)
        return None


_MATH_CHARS = set("0123456789*+-/.() ")
_TEXT_CHARS = set("abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXYZ0123456789'\"()._ ")
_BANNED = ("__", "import", "exec", "eval", "compile", "open", "file", "input", "raw_input",
           "globals", "locals", "vars", "dir", "getattr", "setattr", "delattr", "hasattr")


def use_calculator(expr):
    """Evaluate a model-written expression: plain arithmetic (no **) or `'..'.count('..')`.

    Anything else returns None (reference: engine.py:46-79).
    """
    expr = expr.replace(",", "")
    if all(ch in _MATH_CHARS for ch in expr):
        if "**" in expr:
            return None
        return eval_with_timeout(expr)
    if not all(ch in _TEXT_CHARS for ch in expr):
        return None
    lowered = expr.lower()
    if any(bad in lowered for bad in _BANNED):
        return None
    if ".count(" not in expr:
        return None
    return eval_with_timeout(expr)


# ----------------------------------------------------------------------------

class KVCache:
    """Per-layer K/V store in (B, T, H, D) layout with in-place append.

    `cache_seqlens` (int32, device) is what kernels read; `_pos` mirrors row 0 on the
    host so the engine never synchronises to learn the position.
    """

    def __init__(self, batch_size, num_heads, seq_len, head_dim, num_layers, device, dtype):
        self.batch_size = batch_size
        self.max_seq_len = seq_len
        self.n_layers = num_layers
        self.n_heads = num_heads
        self.head_dim = head_dim
        shape = (num_layers, batch_size, seq_len, num_heads, head_dim)
        self.k_cache = torch.zeros(shape, device=device, dtype=dtype)
        self.v_cache = torch.zeros(shape, device=device, dtype=dtype)
        self.cache_seqlens = torch.zeros(batch_size, dtype=torch.int32, device=device)
        self.prev_embedding = None
        self._pos = 0

    def reset(self):
        self.cache_seqlens.zero_()
        self.prev_embedding = None
        self._pos = 0

    def get_pos(self):
        return self._pos

    def get_layer_cache(self, layer_idx):
        return self.k_cache[layer_idx], self.v_cache[layer_idx]

    def advance(self, num_tokens):
        self.cache_seqlens += num_tokens
        self._pos += num_tokens

    def prefill(self, other):
        """Fork: copy `other`'s filled prefix (batch 1) into every row of this empty cache."""
        assert self.get_pos() == 0, "Cannot prefill a non-empty KV cache"
        assert (self.n_layers, self.n_heads, self.head_dim) == (other.n_layers, other.n_heads, other.head_dim)
        assert self.max_seq_len >= other.max_seq_len
        n = other.get_pos()
        self.k_cache[:, :, :n] = other.k_cache[:, :, :n]
        self.v_cache[:, :, :n] = other.v_cache[:, :, :n]
        self.cache_seqlens.fill_(n)
        self._pos = n
        if other.prev_embedding is not None:
            self.prev_embedding = other.prev_embedding.expand(self.batch_size, -1, -1).clone()


PAGE_TOKENS = 64


class _PromptView:
    """The shared prompt pages of a PagedKVCache seen as a batch-1 contiguous cache: what the prefill writes into.
    Has the KVCache surface the model's forward uses."""

    def __init__(self, owner, capacity):
        self.owner = owner
        self.batch_size = 1
        self.max_seq_len = capacity
        self.n_layers = owner.n_layers
        self.cache_seqlens = torch.zeros(1, dtype=torch.int32, device=owner.k_pool.device)
        self.prev_embedding = None
        self._pos = 0

    def get_pos(self):
        return self._pos

    def get_layer_cache(self, layer_idx):
        o, n = self.owner, self.max_seq_len // self.owner.page_tokens
        shape = (1, self.max_seq_len, o.n_heads, o.head_dim)
        return o.k_pool[layer_idx, :n].view(shape), o.v_pool[layer_idx, :n].view(shape)

    def advance(self, num_tokens):
        self.cache_seqlens += num_tokens
        self._pos += num_tokens


class PagedKVCache:
    """K/V store of `batch_size` sample rows as pages of PAGE_TOKENS tokens plus a per-row page table
    (reference behaviour: nanochat/engine.py:82-137, a contiguous cache per row and a copy at the fork).

    Pool pages [0, shared_pages) hold the prompt, written once by the batch-1 prefill through `begin_prompt()`;
    `fork()` points every row's table at the prompt's full pages and gives each row private pages for the prompt's
    partial last page (copied: rows append into it) and for what it decodes. The decode kernels address tokens
    through the table (`ops/csrc/decode.cu`: KvPages). The pool grows when a request needs more pages than any before
    it; `pool_version` then moves so that a captured decode graph is rebuilt on the new addresses.
    """

    paged = True

    def __init__(self, batch_size, num_heads, seq_len, head_dim, num_layers, device, dtype, page_tokens=PAGE_TOKENS):
        assert page_tokens & (page_tokens - 1) == 0, "page size must be a power of two"
        self.batch_size = batch_size
        self.max_seq_len = seq_len                  # per-row capacity in tokens (what the page table can address)
        self.n_layers, self.n_heads, self.head_dim = num_layers, num_heads, head_dim
        self.page_tokens = page_tokens
        self.max_pages = -(-seq_len // page_tokens)
        self.device, self.dtype = device, dtype
        self.table = torch.zeros(batch_size, self.max_pages, dtype=torch.int32, device=device)
        self.cache_seqlens = torch.zeros(batch_size, dtype=torch.int32, device=device)
        self.k_pool = self.v_pool = None
        self.shared_pages = self.private_pages = 0
        self.pool_version = 0
        self.prev_embedding = None
        self._pos = 0

    # ----------------------------------------------------------------------------- pool
    def reserve(self, prompt_tokens, new_tokens):
        """Make room for a prompt of `prompt_tokens` and `new_tokens` decoded tokens per row."""
        P = self.page_tokens
        assert prompt_tokens + new_tokens <= self.max_seq_len
        shared = -(-prompt_tokens // P)
        private = -(-(prompt_tokens % P + new_tokens) // P)
        if self.k_pool is not None and shared <= self.shared_pages and private <= self.private_pages:
            return
        self.shared_pages = max(shared, self.shared_pages)
        self.private_pages = max(private, self.private_pages)
        # one spare page at the end: table entries a row has no page for point at it, so a token appended past a row's
        # pages lands there instead of in a page that holds someone's keys
        total = self.shared_pages + self.batch_size * self.private_pages + 1
        self.spare_page = total - 1
        shape = (self.n_layers, total, P, self.n_heads, self.head_dim)
        self.k_pool = self.v_pool = None            # release before allocating the larger pool
        self.k_pool = torch.zeros(shape, device=self.device, dtype=self.dtype)
        self.v_pool = torch.zeros(shape, device=self.device, dtype=self.dtype)
        self.pool_version += 1

    def pool_bytes(self):
        return 0 if self.k_pool is None else 2 * self.k_pool.numel() * self.k_pool.element_size()

    def reset(self):
        self.cache_seqlens.zero_()
        self.prev_embedding = None
        self._pos = 0

    def get_pos(self):
        return self._pos

    def get_layer_cache(self, layer_idx):
        """One layer's pools, (pages, PAGE_TOKENS, H, D): the paged decode kernels take them with `table`."""
        return self.k_pool[layer_idx], self.v_pool[layer_idx]

    def advance(self, num_tokens):
        self.cache_seqlens += num_tokens
        self._pos += num_tokens

    # --------------------------------------------------------------------- prompt, fork
    def begin_prompt(self, prompt_tokens):
        """A batch-1 contiguous view of the shared pages for the prefill of a `prompt_tokens`-token prompt."""
        assert self.k_pool is not None and -(-prompt_tokens // self.page_tokens) <= self.shared_pages
        self.reset()
        return _PromptView(self, -(-prompt_tokens // self.page_tokens) * self.page_tokens)

    def fork(self, view):
        """Every row continues the prompt in `view`: full prompt pages are shared, the partial last one is copied."""
        P, B = self.page_tokens, self.batch_size
        n = view.get_pos()
        full, rem = n // P, n % P
        first_private = self.shared_pages + torch.arange(B, dtype=torch.int32, device=self.device) * self.private_pages
        table = torch.full((B, self.max_pages), self.spare_page, dtype=torch.int32, device=self.device)
        if full:
            table[:, :full] = torch.arange(full, dtype=torch.int32, device=self.device)
        own = min(self.private_pages, self.max_pages - full)
        table[:, full:full + own] = first_private[:, None] + torch.arange(own, dtype=torch.int32, device=self.device)
        self.table.copy_(table)
        if rem:
            idx = first_private.long()
            self.k_pool[:, idx, :rem] = self.k_pool[:, full:full + 1, :rem]
            self.v_pool[:, idx, :rem] = self.v_pool[:, full:full + 1, :rem]
        self.cache_seqlens.fill_(n)
        self._pos = n
        self.prev_embedding = None
        if view.prev_embedding is not None:
            self.prev_embedding = view.prev_embedding.expand(B, -1, -1).clone()

    def row_capacity(self):
        """Tokens a row can hold with the pages it has now."""
        return min(self.max_seq_len, (self._pos // self.page_tokens + self.private_pages) * self.page_tokens)

    def gather_row(self, layer_idx, row):
        """(T, H, D) keys and values of one row in position order (tests and debugging; copies)."""
        n = self._pos
        pages = self.table[row, :-(-n // self.page_tokens)].long()
        k = self.k_pool[layer_idx, pages].reshape(-1, self.n_heads, self.head_dim)[:n]
        v = self.v_pool[layer_idx, pages].reshape(-1, self.n_heads, self.head_dim)[:n]
        return k, v


@torch.inference_mode()
def sample_next_token(logits, rng, temperature=1.0, top_k=None):
    """(B, V) logits -> (B, 1) ids; argmax at temperature 0, else top-k / full multinomial."""
    return ops.sample_next_token(logits, rng, temperature, top_k)


class RowState:
    """Decode-time bookkeeping of one sample row."""

    __slots__ = ("current_tokens", "forced_tokens", "in_python_block", "python_expr_tokens", "completed")

    def __init__(self, current_tokens=None):
        self.current_tokens = current_tokens or []
        self.forced_tokens = deque()
        self.in_python_block = False
        self.python_expr_tokens = []
        self.completed = False


def ids_on_cuda(device):
    return torch.device(device).type == "cuda"


class Engine:
    def __init__(self, model, tokenizer):
        self.model = model
        self.tokenizer = tokenizer
        self._decode_graphs = {}
        self._cache_pool = {}      # rows -> full-length KVCache reused across generations (keeps its decode graph)

    def _decode_step(self, ids, kv_cache):
        """One lock-step decode forward; returns (B, V) logits for the new position."""
        runner = None
        if ids.is_cuda and ops.get_kernel_mode() == "native":
            from nanochat_b200.runtime import decode_graph_for
            runner = decode_graph_for(self, kv_cache)
        if runner is not None:
            return runner.step(ids)
        return self.model.forward(ids, kv_cache=kv_cache)[:, -1, :]

    @torch.inference_mode()
    def generate(self, tokens, num_samples=1, max_tokens=None, temperature=1.0, top_k=None, seed=42):
        assert isinstance(tokens, list) and isinstance(tokens[0], int), "expecting list of ints"
        device = self.model.get_device()
        rng = torch.Generator(device=device)
        rng.manual_seed(seed)

        tok = self.tokenizer
        python_start = tok.encode_special("<|python_start|>")
        python_end = tok.encode_special("<|python_end|>")
        output_start = tok.encode_special("<|output_start|>")
        output_end = tok.encode_special("<|output_end|>")
        assistant_end = tok.encode_special("<|assistant_end|>")
        bos = tok.get_bos_token_id()

        cfg = self.model.config
        geometry = dict(num_heads=cfg.n_kv_head, head_dim=cfg.n_embd // cfg.n_head,
                        num_layers=cfg.n_layer, device=device, dtype=common.COMPUTE_DTYPE)
        ids = torch.tensor([tokens], dtype=torch.long, device=device)
        capacity = (len(tokens) + max_tokens) if max_tokens is not None else cfg.sequence_len
        cache = self._pooled_cache(num_samples, len(tokens), capacity, geometry)
        pooled = cache is not None
        if pooled:
            # 1) batch-1 prefill straight into the pages every row will share  2) fork = page tables + one partial page
            view = cache.begin_prompt(len(tokens))
            logits = self.model.forward(ids, kv_cache=view)
            cache.fork(view)
        else:
            # 1) batch-1 prefill of the prompt  2) fork: copy it into every sample row of a contiguous cache
            prompt_cache = KVCache(batch_size=1, seq_len=len(tokens), **geometry)
            logits = self.model.forward(ids, kv_cache=prompt_cache)
            cache = KVCache(batch_size=num_samples, seq_len=capacity, **geometry)
            cache.prefill(prompt_cache)
            del prompt_cache
        logits = logits[:, -1, :].expand(num_samples, -1)
        try:
            yield from self._decode_loop(tokens, num_samples, max_tokens, temperature, top_k, rng, logits, cache,
                                         (python_start, python_end, output_start, output_end, assistant_end, bos))
        finally:
            if pooled:
                cache.in_use = False

    def _pooled_cache(self, rows, prompt_tokens, capacity, geometry):
        """The paged cache of this row count. It lives as long as the engine, so its captured decode graph is reused;
        its page pool grows to the largest request seen. None when the graph path does not apply or the cache is
        busy (nested generations)."""
        from nanochat_b200.runtime import graph_path_applies
        cfg = self.model.config
        if capacity > cfg.sequence_len or not graph_path_applies(self.model, rows):
            return None
        cache = self._cache_pool.get(rows)
        if cache is None:
            cache = PagedKVCache(batch_size=rows, seq_len=cfg.sequence_len, **geometry)
            cache.pooled = True
            cache.in_use = False
            self._cache_pool[rows] = cache
        if cache.in_use:
            return None
        cache.in_use = True
        cache.reset()
        cache.reserve(prompt_tokens, capacity - prompt_tokens)
        return cache

    def _decode_loop(self, tokens, num_samples, max_tokens, temperature, top_k, rng, logits, cache, specials):
        python_start, python_end, output_start, output_end, assistant_end, bos = specials
        tok = self.tokenizer
        device = self.model.get_device()
        if ids_on_cuda(device) and ops.get_kernel_mode() == "native":
            from nanochat_b200.runtime import decode_graph_for
            runner = decode_graph_for(self, cache)
            if runner is not None:
                runner.begin()
        # 3) lock-step decode with the per-row state machine
        rows = [RowState(tokens.copy()) for _ in range(num_samples)]
        produced = 0
        while True:
            if max_tokens is not None and produced >= max_tokens:
                break
            if all(r.completed for r in rows):
                break
            sampled = sample_next_token(logits, rng, temperature, top_k)[:, 0].tolist()
            column, masks = [], []
            for i, row in enumerate(rows):
                forced = len(row.forced_tokens) > 0
                token = row.forced_tokens.popleft() if forced else sampled[i]
                masks.append(0 if forced else 1)
                column.append(token)
                row.current_tokens.append(token)
                if token == assistant_end or token == bos:
                    row.completed = True
                if token == python_start:
                    row.in_python_block = True
                    row.python_expr_tokens = []
                elif token == python_end and row.in_python_block:
                    row.in_python_block = False
                    if row.python_expr_tokens:
                        result = use_calculator(tok.decode(row.python_expr_tokens))
                        if result is not None:
                            row.forced_tokens.append(output_start)
                            row.forced_tokens.extend(tok.encode(str(result)))
                            row.forced_tokens.append(output_end)
                    row.python_expr_tokens = []
                elif row.in_python_block:
                    row.python_expr_tokens.append(token)
            yield column, masks
            produced += 1
            ids = torch.tensor(column, dtype=torch.long, device=device).unsqueeze(1)
            logits = self._decode_step(ids, cache)

    def generate_batch(self, tokens, num_samples=1, **kwargs):
        """Non-streaming: returns (sequences, masks) without the terminal token; prompt mask is 0."""
        assistant_end = self.tokenizer.encode_special("<|assistant_end|>")
        bos = self.tokenizer.get_bos_token_id()
        results = [tokens.copy() for _ in range(num_samples)]
        masks = [[0] * len(tokens) for _ in range(num_samples)]
        done = [False] * num_samples
        for column, column_masks in self.generate(tokens, num_samples, **kwargs):
            for i, (t, m) in enumerate(zip(column, column_masks)):
                if done[i]:
                    continue
                if t == assistant_end or t == bos:
                    done[i] = True
                else:
                    results[i].append(t)
                    masks[i].append(m)
            if all(done):
                break
        return results, masks


if __name__ == "__main__":
    # Self-check: the naive full-recompute sampler and the Engine must agree at temperature 0.
    import time
    from nanochat_b200.checkpoint_manager import load_model
    device_type = common.autodetect_device_type()
    _, _, _, _, device = common.compute_init(device_type)
    model, tokenizer, meta = load_model("base", device, phase="eval")
    prompt = tokenizer.encode("The chemical formula of water is", prepend=tokenizer.get_bos_token_id())
    t0 = time.time()
    naive = list(model.generate(prompt, max_tokens=64, temperature=0.0))
    t1 = time.time()
    fast = [col[0] for col, _ in Engine(model, tokenizer).generate(prompt, num_samples=1, max_tokens=64, temperature=0.0)]
    t2 = time.time()
    print(tokenizer.decode(naive))
    print(f"naive {t1 - t0:.2f}s | engine {t2 - t1:.2f}s | Match: {naive == fast}")
