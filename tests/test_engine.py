"""Engine contract: cache bookkeeping, sampling semantics, determinism (no model weights needed)."""
from dataclasses import dataclass

import torch

from nanochat_b200.engine import KVCache, Engine, use_calculator


@dataclass
class TinyConfig:
    n_kv_head: int = 4
    n_head: int = 4
    n_embd: int = 64
    n_layer: int = 2
    sequence_len: int = 128


class FlatModel:
    """Uniform logits over the vocabulary; advances the cache like a real forward would."""

    def __init__(self, vocab_size=262):
        self.vocab_size = vocab_size
        self.config = TinyConfig()

    def get_device(self):
        return torch.device("cpu")

    def forward(self, ids, kv_cache=None):
        B, T = ids.shape
        if kv_cache is not None:
            kv_cache.advance(T)
        return torch.zeros(B, T, self.vocab_size)


class ScriptedModel(FlatModel):
    """Emits a fixed token script regardless of input (for the tool-use state machine)."""

    def __init__(self, script, vocab_size=262):
        super().__init__(vocab_size)
        self.script = list(script)
        self.calls = 0

    def forward(self, ids, kv_cache=None):
        B, T = ids.shape
        if kv_cache is not None:
            kv_cache.advance(T)
        logits = torch.full((B, T, self.vocab_size), -50.0)
        tok = self.script[min(self.calls, len(self.script) - 1)]
        logits[:, -1, tok] = 50.0
        self.calls += 1
        return logits


class ByteTok:
    SPECIAL = {"<|python_start|>": 256, "<|python_end|>": 257, "<|output_start|>": 258,
               "<|output_end|>": 259, "<|assistant_end|>": 260, "<|bos|>": 261}

    def encode_special(self, s):
        return self.SPECIAL[s]

    def get_bos_token_id(self):
        return 261

    def encode(self, s, prepend=None):
        ids = list(s.encode("utf-8"))
        return ([prepend] + ids) if prepend is not None else ids

    def decode(self, ids):
        return bytes(t for t in ids if t < 256).decode("utf-8", errors="replace")


PROMPT = [261, 72, 101, 108, 108, 111]


def _cache(**kw):
    args = dict(batch_size=2, num_heads=3, seq_len=64, head_dim=5, num_layers=6, device="cpu", dtype=torch.float32)
    args.update(kw)
    return KVCache(**args)


def test_kv_cache_geometry_and_position():
    c = _cache()
    assert c.get_pos() == 0
    assert c.k_cache.shape == (6, 2, 64, 3, 5) and c.v_cache.shape == (6, 2, 64, 3, 5)
    c.advance(10)
    c.advance(5)
    assert c.get_pos() == 15 and c.cache_seqlens.tolist() == [15, 15]
    c.reset()
    assert c.get_pos() == 0 and c.cache_seqlens.tolist() == [0, 0]
    k0, v0 = c.get_layer_cache(0)
    assert k0.shape == (2, 64, 3, 5) and v0.shape == (2, 64, 3, 5)


def test_kv_cache_prefill_fork():
    src = _cache(batch_size=1, num_heads=4, head_dim=8, num_layers=2, seq_len=32)
    src.k_cache[0, 0, :16] = 1.0
    src.v_cache[0, 0, :16] = 2.0
    src.prev_embedding = torch.ones(1, 1, 7)
    src.advance(16)
    dst = _cache(batch_size=3, num_heads=4, head_dim=8, num_layers=2, seq_len=64)
    dst.prefill(src)
    assert dst.get_pos() == 16
    assert (dst.k_cache[0, :, :16] == 1.0).all() and (dst.v_cache[0, :, :16] == 2.0).all()
    assert dst.prev_embedding.shape == (3, 1, 7)


def test_first_tokens_sampled_independently_per_row():
    eng = Engine(FlatModel(), ByteTok())
    first = None
    for column, masks in eng.generate(PROMPT, num_samples=16, max_tokens=1, temperature=1.0, seed=42):
        first = column
    assert len(set(first)) > 1, "rows share one sampled token: prefill logits were broadcast, not re-sampled"


def test_seed_reproducibility_and_variation():
    eng = Engine(FlatModel(), ByteTok())
    for seed in (1, 42, 123, 999):
        runs = [eng.generate_batch(PROMPT, max_tokens=5, seed=seed)[0] for _ in range(3)]
        assert runs[0] == runs[1] == runs[2]
    outs = {tuple(eng.generate_batch(PROMPT, temperature=1.0, max_tokens=5, seed=s)[0][0]) for s in range(1, 11)}
    assert len(outs) > 1


def test_temperature_zero_ignores_seed():
    eng = Engine(FlatModel(), ByteTok())
    runs = [eng.generate_batch(PROMPT, temperature=0.0, max_tokens=5, seed=s)[0] for s in (1, 42, 123)]
    assert runs[0] == runs[1] == runs[2]


def test_max_tokens_and_num_samples():
    eng = Engine(FlatModel(), ByteTok())
    for n in (1, 4, 16, 64):
        seqs, masks = eng.generate_batch(PROMPT, max_tokens=n)
        assert len(seqs[0]) - len(PROMPT) <= n
        assert len(masks[0]) == len(seqs[0]) and masks[0][:len(PROMPT)] == [0] * len(PROMPT)
    for n in (1, 4, 16, 64):
        seqs, _ = eng.generate_batch(PROMPT, num_samples=n, max_tokens=3)
        assert len(seqs) == n


def test_tool_use_forces_calculator_output():
    tok = ByteTok()
    expr = list(b"12*3")
    script = [256] + expr + [257] + [65] * 10          # <python_start> 12*3 <python_end> then 'A's
    eng = Engine(ScriptedModel(script), tok)
    seqs, masks = eng.generate_batch(PROMPT, temperature=0.0, max_tokens=12)
    gen, m = seqs[0][len(PROMPT):], masks[0][len(PROMPT):]
    assert gen[:6] == [256] + expr + [257]
    assert gen[6:10] == [258] + list(b"36") + [259], gen
    assert m[6:10] == [0, 0, 0, 0] and all(x == 1 for x in m[:6])


def test_calculator_rules():
    assert use_calculator("1,000 + 2") == 1002
    assert use_calculator("2**10") is None
    assert use_calculator("'strawberry'.count('r')") == 3
    assert use_calculator("__import__('os')") is None
    assert use_calculator("'a'.upper()") is None


def test_engine_matches_naive_generation_at_temperature_zero():
    """KV-cached decoding must reproduce full-recompute decoding token for token."""
    from nanochat_b200.models.gpt import GPT, GPTConfig
    cfg = GPTConfig(sequence_len=64, vocab_size=300, n_layer=4, n_head=2, n_kv_head=1, n_embd=256,
                    window_pattern="SL")
    torch.manual_seed(3)
    model = GPT(cfg)
    model.init_weights()
    with torch.no_grad():
        for blk in model.transformer.h:
            blk.attn.c_proj.weight.normal_(0, 0.05)
            blk.mlp.c_proj.weight.normal_(0, 0.05)
        model.lm_head.weight.normal_(0, 0.2)
        model.smear_lambda.fill_(0.5)
    model.eval()
    prompt = [261, 5, 9, 200, 41, 7]
    naive = list(model.generate(prompt, max_tokens=24, temperature=0.0))
    fast = [c[0] for c, _ in Engine(model, ByteTok()).generate(prompt, num_samples=1, max_tokens=24, temperature=0.0)]
    stop = next((i for i, t in enumerate(fast) if t in (260, 261)), len(fast) - 1)
    assert naive[:stop + 1] == fast[:stop + 1]


def test_paged_cache_fork_shares_full_prompt_pages_and_copies_the_partial_one():
    """Page-table bookkeeping on CPU tensors: after a prefill through the contiguous prompt view and a fork, every row
    reads back the prompt in position order, full prompt pages are shared, each row has its own page for the tail."""
    import torch
    from nanochat_b200.engine import PagedKVCache
    L, H, D, P = 2, 2, 8, 16
    cache = PagedKVCache(batch_size=3, num_heads=H, seq_len=96, head_dim=D, num_layers=L, device="cpu",
                         dtype=torch.float32, page_tokens=P)
    prompt, new = 37, 20                                  # 2 full pages + 5 tokens
    cache.reserve(prompt, new)
    assert cache.shared_pages == 3 and cache.private_pages == 2
    view = cache.begin_prompt(prompt)
    assert view.max_seq_len == 48 and view.batch_size == 1
    want = []
    for layer in range(L):
        k, v = view.get_layer_cache(layer)
        kk, vv = torch.randn(1, prompt, H, D), torch.randn(1, prompt, H, D)
        k[:, :prompt] = kk
        v[:, :prompt] = vv
        want.append((kk[0], vv[0]))
    view.advance(prompt)
    cache.fork(view)
    assert cache.get_pos() == prompt and cache.cache_seqlens.tolist() == [prompt] * 3
    table = cache.table
    assert all(table[r, :2].tolist() == [0, 1] for r in range(3))
    tails = table[:, 2].tolist()
    assert len(set(tails)) == 3 and min(tails) >= cache.shared_pages
    assert (table[:, 4:] == cache.spare_page).all()       # nothing mapped past the reserved pages
    for layer in range(L):
        for row in range(3):
            k, v = cache.gather_row(layer, row)
            assert torch.equal(k, want[layer][0]) and torch.equal(v, want[layer][1])
    # a row appending into its tail page does not touch the other rows or the shared pages
    cache.k_pool[0, tails[1], prompt % P] = 7.0
    k0, _ = cache.gather_row(0, 0)
    assert torch.equal(k0, want[0][0])
    # a larger request grows the pool and moves its version (a captured decode graph is rebuilt then)
    version = cache.pool_version
    cache.reserve(prompt, 50)
    assert cache.pool_version == version + 1 and cache.private_pages == 4
    cache.reserve(20, 10)
    assert cache.pool_version == version + 1              # smaller requests reuse the pool
