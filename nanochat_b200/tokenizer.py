"""
GPT-4-style byte-level BPE tokenizer with chat rendering.

Training and encoding run in this framework's own C++ extension
(`csrc/tokenizer/`: Unicode-aware split scanner, multi-threaded word counting,
incremental pair merging, thread-pool batch encoding). A pure-Python body with
the same results backs it where the extension is not built. The reference gets
the same two jobs from two external Rust libraries (rustbpe to train, tiktoken to
encode; reference: nanochat/tokenizer.py:34-138).

File compatibility: `tokenizer.pkl` holds a pickled `tiktoken.Encoding` in the
reference. We read that pickle (taking `pat_str`, `mergeable_ranks`,
`special_tokens` from its state) and write the same kind of pickle when tiktoken
is importable, so tokenizers trained by either code base load in the other.

Chat format (reference: tokenizer.py:140-259):
  <|bos|> <|user_start|>...<|user_end|> <|assistant_start|>...<|assistant_end|> ...
with mask 1 on assistant text, python tool calls (delimiters included) and
<|assistant_end|>; python outputs are mask 0.
"""

import os
import copy
import pickle
from functools import lru_cache

SPECIAL_TOKENS = [
    "<|bos|>",              # document delimiter, first token of every document
    "<|user_start|>", "<|user_end|>",
    "<|assistant_start|>", "<|assistant_end|>",
    "<|python_start|>", "<|python_end|>",     # assistant calls the python tool
    "<|output_start|>", "<|output_end|>",     # tool output fed back to the assistant
]

# GPT-4 split pattern with \p{N}{1,2} (numbers split in groups of at most two digits)
SPLIT_PATTERN = r"""'(?i:[sdmt]|ll|ve|re)|[^\r\n\p{L}\p{N}]?+\p{L}+|\p{N}{1,2}| ?[^\s\p{L}\p{N}]++[\r\n]*|\s*[\r\n]|\s+(?!\S)|\s+"""


# ----------------------------------------------------------------------------
# back ends

def _load_cpp():
    try:
        from nanochat_b200.utils.build import load_tokenizer_extension
        return load_tokenizer_extension()
    except Exception:
        return None


class _PyBPE:
    """Reference-quality (slow) BPE in Python: used when the C++ extension is unavailable."""

    def __init__(self, pattern, mergeable_ranks):
        import regex
        self._re = regex.compile(pattern)
        self.ranks = mergeable_ranks
        self.vocab = {v: k for k, v in mergeable_ranks.items()}

    def _bpe(self, piece: bytes):
        if piece in self.ranks:
            return [self.ranks[piece]]
        parts = [bytes([b]) for b in piece]
        while len(parts) > 1:
            best_rank, best_i = None, -1
            for i in range(len(parts) - 1):
                r = self.ranks.get(parts[i] + parts[i + 1])
                if r is not None and (best_rank is None or r < best_rank):
                    best_rank, best_i = r, i
            if best_rank is None:
                break
            parts[best_i:best_i + 2] = [parts[best_i] + parts[best_i + 1]]
        return [self.ranks[p] for p in parts]

    def encode_ordinary(self, text):
        out = []
        for m in self._re.findall(text):
            out.extend(self._bpe(m.encode("utf-8")))
        return out

    def encode_ordinary_batch(self, texts, num_threads=8):
        return [self.encode_ordinary(t) for t in texts]

    @staticmethod
    def train(text_iterator, vocab_size, pattern):
        """Classic BPE: count pre-split words, repeatedly merge the most frequent adjacent pair.
        Ties break toward the lexicographically smaller pair of ids (deterministic)."""
        import regex
        from collections import Counter
        splitter = regex.compile(pattern)
        words = Counter()
        for text in text_iterator:
            for piece in splitter.findall(text):
                words[piece.encode("utf-8")] += 1
        seqs = [list(w) for w in words]
        counts = [words[w] for w in words]
        token_bytes = [bytes([i]) for i in range(256)]
        merges = []
        while len(token_bytes) < vocab_size:
            pair_counts = Counter()
            for s, c in zip(seqs, counts):
                for a, b in zip(s, s[1:]):
                    pair_counts[(a, b)] += c
            if not pair_counts:
                break
            best = min(pair_counts.items(), key=lambda kv: (-kv[1], kv[0]))[0]
            if pair_counts[best] <= 0:
                break
            new_id = len(token_bytes)
            token_bytes.append(token_bytes[best[0]] + token_bytes[best[1]])
            merges.append(best)
            for s in seqs:
                i = 0
                while i < len(s) - 1:
                    if s[i] == best[0] and s[i + 1] == best[1]:
                        s[i:i + 2] = [new_id]
                    i += 1
        return {tb: i for i, tb in enumerate(token_bytes)}


class _Encoding:
    """Rank table + split pattern + specials; the object `tokenizer.pkl` describes."""

    def __init__(self, name, pat_str, mergeable_ranks, special_tokens):
        self.name = name
        self.pat_str = pat_str
        self.mergeable_ranks = mergeable_ranks
        self.special_tokens = dict(special_tokens)
        self.n_vocab = max(max(mergeable_ranks.values()), max(self.special_tokens.values(), default=0)) + 1
        self._id_to_bytes = {v: k for k, v in mergeable_ranks.items()}
        for s, i in self.special_tokens.items():
            self._id_to_bytes[i] = s.encode("utf-8")
        cpp = _load_cpp()
        if cpp is not None and pat_str == SPLIT_PATTERN:
            ordered = sorted(mergeable_ranks.items(), key=lambda kv: kv[1])
            self._impl = cpp.Encoder([k for k, _ in ordered], [v for _, v in ordered])
        else:
            self._impl = _PyBPE(pat_str, mergeable_ranks)

    @property
    def special_tokens_set(self):
        return set(self.special_tokens)

    def encode_ordinary(self, text):
        return list(self._impl.encode_ordinary(text))

    def encode_ordinary_batch(self, texts, num_threads=8):
        return [list(x) for x in self._impl.encode_ordinary_batch(texts, num_threads)]

    def encode_single_token(self, text):
        if text in self.special_tokens:
            return self.special_tokens[text]
        return self.mergeable_ranks[text.encode("utf-8")]

    def decode_bytes(self, ids):
        return b"".join(self._id_to_bytes[i] for i in ids)

    def decode(self, ids):
        return self.decode_bytes(ids).decode("utf-8", errors="replace")

    def decode_single_token_bytes(self, token_id):
        return self._id_to_bytes[token_id]


def _encoding_from_pickle(path):
    """Read a reference-style tokenizer.pkl (pickled tiktoken.Encoding) or our own dict form."""
    class _State:
        def __setstate__(self, state):
            self.state = state

    class _Unpickler(pickle.Unpickler):
        def find_class(self, module, name):
            if module.startswith("tiktoken") and name == "Encoding":
                return _State
            return super().find_class(module, name)

    with open(path, "rb") as f:
        obj = _Unpickler(f).load()
    state = obj.state if isinstance(obj, _State) else obj
    if not isinstance(state, dict):
        raise ValueError(f"unrecognised tokenizer pickle: {path}")
    return _Encoding(state.get("name", "nanochat"), state["pat_str"], state["mergeable_ranks"],
                     state["special_tokens"])


# ----------------------------------------------------------------------------

class BPETokenizer:
    """Tokenizer with the reference's public surface (`RustBPETokenizer`, tokenizer.py:34-259)."""

    def __init__(self, enc, bos_token):
        self.enc = enc
        self.bos_token_id = self.encode_special(bos_token)

    @classmethod
    def train_from_iterator(cls, text_iterator, vocab_size):
        n_ordinary = vocab_size - len(SPECIAL_TOKENS)
        assert n_ordinary >= 256, f"vocab_size_no_special must be at least 256, got {n_ordinary}"
        cpp = _load_cpp()
        if cpp is not None:
            pairs = cpp.train_bpe(text_iterator, n_ordinary)
            ranks = {bytes(b): r for b, r in pairs}
        else:
            ranks = _PyBPE.train(text_iterator, n_ordinary, SPLIT_PATTERN)
        offset = len(ranks)
        specials = {name: offset + i for i, name in enumerate(SPECIAL_TOKENS)}
        return cls(_Encoding("nanochat_bpe", SPLIT_PATTERN, ranks, specials), "<|bos|>")

    @classmethod
    def from_directory(cls, tokenizer_dir):
        return cls(_encoding_from_pickle(os.path.join(tokenizer_dir, "tokenizer.pkl")), "<|bos|>")

    @classmethod
    def from_pretrained(cls, tiktoken_name):
        """GPT-2 / cl100k encodings for `tok_eval` comparisons; their <|endoftext|> plays BOS."""
        import tiktoken
        t = tiktoken.get_encoding(tiktoken_name)
        enc = _Encoding(t.name, t._pat_str, t._mergeable_ranks, t._special_tokens)
        return cls(enc, "<|endoftext|>")

    def get_vocab_size(self):
        return self.enc.n_vocab

    def get_special_tokens(self):
        return self.enc.special_tokens_set

    def id_to_token(self, id):
        return self.enc.decode([id])

    @lru_cache(maxsize=32)
    def encode_special(self, text):
        return self.enc.encode_single_token(text)

    def get_bos_token_id(self):
        return self.bos_token_id

    def encode(self, text, prepend=None, append=None, num_threads=8):
        """Ordinary text only: special-token strings inside `text` are NOT recognised."""
        pre = None if prepend is None else (prepend if isinstance(prepend, int) else self.encode_special(prepend))
        post = None if append is None else (append if isinstance(append, int) else self.encode_special(append))
        if isinstance(text, str):
            rows = [self.enc.encode_ordinary(text)]
        elif isinstance(text, list):
            rows = self.enc.encode_ordinary_batch(text, num_threads=num_threads)
        else:
            raise ValueError(f"Invalid input type: {type(text)}")
        if pre is not None:
            rows = [[pre] + r for r in rows]
        if post is not None:
            for r in rows:
                r.append(post)
        return rows[0] if isinstance(text, str) else rows

    def __call__(self, *args, **kwargs):
        return self.encode(*args, **kwargs)

    def decode(self, ids):
        return self.enc.decode(ids)

    def decode_single_token_bytes(self, token_id):
        return self.enc.decode_single_token_bytes(token_id)

    def save(self, tokenizer_dir):
        os.makedirs(tokenizer_dir, exist_ok=True)
        path = os.path.join(tokenizer_dir, "tokenizer.pkl")
        state = dict(name=self.enc.name, pat_str=self.enc.pat_str,
                     mergeable_ranks=self.enc.mergeable_ranks, special_tokens=self.enc.special_tokens)
        try:
            import tiktoken
            payload = tiktoken.Encoding(**state)   # same pickle the reference writes and reads
        except Exception:
            payload = state
        with open(path, "wb") as f:
            pickle.dump(payload, f)
        print(f"Saved tokenizer encoding to {path}")

    # ------------------------------------------------------------ chat
    def render_conversation(self, conversation, max_tokens=2048):
        """Conversation dict -> (ids, mask); mask 1 marks tokens the assistant is trained on."""
        messages = conversation["messages"]
        if messages[0]["role"] == "system":
            # fold the system prompt into the first user turn
            assert messages[1]["role"] == "user", "System message must be followed by a user message"
            merged = dict(messages[1])
            merged["content"] = messages[0]["content"] + "\n\n" + messages[1]["content"]
            messages = [merged] + list(messages[2:])
        assert len(messages) >= 1, f"Conversation has less than 1 message: {messages}"
        sp = self.encode_special
        ids, mask = [], []

        def emit(tokens, m):
            if isinstance(tokens, int):
                tokens = [tokens]
            ids.extend(tokens)
            mask.extend([m] * len(tokens))

        emit(self.get_bos_token_id(), 0)
        for i, message in enumerate(messages):
            expected = "user" if i % 2 == 0 else "assistant"
            assert message["role"] == expected, f"Message {i} is from {message['role']} but should be from {expected}"
            content = message["content"]
            if expected == "user":
                assert isinstance(content, str), "User messages are simply expected to be strings"
                emit(sp("<|user_start|>"), 0)
                emit(self.encode(content), 0)
                emit(sp("<|user_end|>"), 0)
                continue
            emit(sp("<|assistant_start|>"), 0)
            if isinstance(content, str):
                emit(self.encode(content), 1)
            elif isinstance(content, list):
                for part in content:
                    body = self.encode(part["text"])
                    kind = part["type"]
                    if kind == "text":
                        emit(body, 1)
                    elif kind == "python":
                        emit(sp("<|python_start|>"), 1)
                        emit(body, 1)
                        emit(sp("<|python_end|>"), 1)
                    elif kind == "python_output":
                        # produced by the tool at test time, never supervised
                        emit(sp("<|output_start|>"), 0)
                        emit(body, 0)
                        emit(sp("<|output_end|>"), 0)
                    else:
                        raise ValueError(f"Unknown part type: {kind}")
            else:
                raise ValueError(f"Unknown content type: {type(content)}")
            emit(sp("<|assistant_end|>"), 1)
        return ids[:max_tokens], mask[:max_tokens]

    def visualize_tokenization(self, ids, mask, with_token_id=False):
        """Debug helper: supervised tokens green, the rest red."""
        out = []
        for t, m in zip(ids, mask):
            colour = "\033[92m" if m == 1 else "\033[91m"
            out.append(f"{colour}{self.decode([t])}\033[0m")
            if with_token_id:
                out.append(f"\033[90m({t})\033[0m")
        return "|".join(out)

    def render_for_completion(self, conversation):
        """Prompt for sampling: the conversation minus its last assistant turn, plus <|assistant_start|>."""
        conversation = copy.deepcopy(conversation)
        messages = conversation["messages"]
        assert messages[-1]["role"] == "assistant", "Last message must be from the Assistant"
        messages.pop()
        ids, _ = self.render_conversation(conversation)
        ids.append(self.encode_special("<|assistant_start|>"))
        return ids


RustBPETokenizer = BPETokenizer  # name used by code written against the reference


def get_tokenizer():
    from nanochat_b200.common import get_base_dir
    return BPETokenizer.from_directory(os.path.join(get_base_dir(), "tokenizer"))


def get_token_bytes(device="cpu"):
    import torch
    from nanochat_b200.common import get_base_dir
    path = os.path.join(get_base_dir(), "tokenizer", "token_bytes.pt")
    assert os.path.exists(path), f"Token bytes not found at {path}? It gets written by tok_train.py"
    with open(path, "rb") as f:
        return torch.load(f, map_location=device)
