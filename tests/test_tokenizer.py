"""Tokenizer contract: hermetic in-process training, round trips, special tokens, chat rendering."""
import pytest

from nanochat_b200.tokenizer import BPETokenizer, SPECIAL_TOKENS, SPLIT_PATTERN

CORPUS = [
    "Hello world! The quick brown fox jumps over the lazy dog. 12345 67890.",
    "def f(x):\n    return x + 1\n\nclass A:\n    pass\n",
    "Héllo wörld — ünïcode ☃ 日本語のテキスト 🙂 it's we've they'll I'd",
    "Numbers 3.14159, 2024-01-01, and   spaces\t\ttabs\r\nnewlines\n\n\n",
] * 20


@pytest.fixture(scope="module")
def tok():
    return BPETokenizer.train_from_iterator(iter(CORPUS), vocab_size=300)


def test_vocab_and_specials(tok):
    assert tok.get_vocab_size() == 300
    assert tok.get_special_tokens() == set(SPECIAL_TOKENS)
    ids = [tok.encode_special(s) for s in SPECIAL_TOKENS]
    assert len(set(ids)) == len(SPECIAL_TOKENS) and min(ids) == 300 - len(SPECIAL_TOKENS)
    assert tok.get_bos_token_id() == tok.encode_special("<|bos|>")


@pytest.mark.parametrize("text", ["hello world", "", "   ", "Ünïcödé 日本語 🙂", "a\nb\r\nc", "it's 12345 x=3.14",
                                  "trailing space ", "\n\n\nlead"])
def test_round_trip(tok, text):
    assert tok.decode(tok.encode(text)) == text


def test_special_strings_are_ordinary_text(tok):
    ids = tok.encode("<|bos|> and <|assistant_end|>")
    assert all(i < 300 - len(SPECIAL_TOKENS) for i in ids)
    assert tok.decode(ids) == "<|bos|> and <|assistant_end|>"


def test_prepend_append_and_batch(tok):
    bos = tok.get_bos_token_id()
    base = tok.encode("hello")
    assert tok.encode("hello", prepend="<|bos|>") == [bos] + base
    assert tok.encode("hello", prepend=bos, append="<|assistant_end|>") == [bos] + base + [tok.encode_special("<|assistant_end|>")]
    batch = tok.encode(["hello", "world wide"], prepend=bos, num_threads=2)
    assert batch == [[bos] + tok.encode("hello"), [bos] + tok.encode("world wide")]
    assert tok("hello") == base
    with pytest.raises(ValueError):
        tok.encode(123)


def test_decode_single_token_bytes_and_id_to_token(tok):
    assert tok.decode_single_token_bytes(65) == b"A"
    assert tok.id_to_token(tok.encode_special("<|bos|>")) == "<|bos|>"


def test_conversation_masks(tok):
    conv = {"messages": [{"role": "user", "content": "Hi"}, {"role": "assistant", "content": "Yo"}]}
    ids, mask = tok.render_conversation(conv)
    sp = tok.encode_special
    assert ids[0] == tok.get_bos_token_id() and ids[1] == sp("<|user_start|>")
    assert len(ids) == len(mask)
    a0 = ids.index(sp("<|assistant_start|>"))
    assert all(m == 0 for m in mask[:a0 + 1])
    assert all(m == 1 for m in mask[a0 + 1:]) and ids[-1] == sp("<|assistant_end|>")


def test_system_message_is_merged_and_original_untouched(tok):
    conv = {"messages": [{"role": "system", "content": "Be nice."}, {"role": "user", "content": "Hi"},
                         {"role": "assistant", "content": "Yo"}]}
    ids, _ = tok.render_conversation(conv)
    assert tok.decode(ids).count("Be nice.\n\nHi") == 1
    assert conv["messages"][1]["content"] == "Hi"


def test_tool_parts_supervision(tok):
    parts = [{"type": "text", "text": "calc "}, {"type": "python", "text": "1+1"},
             {"type": "python_output", "text": "2"}, {"type": "text", "text": " done"}]
    conv = {"messages": [{"role": "user", "content": "q"}, {"role": "assistant", "content": parts}]}
    ids, mask = tok.render_conversation(conv)
    sp = tok.encode_special
    ps, pe, os_, oe = (ids.index(sp(s)) for s in ("<|python_start|>", "<|python_end|>", "<|output_start|>", "<|output_end|>"))
    assert all(mask[i] == 1 for i in range(ps, pe + 1))
    assert all(mask[i] == 0 for i in range(os_, oe + 1))
    assert mask[-1] == 1


def test_truncation_and_bad_roles(tok):
    conv = {"messages": [{"role": "user", "content": "word " * 500}, {"role": "assistant", "content": "x"}]}
    ids, mask = tok.render_conversation(conv, max_tokens=32)
    assert len(ids) == 32 and len(mask) == 32
    with pytest.raises(AssertionError):
        tok.render_conversation({"messages": [{"role": "assistant", "content": "x"}]})


def test_render_for_completion(tok):
    conv = {"messages": [{"role": "user", "content": "Hi"}, {"role": "assistant", "content": "Yo"}]}
    ids = tok.render_for_completion(conv)
    assert ids[-1] == tok.encode_special("<|assistant_start|>")
    assert tok.encode_special("<|assistant_end|>") not in ids
    assert len(conv["messages"]) == 2


def test_save_load_round_trip_and_tiktoken_parity(tok, tmp_path):
    tok.save(str(tmp_path))
    again = BPETokenizer.from_directory(str(tmp_path))
    text = "The same ids after a reload: naïve café 42!"
    assert again.encode(text) == tok.encode(text)
    assert again.get_vocab_size() == tok.get_vocab_size()
    tiktoken = pytest.importorskip("tiktoken")
    enc = tiktoken.Encoding(name="t", pat_str=SPLIT_PATTERN, mergeable_ranks=tok.enc.mergeable_ranks,
                            special_tokens=tok.enc.special_tokens)
    for t in CORPUS[:4] + [text, "  multiple   spaces  \n\n and\ttabs "]:
        assert enc.encode_ordinary(t) == tok.encode(t)


# ------------------------------------------------------------- the C++ pieces against independent oracles

def _random_text(rng, n):
    alphabet = ["a", "b", "Z", "é", "ß", "中", "文", "\U0001f600", " ", "  ", "\n", "\r\n", "\t", "'s", "'T", "'ll", "'x", "1",
                "23", "4567", "!", "?!", "...", "_", "-", "́", " ", " ", "x" * 9, "I'm", "don't", "WE'VE"]
    return "".join(rng.choice(alphabet) for _ in range(n))


def test_cpp_scanner_splits_like_the_regex_engine():
    import random
    import regex
    from nanochat_b200.tokenizer import SPLIT_PATTERN, _load_cpp
    cpp = _load_cpp()
    if cpp is None:
        pytest.skip("C++ tokenizer extension not available")
    splitter = regex.compile(SPLIT_PATTERN)
    rng = random.Random(0)
    cases = ["", " ", "\n\n", "a  b", "it's  12345 abc", "  leading", "trailing  ", "x\n \ny", "１２３４"]     # incl. full-width digits
    cases += [_random_text(rng, rng.randint(1, 60)) for _ in range(3000)]
    for text in cases:
        got = [p if isinstance(p, bytes) else p.encode("utf-8") for p in cpp.split(text)]
        want = [m.encode("utf-8") for m in splitter.findall(text)]
        assert got == want, (text, got, want)


@pytest.mark.parametrize("threads", [1, 4])
def test_cpp_trainer_learns_the_same_merges_as_the_python_oracle(threads):
    import random
    from nanochat_b200.tokenizer import SPLIT_PATTERN, _PyBPE, _load_cpp
    cpp = _load_cpp()
    if cpp is None:
        pytest.skip("C++ tokenizer extension not available")
    rng = random.Random(1)
    words = ["the", "quick", "brown", "fox", "jumps", "over", "lazy", "dog", "naïve", "中文", "don't", "1234", "x_y", "..."]
    corpus = [" ".join(rng.choice(words) for _ in range(rng.randint(5, 60))) + rng.choice(["", "\n", "!"]) for _ in range(300)]
    corpus += ["", " "]
    vocab = 256 + 120
    want = _PyBPE.train(iter(corpus), vocab, SPLIT_PATTERN)
    got = {bytes(b): r for b, r in cpp.train_bpe(iter(corpus), vocab, threads)}
    assert got == want
