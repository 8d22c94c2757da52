"""
The C++ tokenizer / packer under AddressSanitizer and UndefinedBehaviorSanitizer.

A second copy of the extension is built with `-fsanitize=address,undefined` and driven, in a child process that
has the sanitizer runtimes preloaded, through every entry point on awkward inputs: empty strings, lone
continuation bytes, very long runs, many threads, documents longer than a row. Any report aborts the child.
"""
import os
import subprocess
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_WORKER = r'''
import importlib.util, os, random, sys
spec = importlib.util.spec_from_file_location("nc_build", os.path.join(sys.argv[1], "nanochat_b200", "utils", "build.py"))
build = importlib.util.module_from_spec(spec); spec.loader.exec_module(build)
tok = build.load_tokenizer_extension()
assert os.sep + "sanitize" + os.sep in tok.__file__, tok.__file__

rng = random.Random(0)
alphabet = ["a", "b", "Z", " ", "  ", "\n", "\r\n", "\t", "'s", "'LL", "1", "23", "4567", "!", "?!", "é", "中", "\U0001f600",
            "́", " ", "_", "-", "x" * 40]
def text(n):
    return "".join(rng.choice(alphabet) for _ in range(n))

# scanner: pieces concatenate back to the input, whatever the input
cases = ["", " ", "\n", "a", "'", "''s", " " * 1000, "9" * 1001, "中" * 300, "a\x00b", "\r\n\r\n  x"] + [text(rng.randint(1, 400)) for _ in range(300)]
for s in cases:
    pieces = tok.split(s)
    joined = b"".join(p if isinstance(p, bytes) else p.encode("utf-8", "surrogatepass") for p in pieces)
    assert joined == s.encode("utf-8"), (s, pieces)

# trainer: several thread counts, empty texts inside the stream, tiny and larger vocabularies
corpus = [text(rng.randint(0, 300)) for _ in range(600)] + ["", "", "a"]
for vocab, threads in ((256, 1), (300, 3), (700, 8)):
    pairs = tok.train_bpe(iter(corpus), vocab, threads)
    assert len(pairs) <= vocab and len(pairs) >= 256
ranks = {bytes(b): r for b, r in pairs}
ordered = sorted(ranks.items(), key=lambda kv: kv[1])
enc = tok.Encoder([k for k, _ in ordered], [v for _, v in ordered])
inv = {v: k for k, v in ranks.items()}
for s in cases[:200]:
    ids = enc.encode_ordinary(s)
    assert b"".join(inv[i] for i in ids) == s.encode("utf-8")
batch = [text(rng.randint(0, 2000)) for _ in range(257)] + [""]
for threads in (1, 4, 16):
    out = enc.encode_ordinary_batch(batch, threads)
    assert len(out) == len(batch)
    assert all(b"".join(inv[i] for i in ids) == s.encode("utf-8") for ids, s in zip(out, batch))

# packer: documents shorter than, equal to and far longer than a row; refill from a callback
cap, buf = 33, 12
packer = tok.BestFitPacker(cap, buf)
def docs(n):
    return [[rng.randrange(1000) for _ in range(rng.choice([1, 2, 5, 32, 33, 34, 200]))] for _ in range(n)]
refill = lambda: packer.add_documents(docs(5))
for _ in range(40):
    rows = packer.pack(7, refill)
    assert rows.shape == (7, cap)
assert len(packer) >= 0 and isinstance(packer.needs_documents(), bool)
print("sanitized ok")
'''


def test_tokenizer_extension_is_clean_under_asan_and_ubsan(tmp_path):
    sys.path.insert(0, REPO)
    from nanochat_b200.utils import build
    libs = build.sanitizer_runtime_libs()
    if libs is None:
        pytest.skip("the host compiler has no ASan/UBSan runtime")
    build.build_tokenizer_extension(sanitize=True)
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    env = dict(os.environ, NANOCHAT_TOK_SANITIZE="1", LD_PRELOAD=":".join(libs),
               ASAN_OPTIONS="detect_leaks=0:abort_on_error=1:halt_on_error=1",     # the interpreter itself "leaks" at exit
               UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1")
    r = subprocess.run([sys.executable, str(script), REPO], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "sanitized ok" in r.stdout, (r.stdout[-2000:], r.stderr[-6000:])
    assert "AddressSanitizer" not in r.stderr and "runtime error" not in r.stderr, r.stderr[-6000:]
