"""Sandbox properties, each attacked once."""
import os
import time

import pytest

from nanochat_b200.execution import execute_code


def test_stdout_and_exception_capture():
    r = execute_code("print('hello world')")
    assert r.success and r.stdout == "hello world\n"
    r = execute_code("1/0")
    assert not r.success and "ZeroDivisionError" in r.error


def test_timeout_kills_promptly():
    t0 = time.time()
    r = execute_code("while True: pass", timeout=2.0)
    assert r.timeout and not r.success and time.time() - t0 < 5


def test_memory_limit():
    r = execute_code("x = bytearray(1024 * 1024 * 1024)")
    assert not r.success and r.memory_exceeded


@pytest.mark.parametrize("evil", [
    "import os; os.system('echo pwned')", "import shutil; shutil.rmtree('/tmp')",
    "import subprocess; subprocess.Popen(['ls'])", "import os; os.kill(1, 9)", "import os; os.fork()",
])
def test_destructive_calls_fail(evil):
    assert not execute_code(evil).success


def test_no_stdin_tempdir_cwd_clean_env_fresh_globals():
    assert not execute_code("input()").success
    r = execute_code("open('landmine.txt', 'w').write('x'); print(open('landmine.txt').read())")
    assert r.success and r.stdout == "x\n" and not os.path.exists("landmine.txt")
    os.environ["FAKE_SECRET_KEY"] = "hunter2"
    try:
        r = execute_code("import os; print('FAKE_SECRET_KEY' in os.environ)")
        assert r.success and r.stdout.strip() == "False"
    finally:
        del os.environ["FAKE_SECRET_KEY"]
    r = execute_code("print('_lockdown' in dir(), '_PRELUDE' in dir())")
    assert r.success and r.stdout.strip() == "False False"


def test_quotes_backslashes_braces_survive_embedding():
    tricky = '''s = 'it\\'s "quoted" \\\\ {braces} %s \\n'; print(len(s))'''
    assert execute_code(tricky).success
