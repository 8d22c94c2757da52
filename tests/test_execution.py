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


# ---- cases of this repository's own (the ones above follow the reference suite's contracts)

@pytest.mark.parametrize("evil", [
    "import subprocess; subprocess.run(['ls'])",                     # run() goes through the removed Popen
    "import subprocess; subprocess.check_output('echo hi', shell=True)",
    "import os; os.rename('a', 'b')",
    "import os; os.chdir('/')",
    "import os, tempfile; f = tempfile.mkstemp()[1]; os.unlink(f)",
    "import shutil; shutil.move('a', 'b')",
    "import resource; resource.setrlimit(resource.RLIMIT_AS, (-1, -1))",   # cannot lift its own memory limit
    "import psutil",
    "exit(0)",                                                        # the builtin is gone: not a clean way out
])
def test_more_ways_to_do_damage_fail(evil):
    assert not execute_code(evil).success


def test_limits_hold_against_tampering_with_the_prelude():
    """The memory limit is an rlimit of the child process, installed before the interpreter starts: restoring the
    Python-level guards (or importing them afresh) does not bring the memory back."""
    r = execute_code("import importlib, os; importlib.reload(os); x = bytearray(2 * 1024 ** 3)")
    assert not r.success and r.memory_exceeded
    r = execute_code("def f(n):\n    return f(n + 1)\nimport sys; sys.setrecursionlimit(10 ** 9); f(0)", timeout=20.0)
    assert not r.success                                   # stack rlimit / recursion error, not a hung or crashed parent


def test_output_flood_and_sleeping_children_end_with_the_timeout():
    t0 = time.time()
    r = execute_code("import time\nwhile True:\n    print('x' * 4096)\n    time.sleep(0.001)", timeout=1.5)
    assert r.timeout and not r.success and time.time() - t0 < 6
    t0 = time.time()
    r = execute_code("import threading, time\nfor _ in range(8):\n    threading.Thread(target=time.sleep, args=(60,)).start()",
                     timeout=1.5)
    # threads either cannot be started under the address-space limit (a thread stack is as large as the stack rlimit) or
    # keep the child alive until the parent kills it: both end the call promptly and unsuccessfully
    assert not r.success and time.time() - t0 < 6


def test_each_call_is_a_fresh_interpreter_in_a_fresh_directory():
    assert execute_code("import builtins; builtins.leak = 41; open('state.txt', 'w').write('1')").success
    r = execute_code("import builtins, os; print(hasattr(builtins, 'leak'), os.path.exists('state.txt'))")
    assert r.success and r.stdout.split() == ["False", "False"]
    r = execute_code("import sys; print(sys.flags.isolated, sys.stdin.read() == '')")
    assert r.success and r.stdout.split() == ["1", "True"]
