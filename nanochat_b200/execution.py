"""
Run model-written Python in a throw-away interpreter.

Each call starts a fresh `python -I` child in a temporary working directory with an
empty environment and no stdin. Address-space / data / stack rlimits (256 MB by
default) are installed in the child between fork and exec, so they hold even if the
program tampers with Python-level guards; a prelude then removes the destructive
entry points (os.system, os.kill, os.fork, shutil.rmtree, subprocess.Popen, ...) and
the program runs with fresh globals. The parent enforces the wall-clock timeout by
killing the child.

This protects an evaluation loop from accidents (fork bombs, deleted files, runaway
memory). It is not a security boundary: sockets are not blocked, ctypes can undo the
prelude, and there is no kernel-level isolation. (Reference behaviour:
nanochat/execution.py:32-134.)
"""

import json
import subprocess
import sys
import tempfile
from dataclasses import dataclass
from typing import Optional


@dataclass
class ExecutionResult:
    success: bool
    stdout: str
    stderr: str
    error: Optional[str] = None
    timeout: bool = False
    memory_exceeded: bool = False


_OS_BLOCKED = ("kill", "system", "putenv", "remove", "removedirs", "rmdir", "fchdir", "setuid", "fork",
               "forkpty", "killpg", "rename", "renames", "truncate", "replace", "unlink", "fchmod",
               "fchown", "chmod", "chown", "chroot", "lchflags", "lchmod", "lchown", "getcwd", "chdir")
_SHUTIL_BLOCKED = ("rmtree", "move", "chown")
_MODULES_BLOCKED = ("ipdb", "joblib", "resource", "psutil", "tkinter")

# Runs inside the child. Everything it defines is deleted before the user program starts, and the
# program gets its own globals dict.
_PRELUDE = """
def _lockdown(cfg):
    import builtins, faulthandler, os, shutil, subprocess, sys
    faulthandler.disable()
    for name in ("exit", "quit", "help"):
        setattr(builtins, name, None)
    os.environ["OMP_NUM_THREADS"] = "1"
    for name in cfg["os"]:
        setattr(os, name, None)
    for name in cfg["shutil"]:
        setattr(shutil, name, None)
    subprocess.Popen = None
    for name in cfg["modules"]:
        sys.modules[name] = None
_lockdown(%s)
del _lockdown
exec(compile(%s, "<llm>", "exec"), {"__name__": "__main__"})
"""

GUARD = _PRELUDE        # name used by code written against the reference: the source run in the child before the program


def _limit_memory(nbytes):
    """Returns a callable that runs in the child after fork and before exec."""
    def apply():
        import resource
        for kind in (resource.RLIMIT_AS, resource.RLIMIT_DATA, resource.RLIMIT_STACK):
            resource.setrlimit(kind, (nbytes, nbytes))
    return apply


def execute_code(code: str, timeout: float = 5.0,
                 maximum_memory_bytes: Optional[int] = 256 * 1024 * 1024) -> ExecutionResult:
    """Execute `code`; never raises for failures of the program itself."""
    cfg = json.dumps({"os": _OS_BLOCKED, "shutil": _SHUTIL_BLOCKED, "modules": _MODULES_BLOCKED})
    program = _PRELUDE % (f"__import__('json').loads({cfg!r})", repr(code))
    preexec = None
    if maximum_memory_bytes is not None and sys.platform != "darwin":
        preexec = _limit_memory(maximum_memory_bytes)
    with tempfile.TemporaryDirectory() as workdir:
        try:
            proc = subprocess.run([sys.executable, "-I", "-c", program], cwd=workdir, env={"PATH": "/usr/bin:/bin"},
                                  stdin=subprocess.DEVNULL, capture_output=True, text=True, timeout=timeout,
                                  preexec_fn=preexec)
        except subprocess.TimeoutExpired:
            return ExecutionResult(False, "", "", error="Execution timed out (process killed)", timeout=True)
    ok = proc.returncode == 0
    err_lines = proc.stderr.strip().splitlines()
    error = None if ok else (err_lines[-1] if err_lines else "Execution failed")
    return ExecutionResult(ok, proc.stdout, proc.stderr, error=error,
                           memory_exceeded=("MemoryError" in proc.stderr))
