"""
In-tree build of the native extensions with explicit compiler commands.

  nanochat_b200/_C*.so    CUDA kernels (nvcc, sm_100a only) + torch bindings
  nanochat_b200/_tok*.so  C++ tokenizer (BPE trainer / encoder) + best-fit packer

The shared objects are written next to the package so they are found wherever the
source tree is copied; a content hash of the sources is stored beside each one and a
rebuild happens only when the hash differs (or the .so is missing). Build from the
command line with `python -m nanochat_b200.utils.build`.
"""

import os
import sys
import glob
import fcntl
import hashlib
import contextlib
import importlib.util
import subprocess
import sysconfig
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(PKG_DIR, "ops", "csrc")
TOK_SRC = os.path.join(PKG_DIR, "csrc", "tokenizer")
BUILD_DIR = os.path.join(PKG_DIR, "_build")
EXT_SUFFIX = sysconfig.get_config_var("EXT_SUFFIX") or ".so"

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _hash_files(paths, extra=""):
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build command failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    return r.stdout + r.stderr


def _nvcc():
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    path = os.path.join(cuda_home, "bin", "nvcc")
    return path if os.path.exists(path) else "nvcc"


def _stale(so_path, digest):
    stamp = so_path + ".hash"
    if not os.path.exists(so_path) or not os.path.exists(stamp):
        return True
    with open(stamp) as f:
        return f.read().strip() != digest


@contextlib.contextmanager
def _build_lock():
    """Exclusive lock over check + compile + link + stamp. Every rank of a multi-process job imports the package; on
    a fresh checkout (or after a source edit) all of them find the build stale, and without the lock they would
    compile into the same object files and load a library another rank is still writing. The first rank through
    builds, the others wait here and then find the stamp current."""
    os.makedirs(BUILD_DIR, exist_ok=True)
    with open(os.path.join(BUILD_DIR, ".lock"), "w") as f:
        fcntl.flock(f, fcntl.LOCK_EX)
        try:
            yield
        finally:
            fcntl.flock(f, fcntl.LOCK_UN)


def _write_stamp(so_path, digest):
    tmp = so_path + ".hash.tmp"
    with open(tmp, "w") as f:
        f.write(digest)
    os.replace(tmp, so_path + ".hash")


# Optimizer and collective kernels keep IEEE division / square root and denormals: their state (second moments,
# running norms) lives for the whole run, and approximate math there shows up as drift, not as noise.
PRECISE_SOURCES = ("optim.cu", "comm.cu")


def _load(name, so_path):
    spec = importlib.util.spec_from_file_location(name, so_path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[name] = mod
    return mod


# ------------------------------------------------------------------------------- CUDA

def cuda_sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu"))), sorted(glob.glob(os.path.join(CSRC, "*.cpp")))


def build_cuda_extension(verbose=False, force=False):
    """Compile every .cu for sm_100a and link `_C`. Returns the path of the shared object."""
    import torch
    name = "_C"
    so_path = os.path.join(PKG_DIR, name + EXT_SUFFIX)
    cus, cpps = cuda_sources()
    headers = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh"))
    extra_flags = os.environ.get("NANOCHAT_NVCC_FLAGS", "").split()     # e.g. -DNC_ATTN_TRACE for kernel timelines
    digest = _hash_files(cus + cpps + headers, extra=torch.__version__ + " ".join(extra_flags) + " precise:" + ",".join(PRECISE_SOURCES))
    if not force and not _stale(so_path, digest):
        return so_path
    with _build_lock():
        if not force and not _stale(so_path, digest):      # another process built it while this one waited
            return so_path
        return _build_cuda_locked(name, so_path, cus, cpps, extra_flags, digest, verbose)


def _build_cuda_locked(name, so_path, cus, cpps, extra_flags, digest, verbose):
    import torch
    from torch.utils import cpp_extension as ce
    incs = []
    for p in ce.include_paths("cuda"):
        incs += ["-I", p]
    incs += ["-I", sysconfig.get_paths()["include"], "-I", CSRC]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    common_defs = [f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H",
                   f"-D_GLIBCXX_USE_CXX11_ABI={abi}"]
    nvcc = _nvcc()
    jobs = []
    for src in cus:
        obj = os.path.join(BUILD_DIR, os.path.basename(src) + ".o")
        fast = [] if os.path.basename(src) in PRECISE_SOURCES else ["--use_fast_math"]
        cmd = [nvcc, *NVCC_ARCH, "-lineinfo", "-O3", "-std=c++17", *fast, "-Xcompiler", "-fPIC",
               "-Xptxas", "-v" if verbose else "-O3", *extra_flags, "-I", CSRC, "-c", src, "-o", obj]
        jobs.append((cmd, obj))
    for src in cpps:
        obj = os.path.join(BUILD_DIR, os.path.basename(src) + ".o")
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", *common_defs, *incs, "-c", src, "-o", obj]
        jobs.append((cmd, obj))
    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
        logs = list(pool.map(lambda j: _run(j[0]), jobs))
    if verbose:
        for (cmd, _), log in zip(jobs, logs):
            print(" ".join(cmd))
            print(log)
    libs = []
    for p in ce.library_paths("cuda"):
        libs += ["-L", p, f"-Wl,-rpath,{p}"]
    tmp_so = so_path + ".tmp"           # link under another name: a process that already mapped the old file keeps it
    link = ["g++", "-shared", "-o", tmp_so, *[j[1] for j in jobs], *libs,
            "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    _run(link)
    os.replace(tmp_so, so_path)
    _write_stamp(so_path, digest)
    return so_path


_cuda_ext = None


def load_cuda_extension():
    """Import `_C`, building it first if it is missing or out of date."""
    global _cuda_ext
    if _cuda_ext is None:
        import torch  # noqa: F401  (libtorch must be loaded before the extension)
        _cuda_ext = _load("nanochat_b200._C", build_cuda_extension())
    return _cuda_ext


# -------------------------------------------------------------------------- tokenizer

def build_tokenizer_extension(force=False, sanitize=False):
    """Build `_tok`. `sanitize=True` builds a second copy under `_build/sanitize/` with AddressSanitizer and
    UndefinedBehaviorSanitizer (run it in a process started with libasan preloaded; see tests/test_tok_sanitize.py)."""
    import pybind11
    name = "_tok"
    so_path = os.path.join(PKG_DIR, name + EXT_SUFFIX)
    opt = ["-O3"]
    if sanitize:
        os.makedirs(os.path.join(BUILD_DIR, "sanitize"), exist_ok=True)
        so_path = os.path.join(BUILD_DIR, "sanitize", name + EXT_SUFFIX)
        opt = ["-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"]
    srcs = sorted(glob.glob(os.path.join(TOK_SRC, "*.cpp")))
    if not srcs:
        raise FileNotFoundError("tokenizer sources not found")
    headers = glob.glob(os.path.join(TOK_SRC, "*.h")) + glob.glob(os.path.join(TOK_SRC, "*.inc"))
    digest = _hash_files(srcs + headers)
    if not force and not _stale(so_path, digest):
        return so_path
    with _build_lock():
        if not force and not _stale(so_path, digest):
            return so_path
        tmp_so = so_path + ".tmp"
        cmd = ["g++", *opt, "-std=c++17", "-fPIC", "-shared", "-pthread", "-I", pybind11.get_include(),
               "-I", sysconfig.get_paths()["include"], "-I", TOK_SRC, *srcs, "-o", tmp_so]
        _run(cmd)
        os.replace(tmp_so, so_path)
        _write_stamp(so_path, digest)
    return so_path


_tok_ext = None


def load_tokenizer_extension():
    global _tok_ext
    if _tok_ext is None:
        sanitize = os.environ.get("NANOCHAT_TOK_SANITIZE", "0") == "1"      # ASan/UBSan copy, for the sanitizer test
        _tok_ext = _load("nanochat_b200._tok", build_tokenizer_extension(sanitize=sanitize))
    return _tok_ext


def sanitizer_runtime_libs():
    """Paths of the ASan and UBSan runtimes of the host compiler (for LD_PRELOAD), or None if either is missing."""
    out = []
    for lib in ("libasan.so", "libubsan.so"):
        r = subprocess.run(["gcc", f"-print-file-name={lib}"], capture_output=True, text=True)
        path = r.stdout.strip()
        if r.returncode != 0 or not os.path.isabs(path) or not os.path.exists(path):
            return None
        out.append(os.path.realpath(path))
    return out


def build_all(verbose=False, force=False):
    out = [build_cuda_extension(verbose=verbose, force=force)]
    try:
        out.append(build_tokenizer_extension(force=force))
    except FileNotFoundError:
        pass
    return out


if __name__ == "__main__":
    for path in build_all(verbose="-v" in sys.argv, force="-f" in sys.argv):
        print("built", path)
