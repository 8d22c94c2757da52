"""
Core runtime shared by every layer of the framework: compute dtype selection,
logging, base directory, rank-0 printing, distributed bring-up and the peak
FLOP/bandwidth tables used for MFU/MBU reporting.

Parity notes (reference: nanochat/common.py):
  * COMPUTE_DTYPE selection follows `_detect_compute_dtype` (common.py:17-32):
    NANOCHAT_DTYPE env override, bf16 on SM>=80, fp32 otherwise.
  * `compute_init` (common.py:174-209) seeds with 42 and enables tf32. Unlike the
    reference, a process group is ALSO created for CPU runs (gloo backend) so a
    multi-rank CPU job really synchronises its gradients.
  * Peak tables keep the reference's nominal numbers for B200/H100
    (common.py:236,244,291,297) so `bf16_mfu` stays comparable.
"""

import os
import re
import logging
import datetime
import urllib.request

import torch
import torch.distributed as dist

_DTYPES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}


def _pick_compute_dtype():
    forced = os.environ.get("NANOCHAT_DTYPE")
    if forced is not None:
        return _DTYPES[forced], f"set via NANOCHAT_DTYPE={forced}"
    if torch.cuda.is_available():
        major, minor = torch.cuda.get_device_capability()
        if (major, minor) >= (8, 0):
            return torch.bfloat16, f"auto-detected: CUDA SM {major}{minor} (bf16 supported)"
        return torch.float32, f"auto-detected: CUDA SM {major}{minor} (no bf16 tensor cores, using fp32)"
    return torch.float32, "auto-detected: no CUDA (CPU)"


COMPUTE_DTYPE, COMPUTE_DTYPE_REASON = _pick_compute_dtype()


# ----------------------------------------------------------------------------
# logging

class _ColorFormatter(logging.Formatter):
    _C = {"DEBUG": "\033[36m", "INFO": "\033[32m", "WARNING": "\033[33m",
          "ERROR": "\033[31m", "CRITICAL": "\033[35m"}

    def format(self, record):
        name = record.levelname
        if name in self._C:
            record.levelname = f"{self._C[name]}\033[1m{name}\033[0m"
        out = super().format(record)
        if name == "INFO":
            out = re.sub(r"(\d+\.?\d*\s*(?:GB|MB|%|docs))", "\033[1m\\1\033[0m", out)
        return out


ColoredFormatter = _ColorFormatter     # name used by code written against the reference


_logging_ready = False


def setup_default_logging():
    global _logging_ready
    if _logging_ready:
        return
    handler = logging.StreamHandler()
    handler.setFormatter(_ColorFormatter("%(asctime)s - %(name)s - %(levelname)s - %(message)s"))
    logging.basicConfig(level=logging.INFO, handlers=[handler])
    _logging_ready = True


setup_default_logging()
logger = logging.getLogger(__name__)


# ----------------------------------------------------------------------------
# filesystem helpers

def get_base_dir():
    """Root of all intermediates: $NANOCHAT_BASE_DIR or ~/.cache/nanochat."""
    root = os.environ.get("NANOCHAT_BASE_DIR")
    if not root:
        root = os.path.join(os.path.expanduser("~"), ".cache", "nanochat")
    os.makedirs(root, exist_ok=True)
    return root


def download_file_with_lock(url, filename, postprocess_fn=None):
    """Fetch `url` into the base dir once; concurrent ranks serialise on a file lock."""
    from filelock import FileLock
    path = os.path.join(get_base_dir(), filename)
    if os.path.exists(path):
        return path
    with FileLock(path + ".lock"):
        if os.path.exists(path):  # another rank finished while we waited
            return path
        print(f"Downloading {url}...")
        with urllib.request.urlopen(url) as resp:
            payload = resp.read()
        tmp = path + ".part"
        with open(tmp, "wb") as f:
            f.write(payload)
        os.replace(tmp, path)
        print(f"Downloaded to {path}")
        if postprocess_fn is not None:
            postprocess_fn(path)
    return path


def print0(s="", **kwargs):
    if int(os.environ.get("RANK", 0)) == 0:
        print(s, **kwargs)


def print_banner():
    print0(r"""
  _ __   __ _ _ __   ___   ___| |__   __ _| |_      | |__|___ \ / _ \ / _ \
 | '_ \ / _` | '_ \ / _ \ / __| '_ \ / _` | __|_____| '_ \ __) | | | | | | |
 | | | | (_| | | | | (_) | (__| | | | (_| | ||_____| |_) / __/| |_| | |_| |
 |_| |_|\__,_|_| |_|\___/ \___|_| |_|\__,_|\__|     |_.__/_____|\___/ \___/
""")


# ----------------------------------------------------------------------------
# distributed

def is_ddp_requested() -> bool:
    return all(k in os.environ for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"))


def is_ddp_initialized() -> bool:
    return dist.is_available() and dist.is_initialized()


def get_dist_info():
    """(requested, rank, local_rank, world_size) from the torchrun environment."""
    if is_ddp_requested():
        return True, int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    return False, 0, 0, 1


def autodetect_device_type():
    kind = "cuda" if torch.cuda.is_available() else "cpu"
    print0(f"Autodetected device type: {kind}")
    return kind


def compute_init(device_type="cuda", timeout_s=None):
    """Seeds, matmul precision and (when launched by torchrun) the process group.

    CUDA ranks use NCCL bound to their local device; CPU ranks use gloo so that
    `MuonAdamW.step()` can average gradients between them.
    """
    assert device_type in ("cuda", "cpu", "mps"), f"unknown device type {device_type}"
    if device_type == "cuda":
        assert torch.cuda.is_available(), "device_type=cuda but CUDA is unavailable"
    torch.manual_seed(42)
    if device_type == "cuda":
        torch.cuda.manual_seed(42)
        torch.set_float32_matmul_precision("high")
    requested, rank, local_rank, world = get_dist_info()
    kwargs = {}
    if timeout_s is not None:
        kwargs["timeout"] = datetime.timedelta(seconds=timeout_s)
    if requested and device_type == "cuda":
        device = torch.device("cuda", local_rank)
        torch.cuda.set_device(device)
        if not is_ddp_initialized():
            dist.init_process_group(backend="nccl", device_id=device, **kwargs)
        dist.barrier()
    elif requested and world > 1:
        device = torch.device(device_type)
        if not is_ddp_initialized():
            dist.init_process_group(backend="gloo", **kwargs)
        dist.barrier()
    else:
        device = torch.device(device_type)
    if rank == 0:
        logger.info(f"Distributed world size: {world}")
    return requested, rank, local_rank, world, device


def compute_cleanup():
    if is_ddp_initialized():
        dist.destroy_process_group()


class DummyWandb:
    """Stand-in with wandb's logging surface; used when --run=dummy or on non-master ranks."""

    def log(self, *args, **kwargs):
        pass

    def finish(self):
        pass


# ----------------------------------------------------------------------------
# nominal hardware peaks (dense bf16 FLOP/s, HBM bytes/s)

_PEAK_FLOPS = (
    (("gb200",), 2.5e15), (("grace blackwell",), 2.5e15), (("b200",), 2.25e15), (("b100",), 1.8e15),
    (("h200", "nvl"), 836e12), (("h200", "pcie"), 836e12), (("h200",), 989e12),
    (("h100", "nvl"), 835e12), (("h100", "pcie"), 756e12), (("h100",), 989e12),
    (("h800", "nvl"), 989e12), (("h800",), 756e12),
    (("a100",), 312e12), (("a800",), 312e12), (("a40",), 149.7e12), (("a30",), 165e12),
    (("l40s",), 362e12), (("l40-s",), 362e12), (("l40 s",), 362e12), (("l4",), 121e12),
    (("5090",), 209.5e12), (("4090",), 165.2e12), (("3090",), 71e12),
)

_PEAK_BW = (
    (("gb200",), 8.0e12), (("grace blackwell",), 8.0e12), (("b200",), 8.0e12), (("b100",), 8.0e12),
    (("h200",), 4.8e12), (("h100", "nvl"), 3.9e12), (("h100", "pcie"), 2.0e12), (("h100",), 3.35e12),
    (("h800", "pcie"), 2.0e12), (("h800",), 3.35e12),
    (("a100",), 2.0e12), (("a800",), 2.0e12), (("a40",), 696e9), (("a30",), 933e9),
    (("l40s",), 864e9), (("l40-s",), 864e9), (("l40 s",), 864e9), (("l4",), 300e9),
    (("5090",), 1.79e12), (("4090",), 1.01e12), (("3090",), 936e9),
)


def _lookup(table, device_name, what):
    name = device_name.lower()
    for keys, value in table:
        if all(k in name for k in keys):
            return value
    logger.warning(f"Peak {what} undefined for: {device_name}; utilisation will read 0%")
    return float("inf")


def get_peak_flops(device_name: str) -> float:
    return _lookup(_PEAK_FLOPS, device_name, "flops")


def get_peak_bandwidth(device_name: str) -> float:
    return _lookup(_PEAK_BW, device_name, "bandwidth")
