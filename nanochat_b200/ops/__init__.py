"""
Fused-op surface used by the model, optimizer and engine.

Every op has two bodies with one meaning:
  * `reference.py` — plain PyTorch, runs anywhere (CPU path, test oracle);
  * `native.py`    — autograd wrappers over the hand-written sm_100a kernels in
                     `csrc/` (tcgen05/TMEM GEMMs, flash attention, fused
                     norm/rope/loss/optimizer kernels).

`use_native(t)` decides per call: CUDA bf16 tensors go to the kernels, everything
else to the reference body. On a CUDA device a missing extension is an error, not
a silent fallback, unless NANOCHAT_KERNELS=torch is set explicitly.
"""

import os

import torch

from . import reference

_MODE = os.environ.get("NANOCHAT_KERNELS", "native")  # native | torch
_native = None
_native_err = None


def set_kernel_mode(mode: str):
    """'native' (default) or 'torch' (reference bodies even on CUDA; used for A/B tests)."""
    global _MODE
    assert mode in ("native", "torch")
    _MODE = mode


def get_kernel_mode() -> str:
    return _MODE


def native_module():
    """Import the native op module (loads the compiled extension) once."""
    global _native, _native_err
    if _native is None and _native_err is None:
        try:
            from . import native as _n
            _native = _n
        except Exception as e:  # keep the reason for the error message
            _native_err = e
    if _native is None:
        raise RuntimeError(
            "nanochat_b200 native kernels are required on CUDA devices but the extension "
            f"could not be loaded: {_native_err!r}. Build it with `python -m nanochat_b200.utils.build` "
            "or set NANOCHAT_KERNELS=torch to run the PyTorch reference path.")
    return _native


def use_native(t: torch.Tensor) -> bool:
    if _MODE != "native" or not t.is_cuda:
        return False
    if t.dtype not in (torch.bfloat16, torch.int64, torch.int32):
        return False
    native_module()
    return True


def _pick(name, probe):
    return getattr(native_module(), name) if use_native(probe) else getattr(reference, name)


def rms_norm(x):
    return _pick("rms_norm", x)(x)


def embed_norm_smear(idx, wte, gate_w, lam, compute_dtype):
    if compute_dtype == torch.bfloat16 and wte.dtype == torch.bfloat16 and use_native(wte):
        return native_module().embed_norm_smear(idx, wte, gate_w, lam)
    return reference.embed_norm_smear(idx, wte, gate_w, lam, compute_dtype)


def resid_mix_norm(x, x0, resid_lambdas, x0_lambdas, layer):
    if use_native(x):
        return native_module().resid_mix_norm(x, x0, resid_lambdas, x0_lambdas, layer)
    return reference.resid_mix_norm(x, x0, resid_lambdas[layer], x0_lambdas[layer])


def linear(x, w):
    return _pick("linear", x)(x, w)


def linear_relu2(x, w):
    return _pick("linear_relu2", x)(x, w)


def ve_gate_add(v, xn, gate_w, ve_w, idx):
    return _pick("ve_gate_add", v)(v, xn, gate_w, ve_w, idx)


def rope_qknorm(q, k, cos, sin):
    return _pick("rope_qknorm", q)(q, k, cos, sin)


def attention(q, k, v, window_left):
    return _pick("attention", q)(q, k, v, window_left)


def add_norm(x, delta):
    return _pick("add_norm", x)(x, delta)


def backout_norm(x, x_backout, lam):
    return _pick("backout_norm", x)(x, x_backout, lam)


def softcap_logits(x, w, vocab_size, softcap=reference.SOFTCAP):
    return _pick("softcap_logits", x)(x, w, vocab_size, softcap)


def softcap_cross_entropy(x, w, targets, vocab_size, reduction="mean", softcap=reference.SOFTCAP):
    return _pick("softcap_cross_entropy", x)(x, w, targets, vocab_size, reduction, softcap)


def sample_next_token(logits, rng, temperature=1.0, top_k=None):
    if (logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 2 and logits.size(1) <= 32768
            and _MODE == "native"):
        return native_module().sample_next_token(logits, rng, temperature, top_k)
    return reference.sample_next_token(logits, rng, temperature, top_k)
