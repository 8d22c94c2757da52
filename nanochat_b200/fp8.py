"""
FP8 linear layers for training.

Public surface of the reference module (nanochat/fp8.py:195-266): `Float8Linear`,
`Float8LinearConfig.from_recipe_name`, `convert_to_float8_training(module, config=, module_filter_fn=)`.
The swapped-in module shares the original weight; evaluation code can switch all FP8 layers back to
bf16 for the duration of a `with fp8_disabled(model):` block (what the reference does by swapping
modules around its evaluations, scripts/base_train.py:195-240).

Recipes
  tensorwise  one dynamic scale per tensor: e4m3 inputs and weights in the forward GEMM, e5m2 output
              gradients in the two backward GEMMs (the reference's only recipe). Runs on
              `torch._scaled_mm`; kept as the numerical comparison point.
  mxfp8       block scaling: every 32 consecutive elements along the reduction dim share one
              power-of-two (E8M0) scale, so quantisation needs no global amax pass. On a B200 with
              the native kernels the three matmuls of a layer run on the hardware block-scaled GEMM
              (`tcgen05.mma.kind::mxf8f6f4.block_scale`, `ops/csrc/gemm.cu: gemm_mx_kernel`) on
              operands quantised by `ops/csrc/quant.cu: mx_quantize_bf16_kernel`; elsewhere, or when a
              reduction dim is not a multiple of 128, the same numerics are emulated
              (quantise-dequantise to bf16 + bf16 GEMM).
`rowwise` is accepted by the command line of the reference but rejected here exactly as there.
"""

from contextlib import contextmanager

import torch
import torch.nn as nn

from nanochat_b200 import common

EPS = 1e-12


@torch.no_grad()
def _tensorwise_quant(x, dtype):
    """(fp8 tensor, inverse scale) with scale = fp8_max / amax computed in float64."""
    fmax = torch.finfo(dtype).max
    amax = x.float().abs().max()
    scale = (fmax / amax.double().clamp(min=EPS)).float()
    q = (x.float() * scale).clamp(-fmax, fmax).to(dtype)
    return q, scale.reciprocal()


def _col_major(t):
    return t.t().contiguous().t()


class _TensorwiseMatmul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, w):
        xq, xs = _tensorwise_quant(x2, torch.float8_e4m3fn)
        wq, ws = _tensorwise_quant(w, torch.float8_e4m3fn)
        ctx.save_for_backward(xq, xs, wq, ws)
        return torch._scaled_mm(xq, wq.t(), scale_a=xs, scale_b=ws, out_dtype=x2.dtype, use_fast_accum=True)

    @staticmethod
    def backward(ctx, dy):
        xq, xs, wq, ws = ctx.saved_tensors
        gq, gs = _tensorwise_quant(dy, torch.float8_e5m2)
        dx = torch._scaled_mm(gq, _col_major(wq), scale_a=gs, scale_b=ws, out_dtype=dy.dtype, use_fast_accum=False)
        dw = torch._scaled_mm(gq.t().contiguous(), _col_major(xq), scale_a=gs, scale_b=xs, out_dtype=dy.dtype,
                              use_fast_accum=False)
        return dx, dw


@torch.no_grad()
def mx_quant_dequant(x, dtype=torch.float8_e4m3fn, block=32):
    """Round-trip through MXFP8: per 32-element block along the last dim, scale = 2^(floor(log2 amax) - emax)."""
    shape = x.shape
    xb = x.float().reshape(-1, block)
    amax = xb.abs().amax(dim=1, keepdim=True).clamp_min(2.0 ** -127)
    emax = 8 if dtype == torch.float8_e4m3fn else 15          # exponent of the largest power of two in range
    scale = torch.exp2(torch.floor(torch.log2(amax)) - emax)
    fmax = torch.finfo(dtype).max
    q = (xb / scale).clamp(-fmax, fmax).to(dtype).float() * scale
    return q.reshape(shape).to(x.dtype)


class _MxEmulatedMatmul(torch.autograd.Function):
    """MXFP8 numerics with bf16 GEMMs: operands are block-quantised along each GEMM's reduction dim."""

    @staticmethod
    def forward(ctx, x2, w):
        ctx.save_for_backward(x2, w)
        return mx_quant_dequant(x2) @ mx_quant_dequant(w.to(x2.dtype)).t()

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        wb = w.to(dy.dtype)
        dx = mx_quant_dequant(dy, torch.float8_e5m2) @ mx_quant_dequant(wb.t().contiguous()).t()
        dw = mx_quant_dequant(dy.t().contiguous(), torch.float8_e5m2) @ mx_quant_dequant(x2.t().contiguous()).t()
        return dx, dw.to(w.dtype)


class _MxHardwareMatmul(torch.autograd.Function):
    """MXFP8 on the tensor cores: each of the three products quantises its two operands along ITS reduction dim
    (activations / weights e4m3, output gradients e5m2) and runs the block-scaled GEMM."""

    @staticmethod
    def forward(ctx, x2, w):
        from nanochat_b200 import ops
        nat = ops.native_module()
        ctx.save_for_backward(x2, w)
        return nat.mx_linear(x2, w)                                              # (M, K) x (N, K)^T, reduce over K

    @staticmethod
    def backward(ctx, dy):
        from nanochat_b200 import ops
        nat = ops.native_module()
        x2, w = ctx.saved_tensors
        E5M2 = torch.float8_e5m2
        dy = dy.to(torch.bfloat16)
        wt = w.to(torch.bfloat16).t().contiguous()                               # (K, N): reduce over N
        dx = nat.mx_linear(dy, wt, x_dtype=E5M2)
        dyt, xt = dy.t().contiguous(), x2.to(torch.bfloat16).t().contiguous()    # (N, M), (K, M): reduce over M
        dw = nat.mx_linear(dyt, xt, x_dtype=E5M2, out_dtype=torch.float32)
        return dx.to(x2.dtype), dw.to(w.dtype)


def _mx_hardware_ok(x2, w):
    """The block-scaled GEMM needs every reduction dim (K, N and M of the three products) to be a multiple of 128."""
    return (_native_active() and x2.is_cuda and x2.dtype == torch.bfloat16
            and x2.shape[0] % 128 == 0 and x2.shape[1] % 128 == 0 and w.shape[0] % 128 == 0)


class Float8Linear(nn.Linear):
    """nn.Linear whose matmuls run in FP8; weights (and bias) keep their storage precision."""

    recipe = "tensorwise"
    fp8_enabled = True

    def forward(self, input):
        x = input.to(common.COMPUTE_DTYPE)
        if not self.fp8_enabled:
            from nanochat_b200 import ops
            return ops.linear(x, self.weight)
        x2 = x.reshape(-1, x.shape[-1])
        if self.recipe == "mxfp8":
            y = (_MxHardwareMatmul if _mx_hardware_ok(x2, self.weight) else _MxEmulatedMatmul).apply(x2, self.weight)
        else:
            y = _TensorwiseMatmul.apply(x2, self.weight)
        y = y.reshape(*x.shape[:-1], y.shape[-1])
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y

    @classmethod
    def from_float(cls, mod, recipe="tensorwise"):
        with torch.device("meta"):
            new = cls(mod.in_features, mod.out_features, bias=False)
        new.weight = mod.weight
        new.bias = mod.bias
        new.recipe = recipe
        return new


class Float8LinearConfig:
    def __init__(self, recipe="tensorwise"):
        self.recipe = recipe

    @staticmethod
    def from_recipe_name(recipe_name):
        if recipe_name not in ("tensorwise", "mxfp8"):
            raise ValueError(f"Only 'tensorwise' and 'mxfp8' recipes are supported, got '{recipe_name}'.")
        return Float8LinearConfig(recipe_name)


def default_fp8_filter(mod, fqn):
    """Both dims divisible by 16 and at least 128 (reference: scripts/base_train.py:178-185)."""
    if not isinstance(mod, nn.Linear):
        return False
    if mod.in_features % 16 != 0 or mod.out_features % 16 != 0:
        return False
    return min(mod.in_features, mod.out_features) >= 128


def convert_to_float8_training(module, *, config=None, module_filter_fn=None):
    """Swap matching nn.Linear children (post-order) for Float8Linear sharing the same parameters."""
    recipe = config.recipe if config is not None else "tensorwise"

    def walk(mod, prefix=""):
        for name, child in mod.named_children():
            fqn = f"{prefix}.{name}" if prefix else name
            walk(child, fqn)
            if isinstance(child, nn.Linear) and not isinstance(child, Float8Linear):
                if module_filter_fn is None or module_filter_fn(child, fqn):
                    setattr(mod, name, Float8Linear.from_float(child, recipe))
    walk(module)
    if recipe == "tensorwise":
        _set_native_fp8(True)
    else:
        # the fused per-layer path runs the tensorwise recipe only; block-scaled layers go through the modules
        module._fp8_module_path = True
    return module


def _set_native_fp8(enabled):
    """The fused sm_100a layer path does not go through the nn.Linear modules: it has its own switch."""
    from nanochat_b200 import ops
    if _native_active():
        ops.native_module().set_fp8(enabled)


def _native_active():
    from nanochat_b200 import ops
    return ops.get_kernel_mode() == "native" and torch.cuda.is_available()


@contextmanager
def fp8_disabled(model):
    """Run every Float8Linear of `model` as a bf16 linear inside the block."""
    mods = [m for m in model.modules() if isinstance(m, Float8Linear)]
    for m in mods:
        m.fp8_enabled = False
    from nanochat_b200 import ops
    native_was_on = _native_active() and ops.native_module().fp8_enabled()
    if native_was_on:
        _set_native_fp8(False)
    try:
        yield
    finally:
        for m in mods:
            m.fp8_enabled = True
        if native_was_on:
            _set_native_fp8(True)
