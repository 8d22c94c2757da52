"""
Hardware block-scaled fp8 (MXFP8): the quantisation kernel against the plain-PyTorch definition of the format, the
tcgen05 block-scaled GEMM against the fp32 product of the de-quantised operands (ragged shapes, both tile widths,
both element formats), and the mxfp8 `Float8Linear` on the hardware path against its bf16 emulation.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

BF16 = torch.bfloat16
E4M3, E5M2 = torch.float8_e4m3fn, torch.float8_e5m2


@pytest.fixture(scope="module")
def nat():
    from nanochat_b200.ops import native
    return native


def _unblock(sf, rows, k):
    """(rows, k/32) exponent bytes from the tensor core's blocked layout: chunk [row block][k block] of 512 bytes,
    byte (r % 32) * 16 + ((r % 128) / 32) * 4 + (k / 32) % 4."""
    r = torch.arange(rows, device=sf.device)[:, None]
    kb = torch.arange(k // 32, device=sf.device)[None, :]
    idx = ((r // 128) * (k // 128) + kb // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4
    return sf[idx.reshape(-1)].view(rows, k // 32)


def _dequant(q, sf, rows, k):
    scale = torch.exp2(_unblock(sf, rows, k).float() - 127.0)
    return (q.float().view(rows, k // 32, 32) * scale[:, :, None]).view(rows, k)


def _mk(shape, seed, spread=True):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(shape, device="cuda", generator=g)
    if spread:       # blocks of very different magnitude: what block scaling is for
        x = x * torch.exp2(torch.randint(-12, 6, (shape[0], 1), device="cuda", generator=g).float())
    return x.to(BF16)


@pytest.mark.parametrize("dtype", [E4M3, E5M2])
@pytest.mark.parametrize("rows,k", [(128, 128), (200, 384), (513, 1664)])
def test_mx_quantize_is_the_formats_definition(nat, rows, k, dtype):
    from nanochat_b200.fp8 import mx_quant_dequant
    x = _mk((rows, k), seed=rows + k)
    x[3, 32:64] = 0                                           # an all-zero block
    q, sf = nat.mx_quantize(x, dtype)
    got = _dequant(q, sf, rows, k)
    want = mx_quant_dequant(x.float(), dtype)
    assert torch.equal(got, want.float())
    assert q.dtype == dtype and sf.numel() == -(-rows // 128) * (k // 128) * 512


@pytest.mark.parametrize("M,N,K,bn,a_dtype", [
    (256, 256, 256, 0, E4M3), (256, 256, 256, 128, E4M3), (384, 1664, 1664, 256, E4M3), (200, 136, 128, 0, E5M2),
    (1024, 4992, 1664, 0, E5M2), (128, 1664, 6656, 128, E4M3), (640, 384, 512, 256, E5M2),
])
def test_block_scaled_gemm_matches_fp32_product_of_dequantised_operands(nat, M, N, K, bn, a_dtype):
    a, b = _mk((M, K), seed=M + N), _mk((N, K), seed=M + K + 1)
    aq, asf = nat.mx_quantize(a, a_dtype)
    bq, bsf = nat.mx_quantize(b, E4M3)
    ref = _dequant(aq, asf, M, K) @ _dequant(bq, bsf, N, K).t()
    out = torch.empty(M, N, dtype=torch.float32, device="cuda")
    nat.gemm_mx(aq, asf, bq, bsf, out, bn=bn)
    nat.check_status(out)
    err = ((out - ref).norm() / ref.norm()).item()
    assert err < 1e-5, err                                    # same products, fp32 accumulation in another order
    # bf16 output with a residual add in the epilogue, and bitwise repeatability
    res = _mk((M, N), seed=7, spread=False)
    y1 = torch.empty(M, N, dtype=BF16, device="cuda")
    y2 = torch.empty_like(y1)
    nat.gemm_mx(aq, asf, bq, bsf, y1, aux=res, beta=1.0, bn=bn)
    nat.gemm_mx(aq, asf, bq, bsf, y2, aux=res, beta=1.0, bn=bn)
    assert torch.equal(y1, y2)
    want = ref + res.float()
    assert ((y1.float() - want).norm() / want.norm()).item() < 1e-2


def test_mxfp8_linear_runs_on_the_block_scaled_gemm_and_matches_its_emulation(nat):
    from nanochat_b200 import fp8
    torch.manual_seed(0)
    lin = torch.nn.Linear(512, 384, bias=False).cuda()
    mx = fp8.Float8Linear.from_float(lin, recipe="mxfp8")
    x = _mk((256, 512), seed=3, spread=False).requires_grad_(True)
    g = _mk((256, 384), seed=4, spread=False)
    calls = []
    orig = nat.gemm_mx
    nat.gemm_mx = lambda *a, **k: (calls.append(1), orig(*a, **k))[1]
    try:
        y = mx(x)
        y.backward(g)
    finally:
        nat.gemm_mx = orig
    assert len(calls) == 3, "forward, dgrad and wgrad must each run the hardware GEMM"
    dx, dw = x.grad.clone(), lin.weight.grad.clone()
    x.grad = None
    lin.weight.grad = None
    y_ref = fp8._MxEmulatedMatmul.apply(x, lin.weight)
    y_ref.backward(g)
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm()).item()
    assert rel(y, y_ref) < 1e-2 and rel(dx, x.grad) < 1e-2 and rel(dw, lin.weight.grad) < 1e-2
    nat.check_status(x)
