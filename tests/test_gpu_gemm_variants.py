"""
GPU numerics of the GEMM variants against plain PyTorch fp32 references:
the CTA-pair (cta_group::2, 256 x BN tiles) kernel in every operand layout, and the 8-bit float
(e4m3 / e5m2, per-tensor scaled) kernels in the three layouts a linear layer needs.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

BF16 = torch.bfloat16


@pytest.fixture(scope="module")
def nat():
    from nanochat_b200.ops import native
    return native


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _mk(shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(shape, device="cuda", generator=g) * scale


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K,bn", [
    (256, 256, 64, 256), (512, 256, 192, 256), (512, 416, 128, 208), (768, 128, 320, 128),
    (304, 520, 136, 256), (1280, 1664, 1664, 208), (4992, 1664, 2048, 256),
])
def test_pair_gemm_layouts(nat, M, N, K, bn, a_mn, b_mn):
    A = _mk((K, M) if a_mn else (M, K), seed=1).to(BF16)
    B = _mk((K, N) if b_mn else (N, K), seed=2).to(BF16)
    C = torch.empty(M, N, dtype=BF16, device="cuda")
    nat.gemm(A, B, C, a_mn=a_mn, b_mn=b_mn, bn=bn, pair=1)
    nat.check_status(C)
    ref = (A.float().t() if a_mn else A.float()) @ (B.float() if b_mn else B.float().t())
    assert _rel_err(C, ref) < 1e-2, (M, N, K, bn, a_mn, b_mn)


def test_pair_gemm_epilogues_batched_and_accumulate(nat):
    M, N, K = 512, 512, 256
    A, B = _mk((M, K), seed=3).to(BF16), _mk((N, K), seed=4).to(BF16)
    ref = A.float() @ B.float().t()
    out = torch.empty(M, N, dtype=BF16, device="cuda")
    nat.gemm(A, B, out, epi=nat.EPI_RELU2, pair=1)
    assert _rel_err(out, torch.relu(ref) ** 2) < 1e-2
    aux = _mk((M, N), seed=5).to(BF16)
    nat.gemm(A, B, out, aux=aux, alpha=0.5, beta=2.0, pair=1)
    assert _rel_err(out, 0.5 * ref + 2.0 * aux.float()) < 1e-2
    # wgrad form: fp32 C += A^T B, both operands MN-major, twice into the same buffer
    dy, x = _mk((1024, M), seed=6).to(BF16), _mk((1024, N), seed=7).to(BF16)
    acc = torch.zeros(M, N, device="cuda")
    nat.gemm(dy, x, acc, a_mn=True, b_mn=True, pair=1)
    nat.gemm(dy, x, acc, a_mn=True, b_mn=True, aux=acc, beta=1.0, pair=1)
    assert _rel_err(acc, 2 * (dy.float().t() @ x.float())) < 1e-2
    # batched
    Ab, Bb = _mk((3, M, K), seed=8).to(BF16), _mk((3, N, K), seed=9).to(BF16)
    Cb = torch.empty(3, M, N, dtype=BF16, device="cuda")
    nat.gemm(Ab, Bb, Cb, pair=1)
    assert _rel_err(Cb, Ab.float() @ Bb.float().transpose(1, 2)) < 1e-2
    nat.check_status(Cb)


def _quant(x, dtype):
    """Per-tensor scaling to the format's range; returns (fp8 tensor, de-quantisation scale as a CUDA scalar)."""
    fmax = torch.finfo(dtype).max
    scale = x.abs().max().float().clamp(min=1e-12) / fmax
    return (x.float() / scale).clamp(-fmax, fmax).to(dtype), scale.reshape(1)


@pytest.mark.parametrize("pair", [0, 1])
@pytest.mark.parametrize("M,N,K,bn", [(256, 256, 128, 256), (512, 416, 384, 208), (384, 128, 256, 128), (1024, 1664, 1664, 0)])
def test_fp8_gemm_three_layouts(nat, M, N, K, bn, pair):
    e4, e5 = torch.float8_e4m3fn, torch.float8_e5m2
    if pair and bn == 0:
        bn = 256
    # forward: y = x W^T, both e4m3, K-major
    x, w = _mk((M, K), seed=1), _mk((N, K), seed=2, scale=0.05)
    xq, sx = _quant(x, e4)
    wq, sw = _quant(w, e4)
    y = torch.empty(M, N, dtype=BF16, device="cuda")
    nat.gemm(xq, wq, y, scale_a=sx, scale_b=sw, bn=bn, pair=pair)
    ref = (xq.float() * sx) @ (wq.float() * sw).t()
    assert _rel_err(y, ref) < 1e-2
    assert _rel_err(y, x @ w.t()) < 8e-2          # quantisation error of e4m3 x e4m3
    # dgrad: dx = dy W, dy e5m2 (K-major, reduction over N), W e4m3 read MN-major
    dy = _mk((M, N), seed=3, scale=1e-3)
    dyq, sdy = _quant(dy, e5)
    dx = torch.empty(M, K, dtype=BF16, device="cuda")
    nat.gemm(dyq, wq, dx, b_mn=True, scale_a=sdy, scale_b=sw, pair=pair)
    ref = (dyq.float() * sdy) @ (wq.float() * sw)
    assert _rel_err(dx, ref) < 1e-2
    # wgrad: dW = dy^T x, both MN-major, fp32 accumulate
    dw = torch.zeros(N, K, device="cuda")
    nat.gemm(dyq, xq, dw, a_mn=True, b_mn=True, scale_a=sdy, scale_b=sx, pair=pair)
    ref = (dyq.float() * sdy).t() @ (xq.float() * sx)
    assert _rel_err(dw, ref) < 1e-2
    nat.check_status(y)


def test_gemm_amax_output(nat):
    M, N, K = 512, 384, 256
    A, B = _mk((M, K), seed=3).to(BF16), _mk((N, K), seed=4).to(BF16)
    out = torch.empty(M, N, dtype=BF16, device="cuda")
    amax = torch.zeros(1, device="cuda")
    nat.gemm(A, B, out, amax_out=amax)
    assert abs(amax.item() - out.float().abs().max().item()) <= 1e-2 * amax.item()


@pytest.mark.parametrize("batch,n,k,tall", [(3, 640, 320, False), (2, 384, 512, False), (2, 1664, 256, False),
                                            (2, 904, 448, True), (1, 128, 64, False)])
def test_symmetric_output_gemm_matches_the_full_product(nat, batch, n, k, tall):
    """X X^T (or X^T X) computed on the tiles on and above the diagonal only, then mirrored, is the full product;
    the second Newton-Schulz product b A + c A A (auxiliary operand, alpha, beta) likewise."""
    X = (_mk((batch, k, n) if tall else (batch, n, k), seed=5) / k ** 0.5).to(BF16)
    kw = dict(a_mn=True, b_mn=True) if tall else {}
    full = torch.empty(batch, n, n, dtype=BF16, device="cuda")
    nat.gemm(X, X, full, **kw)
    sym = torch.full((batch, n, n), float("nan"), dtype=BF16, device="cuda")   # untouched elements would show
    nat.gemm(X, X, sym, symmetric=True, **kw)
    nat.check_status(sym)
    ref = X.float().transpose(1, 2) @ X.float() if tall else X.float() @ X.float().transpose(1, 2)
    assert _rel_err(full, ref) < 1e-2
    assert torch.equal(sym, sym.transpose(1, 2))
    assert torch.equal(torch.triu(sym), torch.triu(full))
    full2 = torch.empty_like(full)
    nat.gemm(full, full, full2, aux=full, alpha=0.7, beta=-1.3)
    sym2 = torch.full_like(full, float("nan"))
    nat.gemm(sym, sym, sym2, aux=sym, alpha=0.7, beta=-1.3, symmetric=True)
    nat.check_status(sym2)
    assert not sym2.float().isnan().any()
    assert _rel_err(sym2, full2) < 1e-2


@pytest.mark.parametrize("pair", [0, 1])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("M,N,K,bn", [(512, 416, 192, 208), (768, 512, 128, 256), (600, 1664, 256, 208), (384, 384, 64, 128)])
def test_fused_epilogues_with_an_auxiliary_operand(nat, M, N, K, bn, b_mn, pair):
    """Residual add, relu, multiply-by-auxiliary and 2 sqrt(auxiliary): the kernels that request the auxiliary tile
    ahead of its use (forward and activation-gradient layouts, 256 / 208 / 128-wide tiles), in place and out of place."""
    A = (_mk((M, K), seed=11) / K ** 0.5).to(BF16)
    B = _mk((K, N) if b_mn else (N, K), seed=12).to(BF16)
    aux = _mk((M, N), seed=13).abs().to(BF16)
    prod = A.float() @ (B.float() if b_mn else B.float().t())
    kw = dict(b_mn=b_mn, bn=bn, pair=pair)
    cases = {
        "residual": (dict(aux=aux, beta=0.5, alpha=1.5), 1.5 * prod + 0.5 * aux.float()),
        "mulaux": (dict(aux=aux, epi=nat.EPI_MULAUX, alpha=2.0), 2.0 * prod * aux.float()),
        "mul2sqrt": (dict(aux=aux, epi=nat.EPI_MUL2SQRT), prod * 2.0 * aux.float().sqrt()),
        "relu": (dict(epi=nat.EPI_RELU), prod.clamp_min(0)),
        "relu2": (dict(epi=nat.EPI_RELU2), prod.clamp_min(0) ** 2),
    }
    for name, (extra, want) in cases.items():
        C = torch.empty(M, N, dtype=BF16, device="cuda")
        amax = torch.zeros(1, device="cuda")
        nat.gemm(A, B, C, amax_out=amax, **kw, **extra)
        nat.check_status(C)
        assert _rel_err(C, want) < 1e-2, name
        assert abs(amax.item() - C.float().abs().max().item()) <= 1e-2 * amax.item() + 1e-6, name
    inplace = aux.clone()                                   # accumulate into the auxiliary operand itself
    nat.gemm(A, B, inplace, aux=inplace, beta=1.0, **kw)
    nat.check_status(inplace)
    assert _rel_err(inplace, prod + aux.float()) < 1e-2
