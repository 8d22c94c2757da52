"""
GPU numerics: every hand-written kernel against a plain PyTorch fp32 reference of the same op.
"""
import math

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
    return (torch.randn(shape, device="cuda", generator=g) * scale).to(BF16)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K,bn", [
    (128, 256, 64, 256), (256, 208, 128, 208), (384, 128, 320, 128), (200, 72, 136, 64),
    (96, 32, 64, 32), (1024, 1664, 1664, 0), (512, 4992, 1664, 0),
])
def test_gemm_layouts(nat, M, N, K, bn, a_mn, b_mn):
    A = _mk((K, M) if a_mn else (M, K), seed=1)
    B = _mk((K, N) if b_mn else (N, K), seed=2)
    C = torch.empty(M, N, dtype=BF16, device="cuda")
    nat.gemm(A, B, C, a_mn=a_mn, b_mn=b_mn, bn=bn)
    Af = A.float().t() if a_mn else A.float()
    Bf = B.float() if b_mn else B.float().t()
    ref = Af @ Bf
    nat.check_status(C)
    assert _rel_err(C, ref) < 1e-2, (M, N, K, bn, a_mn, b_mn)


def test_gemm_epilogues_and_fp32_accumulate(nat):
    M, N, K = 512, 384, 256
    A, B = _mk((M, K), seed=3), _mk((N, K), seed=4)
    ref = A.float() @ B.float().t()
    out = torch.empty(M, N, dtype=BF16, device="cuda")
    nat.gemm(A, B, out, epi=nat.EPI_RELU2)
    assert _rel_err(out, torch.relu(ref) ** 2) < 1e-2
    aux = _mk((M, N), seed=5)
    nat.gemm(A, B, out, aux=aux, alpha=0.5, beta=2.0)
    assert _rel_err(out, 0.5 * ref + 2.0 * aux.float()) < 1e-2
    pos = aux.float().abs().to(BF16)
    nat.gemm(A, B, out, aux=pos, epi=nat.EPI_MUL2SQRT)
    assert _rel_err(out, ref * 2 * pos.float().sqrt()) < 1e-2
    # wgrad form: fp32 C += A^T B with both operands MN-major
    dy, x = _mk((K, M), seed=6), _mk((K, N), seed=7)       # reduction dim first
    acc = torch.randn(M, N, device="cuda")
    want = acc + dy.float().t() @ x.float()
    nat.gemm(dy, x, acc, a_mn=True, b_mn=True, aux=acc, beta=1.0)
    nat.check_status(acc)
    assert _rel_err(acc, want) < 2e-3


def test_gemm_batched_and_strided(nat):
    k, r, c = 5, 256, 384
    X = _mk((k, r, c), seed=8)
    A = torch.empty(k, r, r, dtype=BF16, device="cuda")
    nat.gemm(X, X, A)
    assert _rel_err(A, X.float() @ X.float().mT) < 1e-2
    At = torch.empty(k, c, c, dtype=BF16, device="cuda")
    nat.gemm(X, X, At, a_mn=True, b_mn=True)
    assert _rel_err(At, X.float().mT @ X.float()) < 1e-2
    # column-sliced output (ldc > N) as used by the unfused QKV path
    big = torch.zeros(r, 3 * 128, dtype=BF16, device="cuda")
    W = _mk((128, c), seed=9)
    nat.gemm(X[0], W, big[:, 128:256])
    assert _rel_err(big[:, 128:256], X[0].float() @ W.float().t()) < 1e-2
    assert big[:, :128].abs().max().item() == 0 and big[:, 256:].abs().max().item() == 0
    nat.check_status(big)


def test_gemm_deterministic(nat):
    A, B = _mk((1024, 512), seed=10), _mk((768, 512), seed=11)
    o1 = torch.empty(1024, 768, dtype=BF16, device="cuda")
    o2 = torch.empty_like(o1)
    nat.gemm(A, B, o1)
    nat.gemm(A, B, o2)
    assert torch.equal(o1, o2)


def _torch_layer_reference(model, x, x0, idx, i):
    """One block through the reference op bodies (autograd-capable)."""
    from nanochat_b200 import ops
    ops.set_kernel_mode("torch")
    try:
        T = x.shape[1]
        cos_sin = model.cos[:, :T], model.sin[:, :T]
        from nanochat_b200.ops import reference as R
        xm, xn = R.resid_mix_norm(x, x0, model.resid_lambdas[i], model.x0_lambdas[i])
        ve_w = model.value_embeds[str(i)].weight if str(i) in model.value_embeds else None
        return model.transformer.h[i](xm, xn, idx, ve_w, cos_sin, model.window_sizes[i], None)
    finally:
        ops.set_kernel_mode("native")


def _tiny_model(n_layer=2, n_embd=256, n_head=2, seq=256, window="SL"):
    from nanochat_b200.models.gpt import GPT, GPTConfig
    cfg = GPTConfig(sequence_len=seq, vocab_size=2048, n_layer=n_layer, n_head=n_head, n_kv_head=n_head,
                    n_embd=n_embd, window_pattern=window)
    torch.manual_seed(0)
    with torch.device("meta"):
        m = GPT(cfg)
    m.to_empty(device="cuda")
    m.init_weights()
    # projections are zero-initialised; randomise them so every gradient path carries signal
    with torch.no_grad():
        for blk in m.transformer.h:
            blk.attn.c_proj.weight.normal_(0, 0.02)
            blk.mlp.c_proj.weight.normal_(0, 0.02)
        m.lm_head.weight.normal_(0, 0.05)
        m.smear_lambda.fill_(0.3)
    return m


@pytest.mark.parametrize("layer", [0, 1])
def test_layer_forward_backward_matches_reference(nat, layer):
    m = _tiny_model()
    B, T, C = 2, 256, 256
    idx = torch.randint(0, 2048, (B, T), device="cuda")
    x = _mk((B, T, C), seed=20).requires_grad_(True)
    x0 = _mk((B, T, C), seed=21).requires_grad_(True)
    ve_w = m.value_embeds[str(layer)].weight if str(layer) in m.value_embeds else None
    cos_sin = m.cos[:, :T], m.sin[:, :T]
    out = nat.layer_forward(m.transformer.h[layer], x, x0, idx, ve_w, cos_sin, m.window_sizes[layer],
                            m.resid_lambdas, m.x0_lambdas, layer)
    g = _mk((B, T, C), seed=22)
    out.backward(g)
    nat.check_status(out)
    got = dict(out=out.detach().clone(), dx=x.grad.clone(), dx0=x0.grad.clone(),
               dfc=m.transformer.h[layer].mlp.c_fc.weight.grad.clone(),
               dq=m.transformer.h[layer].attn.c_q.weight.grad.clone(),
               dv=m.transformer.h[layer].attn.c_v.weight.grad.clone(),
               dlr=m.resid_lambdas.grad.clone(), dl0=m.x0_lambdas.grad.clone())
    if ve_w is not None:
        got["dve"] = ve_w.grad32.clone()
        got["dwg"] = m.transformer.h[layer].attn.ve_gate.weight.grad.clone()
    m.zero_grad(set_to_none=True)
    x.grad = x0.grad = None
    ref_out = _torch_layer_reference(m, x, x0, idx, layer)
    ref_out.backward(g)
    want = dict(out=ref_out.detach(), dx=x.grad, dx0=x0.grad,
                dfc=m.transformer.h[layer].mlp.c_fc.weight.grad,
                dq=m.transformer.h[layer].attn.c_q.weight.grad,
                dv=m.transformer.h[layer].attn.c_v.weight.grad,
                dlr=m.resid_lambdas.grad, dl0=m.x0_lambdas.grad)
    if ve_w is not None:
        want["dve"] = ve_w.grad
        want["dwg"] = m.transformer.h[layer].attn.ve_gate.weight.grad
    for key in got:
        err = _rel_err(got[key], want[key])
        assert err < 4e-2, f"{key}: rel err {err}"


def test_model_loss_and_grads_match_torch_path(nat):
    from nanochat_b200 import ops
    m = _tiny_model(n_layer=4, window="SSSL")
    B, T = 2, 256
    idx = torch.randint(0, 2048, (B, T), device="cuda")
    tgt = torch.randint(0, 2048, (B, T), device="cuda")
    tgt[0, :7] = -1
    loss = m(idx, tgt)
    loss.backward()
    nat.check_status(loss)
    got = {n: (getattr(p, "grad32", None) if p.grad is None else p.grad).clone() for n, p in m.named_parameters()}
    for p in m.parameters():
        p.grad = None
        if hasattr(p, "grad32"):
            p.grad32.zero_()
    ops.set_kernel_mode("torch")
    try:
        ref_loss = m(idx, tgt)
        ref_loss.backward()
    finally:
        ops.set_kernel_mode("native")
    assert abs(loss.item() - ref_loss.item()) < 2e-2, (loss.item(), ref_loss.item())
    bad = []
    for n, p in m.named_parameters():
        if n == "backout_lambda":
            # d/dlam = -<dz, x_backout> where dz is orthogonal to z ~ (1-lam) x_backout + small: the sum cancels
            # almost completely, so in bf16 both paths return rounding noise (the kernel has its own test below)
            continue
        err = _rel_err(got[n], p.grad)
        if err > 8e-2:
            bad.append((n, err))
    assert not bad, bad
    per_tok = m(idx, tgt, loss_reduction="none")
    ops.set_kernel_mode("torch")
    try:
        ref_tok = m(idx, tgt, loss_reduction="none")
    finally:
        ops.set_kernel_mode("native")
    assert per_tok.shape == ref_tok.shape
    assert (per_tok - ref_tok).abs().max().item() < 5e-2
    logits = m(idx)
    assert logits.shape == (B, T, 2048) and logits.dtype == torch.float32


def test_weighted_per_token_loss_backward_matches_torch_path(nat):
    """The policy-gradient objective: per-token losses times per-token advantages, summed (reduction 'none')."""
    from nanochat_b200 import ops
    m = _tiny_model(n_layer=2, window="SL")
    B, T = 2, 256
    idx = torch.randint(0, 2048, (B, T), device="cuda")
    tgt = torch.randint(0, 2048, (B, T), device="cuda")
    tgt[1, 100:] = -1                                          # padding carries no loss and no gradient
    adv = torch.randn(B, 1, device="cuda").expand(B, T).contiguous()

    def run():
        for p in m.parameters():
            p.grad = None
            if hasattr(p, "grad32"):
                p.grad32.zero_()
        per_tok = m(idx, tgt, loss_reduction="none").view(B, T)
        obj = (per_tok * adv).sum() / (tgt >= 0).sum()
        obj.backward()
        nat.check_status(obj)
        return obj.item(), {n: (getattr(p, "grad32", None) if p.grad is None else p.grad).float().clone()
                            for n, p in m.named_parameters()}
    obj, got = run()
    ops.set_kernel_mode("torch")
    try:
        ref_obj, ref = run()
    finally:
        ops.set_kernel_mode("native")
    assert abs(obj - ref_obj) < 2e-2, (obj, ref_obj)
    bad = [(n, _rel_err(got[n], ref[n])) for n in ref
           if n != "backout_lambda" and ref[n].numel() >= 64 and _rel_err(got[n], ref[n]) > 8e-2]
    assert not bad, bad


def test_quantize_kernels_match_torch(nat):
    x = (_mk((384, 512), seed=11).float() * 3).to(BF16)
    for dt in (torch.float8_e4m3fn, torch.float8_e5m2):
        q, inv = nat.quantize(x[:, :256], dt)          # strided rows
        fmax = torch.finfo(dt).max
        amax = x[:, :256].float().abs().max()
        ref = (x[:, :256].float() * (fmax / amax)).clamp(-fmax, fmax).to(dt)
        assert abs(inv.item() - (amax / fmax).item()) <= 1e-6 * inv.item()
        assert torch.equal(q.view(torch.uint8), ref.view(torch.uint8))


def test_fp8_layer_path_close_to_bf16_path(nat):
    """Loss and gradients of the tiny model with the fp8 linear layers stay within fp8 noise of the bf16 run."""
    m = _tiny_model(n_layer=4, window="SSSL")
    B, T = 2, 256
    idx = torch.randint(0, 2048, (B, T), device="cuda")
    tgt = torch.randint(0, 2048, (B, T), device="cuda")

    from nanochat_b200.parallel.arena import ParamArena
    ParamArena(m)            # contiguous QKV shadows: the fused (and therefore fp8) projection path

    def run():
        m._arena.zero_grads()
        loss = m(idx, tgt)
        loss.backward()
        nat.check_status(loss)
        return loss.item(), {n: (getattr(p, "grad32", None) if p.grad is None else p.grad).float().clone()
                             for n, p in m.named_parameters()}
    ref_loss, ref = run()
    nat.set_fp8(True)
    try:
        loss, got = run()
        # a second run after a weight change must pick the new weights up
        with torch.no_grad():
            m.lm_head.weight.mul_(0.5)
        nat.bump_weights_epoch()
        loss_half, _ = run()
    finally:
        nat.set_fp8(False)
    assert abs(loss - ref_loss) < 3e-2, (loss, ref_loss)
    assert abs(loss_half - loss) > 1e-3
    bad = []
    for n in ref:
        if n == "backout_lambda" or ref[n].numel() < 64:
            continue
        err = _rel_err(got[n], ref[n])
        if err > 0.25:
            bad.append((n, err))
    assert not bad, bad


def test_fp8_layer_path_matches_the_scaled_mm_module_recipe(nat):
    """The fused fp8 layer kernels against the reference recipe run independently: the same model on the plain-PyTorch
    op bodies with every linear swapped for the tensorwise `Float8Linear`, whose three products are `torch._scaled_mm`
    calls on operands quantised by torch (reference: nanochat/fp8.py:125-192). Differences left: one scale for the
    fused QKV weight instead of three, bf16 rounding points of the fused kernels."""
    from nanochat_b200 import ops
    from nanochat_b200.fp8 import Float8LinearConfig, convert_to_float8_training, default_fp8_filter
    from nanochat_b200.parallel.arena import ParamArena
    B, T = 2, 256
    g = torch.Generator(device="cuda").manual_seed(5)
    idx = torch.randint(0, 2048, (B, T), device="cuda", generator=g)
    tgt = torch.randint(0, 2048, (B, T), device="cuda", generator=g)
    ours = _tiny_model(n_layer=4, window="SSSL")
    ParamArena(ours)
    nat.set_fp8(True)
    try:
        loss = ours(idx, tgt)
        loss.backward()
        nat.check_status(loss)
    finally:
        nat.set_fp8(False)
    assert nat.stats["fp8_layer_forward"] > 0
    got = {n: (getattr(p, "grad32", None) if p.grad is None else p.grad).float().clone() for n, p in ours.named_parameters()}
    ops.set_kernel_mode("torch")
    try:
        ref_model = _tiny_model(n_layer=4, window="SSSL")
        convert_to_float8_training(ref_model, config=Float8LinearConfig.from_recipe_name("tensorwise"),
                                   module_filter_fn=default_fp8_filter)
        ref_loss = ref_model(idx, tgt)
        ref_loss.backward()
    finally:
        ops.set_kernel_mode("native")
    assert abs(loss.item() - ref_loss.item()) < 3e-2, (loss.item(), ref_loss.item())
    bad = []
    for n, p in ref_model.named_parameters():
        if p.grad is None or p.numel() < 64 or n == "backout_lambda":
            continue
        err = _rel_err(got[n], p.grad.float())
        if err > 0.25:
            bad.append((n, round(err, 3)))
    assert not bad, bad


def test_adamw_kernel_matches_reference(nat):
    from nanochat_b200.ops import reference as R
    for dtype in (torch.float32, BF16):
        p = torch.randn(4096, 64, device="cuda").to(dtype)
        g = torch.randn(4096, 64, device="cuda")
        m1, v1 = torch.zeros_like(p), torch.zeros_like(p)
        p2, m2, v2 = p.clone(), m1.clone(), v1.clone()
        for step in range(1, 4):
            nat.adamw_update(p, g, m1, v1, step, 0.01, 0.8, 0.95, 1e-10, 0.01)
            R.adamw_update(p2, g, m2, v2, step, 0.01, 0.8, 0.95, 1e-10, 0.01)
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        assert _rel_err(p, p2) < tol


@pytest.mark.parametrize("shape", [(3, 256, 256), (2, 256, 512), (2, 512, 256)])
def test_muon_kernel_matches_reference(nat, shape):
    from nanochat_b200.ops import reference as R
    k, r, c = shape
    torch.manual_seed(1)
    p = torch.randn(shape, device="cuda") * 0.02
    g = torch.randn(shape, device="cuda")
    mom = torch.zeros_like(p)
    sec = torch.zeros((k, r, 1) if r >= c else (k, 1, c), device="cuda")
    p2, g2, mom2, sec2 = p.clone(), g.clone(), mom.clone(), sec.clone()
    red_dim = -1 if r >= c else -2
    for _ in range(2):
        nat.muon_update(g.clone(), p, mom, sec, 0.95, 0.02, 0.1, 0.9, 5, red_dim)
        R.muon_update(g2.clone(), p2, mom2, sec2, 0.95, 0.02, 0.1, 0.9, 5, red_dim, use_bf16=True)
    nat.check_status(p)
    assert _rel_err(mom, mom2) < 1e-5
    assert _rel_err(sec, sec2) < 5e-2
    assert _rel_err(p, p2) < 5e-2
    # the first update must be close to semi-orthogonal (a square Gaussian matrix has singular values
    # arbitrarily close to zero that five polar steps cannot lift, so only rectangular shapes are checked)
    if r == c:
        return
    p3 = torch.zeros(1, r, c, device="cuda")
    nat.muon_update(torch.randn(1, r, c, device="cuda"), p3, torch.zeros_like(p3),
                    torch.zeros((1, r, 1) if r >= c else (1, 1, c), device="cuda"), 0.95, 1.0, 0.0, 0.9, 5, red_dim)
    s = torch.linalg.svdvals(p3[0].float())
    assert (s.max() / s.min()).item() < 4


@pytest.mark.parametrize("B,T,H,Hkv,window", [
    (2, 256, 2, 2, -1), (1, 512, 4, 4, 128), (2, 384, 4, 2, 256), (1, 1024, 2, 2, 256), (1, 200, 2, 1, 64),
])
def test_flash_attention_forward(nat, B, T, H, Hkv, window):
    from nanochat_b200.ops import reference as R
    D = 128
    qkv = _mk((B, T, (H + 2 * Hkv) * D), seed=30)
    q = qkv[..., :H * D].view(B, T, H, D)                      # strided views, as the layer uses them
    k = qkv[..., H * D:(H + Hkv) * D].view(B, T, Hkv, D)
    v = qkv[..., (H + Hkv) * D:].view(B, T, Hkv, D)
    y = torch.empty(B, T, H, D, dtype=BF16, device="cuda")
    lse = torch.empty(B, H, T, dtype=torch.float32, device="cuda")
    nat._C.attn_fwd(q, k, v, y, lse, window, 1.0 / math.sqrt(D))
    nat.check_status(y)
    ref = R.attention(q.float(), k.float(), v.float(), window)
    assert _rel_err(y, ref) < 2e-2
    # log-sum-exp against an explicit computation
    kk = k.float().repeat_interleave(H // Hkv, dim=2)
    s = torch.einsum("bthd,bshd->bhts", q.float(), kk) / math.sqrt(D)
    i = torch.arange(T, device="cuda")[:, None]
    j = torch.arange(T, device="cuda")[None, :]
    mask = j <= i
    if window >= 0:
        mask = mask & (i - j <= window)
    s = s.masked_fill(~mask, float("-inf"))
    assert (lse - torch.logsumexp(s, dim=-1)).abs().max().item() < 2e-2


@pytest.mark.parametrize("Tq,Tk,window", [(128, 384, -1), (1, 300, -1), (72, 1000, 256), (300, 556, 128)])
def test_flash_attention_forward_queries_at_the_end_of_longer_keys(nat, Tq, Tk, window):
    """Chunked inference: Tq new queries attend to Tk cached keys, aligned to their end."""
    from nanochat_b200.ops import reference as R
    B, H, Hkv, D = 2, 4, 2, 128
    q = _mk((B, Tq, H, D), seed=50)
    k = _mk((B, Tk, Hkv, D), seed=51)
    v = _mk((B, Tk, Hkv, D), seed=52)
    y, lse = nat.attention_forward(q, k, v, window)
    assert lse is not None
    nat.check_status(y)
    ref = R.attention(q.float(), k.float(), v.float(), window)
    assert _rel_err(y, ref) < 2e-2, (Tq, Tk, window)


@pytest.mark.parametrize("B,T,H,Hkv,window", [
    (2, 256, 2, 2, -1), (1, 512, 4, 4, 128), (2, 384, 4, 2, 256), (1, 200, 2, 1, 64), (1, 1024, 2, 2, 512),
])
def test_flash_attention_backward(nat, B, T, H, Hkv, window):
    from nanochat_b200.ops import reference as R
    D = 128
    qkv = _mk((B, T, (H + 2 * Hkv) * D), seed=40)
    q = qkv[..., :H * D].view(B, T, H, D)
    k = qkv[..., H * D:(H + Hkv) * D].view(B, T, Hkv, D)
    v = qkv[..., (H + Hkv) * D:].view(B, T, Hkv, D)
    dy = _mk((B, T, H, D), seed=41)
    y = torch.empty(B, T, H, D, dtype=BF16, device="cuda")
    lse = torch.empty(B, H, T, dtype=torch.float32, device="cuda")
    scale = 1.0 / math.sqrt(D)
    amax_y = torch.zeros(1, device="cuda")
    nat._C.attn_fwd(q, k, v, y, lse, window, scale, amax_y)
    true_max = y.float().abs().max().item()
    assert true_max <= amax_y.item() <= 1.01 * true_max, (true_max, amax_y.item())      # the fp8 scale's input
    dqkv = torch.zeros_like(qkv)
    dq = dqkv[..., :H * D].view(B, T, H, D)
    dk = dqkv[..., H * D:(H + Hkv) * D].view(B, T, Hkv, D)
    dv = dqkv[..., (H + Hkv) * D:].view(B, T, Hkv, D)
    delta = torch.empty(B, H, T, dtype=torch.float32, device="cuda")
    amax_dv = torch.zeros(1, device="cuda")
    nat._C.attn_bwd(q, k, v, y, lse, dy, dq, dk, dv, delta, window, scale, amax_dv)
    nat.check_status(y)
    true_max = dv.float().abs().max().item()
    assert true_max <= amax_dv.item() <= 1.01 * true_max, (true_max, amax_dv.item())
    qf, kf, vf = (t.float().detach().requires_grad_(True) for t in (q, k, v))
    ref = R.attention(qf, kf, vf, window)
    ref.backward(dy.float())
    assert _rel_err(dq, qf.grad) < 3e-2, "dq"
    assert _rel_err(dk, kf.grad) < 3e-2, "dk"
    assert _rel_err(dv, vf.grad) < 3e-2, "dv"
    # fixed reduction order, no atomics: a second run gives the same bits
    first, y_first = dqkv.clone(), y.clone()
    nat._C.attn_fwd(q, k, v, y, lse, window, scale, None)
    nat._C.attn_bwd(q, k, v, y, lse, dy, dq, dk, dv, delta, window, scale, None)
    nat.check_status(y)
    assert torch.equal(y, y_first) and torch.equal(dqkv, first)


def test_backout_norm_kernels_against_fp32_oracle(nat):
    M, C = 512, 256
    x = _mk((M, C), seed=50).requires_grad_(False)
    xb = _mk((M, C), seed=51)
    dy = _mk((M, C), seed=52)
    lam = torch.tensor([0.2], device="cuda")
    y = torch.empty(M, C, dtype=BF16, device="cuda")
    nat._C.backout_norm_fwd(x, xb, lam, y)
    dx, dxb = torch.empty_like(x), torch.empty_like(x)
    dlam = torch.zeros(1, device="cuda")
    nat._C.backout_norm_bwd(dy, x, xb, lam, dx, dxb, dlam)
    xf, xbf = x.float().requires_grad_(True), xb.float().requires_grad_(True)
    lf = lam.clone().requires_grad_(True)
    z = xf - lf.to(BF16).float() * xbf
    yf = z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + 1.1920929e-07)
    yf.backward(dy.float())
    assert _rel_err(y, yf) < 1e-2
    assert _rel_err(dx, xf.grad) < 2e-2 and _rel_err(dxb, xbf.grad) < 2e-2
    assert abs(dlam.item() - lf.grad.item()) < 2e-2 * abs(lf.grad.item()) + 0.5


def test_bounded_wait_reports_a_peer_that_never_arrives(nat):
    """Failure detection without a fault: a 2-rank barrier whose peer slot nothing ever sets. The wait gives up
    after its limit, the kernel returns normally, and the host reads which peer and which epoch it waited for."""
    import time
    my_pad = torch.zeros(64, dtype=torch.int32, device="cuda")
    peer_pad = torch.zeros(64, dtype=torch.int32, device="cuda")     # stands in for the absent rank's pad
    nat.check_status(my_pad)                                         # clean slate
    t0 = time.time()
    nat._C.p2p_barrier([my_pad.data_ptr(), peer_pad.data_ptr()], 0, 1, my_pad)
    with pytest.raises(RuntimeError, match="failed wait: code=5"):
        nat.check_status(my_pad)
    assert 1.0 < time.time() - t0 < 20.0                             # it waited its limit, not forever
    assert my_pad[0].item() == 1 and peer_pad[0].item() == 1         # this rank did announce itself
    nat.check_status(my_pad)                                         # the status word was consumed: clean again
    # the context is intact: an ordinary kernel still runs
    x = torch.ones(8, 256, device="cuda", dtype=BF16)
    y = torch.empty_like(x)
    nat._C.norm_fwd(x, y, None)
    assert torch.isfinite(y.float()).all()
