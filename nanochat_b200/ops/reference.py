"""
Plain-PyTorch definitions of every fused op of the model.

These functions are (a) the CPU execution path, (b) the autograd-capable oracle
the CUDA kernels are tested against, and (c) the precise statement of what each
hand-written sm_100a kernel computes. They use only differentiable torch ops so
`torch.autograd` provides the backward on this path.

Each op cites the reference lines whose arithmetic it reproduces
(reference: nanochat/gpt.py unless stated otherwise).
"""


import torch
import torch.nn.functional as F

QK_SCALE = 1.2          # gpt.py:103-104
VE_GATE_CHANNELS = 12   # gpt.py:81
SMEAR_CHANNELS = 24     # gpt.py:185
SOFTCAP = 15.0          # gpt.py:511


def rms_norm(x):
    """Parameter-free RMSNorm over the last dim, eps = fp32 machine epsilon (gpt.py:42-43)."""
    return F.rms_norm(x, (x.size(-1),))


def embed_norm_smear(idx, wte, gate_w, lam, compute_dtype):
    """Token embedding -> RMSNorm -> smear (gpt.py:471-480).

    Returns (x, last) where `last` is the normalised, pre-smear embedding of the
    final position (what the KV cache keeps as `prev_embedding`).
    """
    x = rms_norm(F.embedding(idx, wte).to(compute_dtype))
    last = x[:, -1:, :]
    if x.size(1) > 1:
        gate = lam.to(x.dtype) * torch.sigmoid(F.linear(x[:, 1:, :SMEAR_CHANNELS], gate_w.to(x.dtype)))
        x = torch.cat([x[:, :1], x[:, 1:] + gate * x[:, :-1]], dim=1)
    return x, last


def resid_mix_norm(x, x0, resid_lambda, x0_lambda):
    """x <- rl*x + xl*x0 ; returns (x, norm(x))  (gpt.py:500 and the norm of gpt.py:151)."""
    x = resid_lambda * x + x0_lambda * x0
    return x, rms_norm(x)


def linear(x, w):
    """y = x @ w.T with w cast to the activation dtype (gpt.py:45-50)."""
    return F.linear(x, w.to(x.dtype))


def linear_relu2(x, w):
    """relu(x @ w.T)^2 (gpt.py:138-139)."""
    return F.relu(F.linear(x, w.to(x.dtype))).square()


def ve_gate_add(v, xn, gate_w, ve_w, idx):
    """v + 3*sigmoid(xn[..., :12] @ gate_w.T)[..., None] * ve_w[idx]  (gpt.py:94-97).

    v: (B,T,Hkv,D); xn: (B,T,C); gate_w: (Hkv,12); ve_w: (V,Hkv*D).
    """
    B, T, H, D = v.shape
    ve = F.embedding(idx, ve_w).to(v.dtype).view(B, T, H, D)
    gate = 3 * torch.sigmoid(F.linear(xn[..., :VE_GATE_CHANNELS], gate_w.to(xn.dtype)))
    return v + gate.unsqueeze(-1) * ve


def _rope(x, cos, sin):
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    return torch.cat([x1 * cos + x2 * sin, x2 * cos - x1 * sin], dim=-1)


def rope_qknorm(q, k, cos, sin):
    """Half-split rotary (rotation by -theta), then RMSNorm, then x1.2 (gpt.py:57-65,100-104).

    q: (B,T,H,D), k: (B,T,Hkv,D), cos/sin: (1,T,1,D/2).
    """
    q = rms_norm(_rope(q, cos, sin)) * QK_SCALE
    k = rms_norm(_rope(k, cos, sin)) * QK_SCALE
    return q, k


def attention(q, k, v, window_left):
    """Causal attention over (B,T,H,D) tensors; query i sees keys j in [i-window_left, i].

    `window_left < 0` or `>= T` means unlimited (flash_attention.py:77-110). When
    Tq < Tk the queries are aligned to the END of the keys (chunked inference).
    """
    Tq, Tk = q.size(1), k.size(1)
    qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    gqa = qh.size(1) != kh.size(1)
    unlimited = window_left < 0 or window_left >= Tk
    if unlimited and Tq == Tk:
        y = F.scaled_dot_product_attention(qh, kh, vh, is_causal=True, enable_gqa=gqa)
    else:
        rows = (Tk - Tq) + torch.arange(Tq, device=q.device).unsqueeze(1)
        cols = torch.arange(Tk, device=q.device).unsqueeze(0)
        mask = cols <= rows
        if not unlimited:
            mask = mask & ((rows - cols) <= window_left)
        y = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=mask, enable_gqa=gqa)
    return y.transpose(1, 2)


def add_norm(x, delta):
    """x <- x + delta ; returns (x, norm(x))  (residual adds of gpt.py:151-152)."""
    x = x + delta
    return x, rms_norm(x)


def backout_norm(x, x_backout, lam):
    """norm(x - lam * x_backout)  (gpt.py:506-508)."""
    if x_backout is not None:
        x = x - lam.to(x.dtype) * x_backout
    return rms_norm(x)


def softcap_logits(x, w, vocab_size, softcap=SOFTCAP):
    """fp32 soft-capped logits over the un-padded vocabulary (gpt.py:511-515)."""
    logits = F.linear(x, w.to(x.dtype))[..., :vocab_size].float()
    return softcap * torch.tanh(logits / softcap)


def softcap_cross_entropy(x, w, targets, vocab_size, reduction="mean", softcap=SOFTCAP):
    """lm_head -> softcap -> cross entropy with ignore_index=-1 (gpt.py:510-521).

    'mean' returns a scalar, 'none' returns per-position losses shaped like targets
    flattened (B*T,), 0 at ignored positions.
    """
    logits = softcap_logits(x, w, vocab_size, softcap)
    return F.cross_entropy(logits.view(-1, logits.size(-1)), targets.reshape(-1),
                           ignore_index=-1, reduction=reduction)


def sample_next_token(logits, rng, temperature=1.0, top_k=None):
    """(B,V) logits -> (B,1) token ids (engine.py:141-156)."""
    assert temperature >= 0.0, "temperature must be non-negative"
    if temperature == 0.0:
        return torch.argmax(logits, dim=-1, keepdim=True)
    if top_k is not None and top_k > 0:
        k = min(top_k, logits.size(-1))
        vals, idx = torch.topk(logits, k, dim=-1)
        probs = F.softmax(vals / temperature, dim=-1)
        choice = torch.multinomial(probs, num_samples=1, generator=rng)
        return idx.gather(1, choice)
    probs = F.softmax(logits / temperature, dim=-1)
    return torch.multinomial(probs, num_samples=1, generator=rng)


# ----------------------------------------------------------------------------
# optimizer math (reference: nanochat/optim.py)

POLAR_EXPRESS_COEFFS = (
    (8.156554524902461, -22.48329292557795, 15.878769915207462),
    (4.042929935166739, -2.808917465908714, 0.5000178451051316),
    (3.8916678022926607, -2.772484153217685, 0.5060648178503393),
    (3.285753657755655, -2.3681294933425376, 0.46449024233003106),
    (2.3465413258596377, -1.7097828382687081, 0.42323551169305323),
)


@torch.no_grad()
def adamw_update(p, grad, exp_avg, exp_avg_sq, step, lr, beta1, beta2, eps, wd):
    """Decoupled-WD AdamW in fp32 with write-back in the storage dtype (optim.py:44-63)."""
    p32, g32 = p.float(), grad.float()
    m32, v32 = exp_avg.float(), exp_avg_sq.float()
    p32.mul_(1 - lr * wd)
    m32.lerp_(g32, 1 - beta1)
    v32.lerp_(g32.square(), 1 - beta2)
    bias1 = 1 - beta1 ** step
    bias2 = 1 - beta2 ** step
    denom = (v32 / bias2).sqrt() + eps
    p32.add_(m32 / denom, alpha=-(lr / bias1))
    p.copy_(p32)
    exp_avg.copy_(m32)
    exp_avg_sq.copy_(v32)


@torch.no_grad()
def polar_express(X, ns_steps):
    """Quintic polar iteration on a (k,r,c) stack; tall matrices iterate on X^T X (optim.py:143-154)."""
    X = X / (X.norm(dim=(-2, -1), keepdim=True) * 1.01 + 1e-6)
    if X.size(-2) > X.size(-1):
        for a, b, c in POLAR_EXPRESS_COEFFS[:ns_steps]:
            A = X.mT @ X
            B = b * A + c * (A @ A)
            X = a * X + X @ B
    else:
        for a, b, c in POLAR_EXPRESS_COEFFS[:ns_steps]:
            A = X @ X.mT
            B = b * A + c * (A @ A)
            X = a * X + B @ X
    return X


@torch.no_grad()
def muon_update(grads, params, momentum_buf, second_buf, momentum, lr, wd, beta2, ns_steps, red_dim,
                use_bf16):
    """One Muon step on stacked (k,r,c) tensors, in place on params and both buffers.

    Nesterov momentum -> row equilibration -> polar iteration -> Frobenius renorm ->
    factored second-moment rescale -> cautious weight decay (optim.py:130-180).
    `grads` is clobbered.
    """
    momentum_buf.lerp_(grads, 1 - momentum)
    g = grads.lerp_(momentum_buf, momentum)
    X = g.bfloat16() if use_bf16 else g
    target = X.float().norm(dim=(-2, -1), keepdim=True) / (X.size(-2) ** 0.5)
    row_norm = X.float().norm(dim=-1, keepdim=True).clamp_min(1e-6)
    X = X * (target / row_norm).to(X.dtype)
    X = polar_express(X, ns_steps)
    g = X.to(params.dtype)
    target_norm = min(g.size(-2), g.size(-1)) ** 0.5
    cur = g.float().norm(dim=(-2, -1), keepdim=True).clamp_min(1e-6)
    g = g * (target_norm / cur).to(g.dtype)
    v_mean = g.float().square().mean(dim=red_dim, keepdim=True)
    n_red = g.size(red_dim)
    v_norm = (v_mean.sum(dim=(-2, -1), keepdim=True) * n_red).sqrt()
    second_buf.lerp_(v_mean.to(second_buf.dtype), 1 - beta2)
    step_size = second_buf.clamp_min(1e-10).rsqrt()
    v_norm_new = ((v_mean * n_red) * step_size.float().square()).sum(dim=(-2, -1), keepdim=True).sqrt()
    g = g * (step_size * (v_norm / v_norm_new.clamp_min(1e-10))).to(g.dtype)
    mask = (g * params) >= 0
    params.sub_(lr * g + lr * wd * params * mask)
