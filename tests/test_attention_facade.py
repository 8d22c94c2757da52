"""
The attention facade on CPU (SDPA body) against an explicit masked-softmax oracle written here: causal,
sliding window, grouped-query heads, gradients, cache prefill, single-token decode, a window shorter than the
filled cache, the implementation override switch. On a B200 the same contracts run against the native kernels
in tests/test_gpu_kernels.py.
"""
import math

import pytest
import torch

from nanochat_b200 import flash_attention as fa


def _oracle(q, k, v, window):
    """q: (B,Tq,H,D), k/v: (B,Tk,Hkv,D); queries are the LAST Tq positions of the keys. fp32 masked softmax."""
    B, Tq, H, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    rep = H // Hkv
    kf = k.float().repeat_interleave(rep, dim=2)
    vf = v.float().repeat_interleave(rep, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), kf) / math.sqrt(D)
    qpos = torch.arange(Tk - Tq, Tk).view(Tq, 1)
    kpos = torch.arange(Tk).view(1, Tk)
    ok = kpos <= qpos
    if window >= 0:
        ok &= kpos >= qpos - window                  # a left window of w admits w + 1 keys
    s = s.masked_fill(~ok, float("-inf"))
    return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, dim=-1), vf)


def _rand(*shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g)


@pytest.fixture(autouse=True)
def _sdpa_body():
    old = fa._override_impl
    fa._override_impl = "sdpa"
    yield
    fa._override_impl = old


@pytest.mark.parametrize("T,H,Hkv,window", [(64, 4, 4, -1), (96, 4, 4, 16), (50, 6, 2, -1), (80, 4, 1, 7), (33, 2, 2, 0),
                                            (40, 2, 2, 1000)])
def test_training_attention_matches_oracle(T, H, Hkv, window):
    q, k, v = _rand(2, T, H, 32, seed=1), _rand(2, T, Hkv, 32, seed=2), _rand(2, T, Hkv, 32, seed=3)
    y = fa.flash_attn.flash_attn_func(q, k, v, causal=True, window_size=(window, 0))
    assert y.shape == q.shape
    assert torch.allclose(y, _oracle(q, k, v, window), atol=2e-5, rtol=1e-4)


def test_gradients_match_oracle():
    q, k, v = (_rand(1, 48, 4, 16, seed=s).requires_grad_(True) for s in (4, 5, 6))
    dy = _rand(1, 48, 4, 16, seed=7)
    fa.flash_attn.flash_attn_func(q, k, v, causal=True, window_size=(12, 0)).backward(dy)
    got = [t.grad.clone() for t in (q, k, v)]
    for t in (q, k, v):
        t.grad = None
    _oracle(q, k, v, 12).backward(dy)
    for g, t, name in zip(got, (q, k, v), "qkv"):
        assert torch.allclose(g, t.grad, atol=2e-5, rtol=1e-4), name


def test_only_causal_attention_is_offered():
    q = _rand(1, 8, 2, 16, seed=8)
    with pytest.raises(AssertionError):
        fa.flash_attn.flash_attn_func(q, q, q, causal=False)


def test_cache_prefill_then_single_tokens_equal_full_attention():
    B, Tmax, H, Hkv, D, Tp = 2, 40, 4, 2, 16, 17
    k_all, v_all = _rand(B, Tmax, Hkv, D, seed=9), _rand(B, Tmax, Hkv, D, seed=10)
    q_all = _rand(B, Tmax, H, D, seed=11)
    kc, vc = torch.zeros(B, Tmax, Hkv, D), torch.zeros(B, Tmax, Hkv, D)
    seqlens = torch.zeros(B, dtype=torch.int32)
    y = fa.flash_attn.flash_attn_with_kvcache(q_all[:, :Tp], kc, vc, k=k_all[:, :Tp], v=v_all[:, :Tp],
                                              cache_seqlens=seqlens, causal=True, window_size=(-1, 0))
    full = _oracle(q_all, k_all, v_all, -1)
    assert torch.allclose(y, full[:, :Tp], atol=2e-5, rtol=1e-4)
    assert torch.equal(kc[:, :Tp], k_all[:, :Tp]) and torch.equal(vc[:, :Tp], v_all[:, :Tp])      # appended in place
    assert kc[:, Tp:].abs().sum() == 0
    for t in range(Tp, Tmax):                                    # decode: one position at a time
        seqlens.fill_(t)
        y = fa.flash_attn.flash_attn_with_kvcache(q_all[:, t:t + 1], kc, vc, k=k_all[:, t:t + 1], v=v_all[:, t:t + 1],
                                                  cache_seqlens=seqlens, causal=True, window_size=(-1, 0))
        assert y.shape == (B, 1, H, D)
        assert torch.allclose(y, full[:, t:t + 1], atol=2e-5, rtol=1e-4), t
    assert torch.equal(kc, k_all)


def test_decode_with_a_window_shorter_than_the_cache():
    B, T, H, D, window = 1, 30, 2, 16, 5
    k_all, v_all, q_all = _rand(B, T, H, D, seed=12), _rand(B, T, H, D, seed=13), _rand(B, T, H, D, seed=14)
    kc, vc = k_all.clone(), v_all.clone()
    kc[:, T - 1], vc[:, T - 1] = 0, 0                            # the last position arrives with the call
    seqlens = torch.full((B,), T - 1, dtype=torch.int32)
    y = fa.flash_attn.flash_attn_with_kvcache(q_all[:, -1:], kc, vc, k=k_all[:, -1:], v=v_all[:, -1:],
                                              cache_seqlens=seqlens, causal=True, window_size=(window, 0))
    want = _oracle(q_all, k_all, v_all, window)[:, -1:]
    assert torch.allclose(y, want, atol=2e-5, rtol=1e-4)
    # keys outside the window do not matter: scrambling them leaves the output unchanged
    kc2, vc2 = kc.clone(), vc.clone()
    kc2[:, : T - 1 - window] = 7.0
    vc2[:, : T - 1 - window] = -3.0
    seqlens.fill_(T - 1)
    y2 = fa.flash_attn.flash_attn_with_kvcache(q_all[:, -1:], kc2, vc2, k=k_all[:, -1:], v=v_all[:, -1:],
                                               cache_seqlens=seqlens, causal=True, window_size=(window, 0))
    assert torch.allclose(y2, want, atol=2e-5, rtol=1e-4)


def test_chunked_prefill_into_a_partly_filled_cache():
    B, H, D = 1, 2, 16
    k_all, v_all, q_all = _rand(B, 24, H, D, seed=15), _rand(B, 24, H, D, seed=16), _rand(B, 24, H, D, seed=17)
    kc, vc = torch.zeros(B, 32, H, D), torch.zeros(B, 32, H, D)
    seqlens = torch.zeros(B, dtype=torch.int32)
    outs = []
    for lo, hi in ((0, 10), (10, 24)):
        seqlens.fill_(lo)
        outs.append(fa.flash_attn.flash_attn_with_kvcache(q_all[:, lo:hi], kc, vc, k=k_all[:, lo:hi], v=v_all[:, lo:hi],
                                                          cache_seqlens=seqlens, causal=True, window_size=(8, 0)))
    assert torch.allclose(torch.cat(outs, dim=1), _oracle(q_all, k_all, v_all, 8), atol=2e-5, rtol=1e-4)


def test_override_switch():
    from nanochat_b200 import ops
    q = _rand(1, 4, 2, 16, seed=18)
    fa._override_impl = None
    assert fa._want_native(q) is False or ops.use_native(q)      # CPU tensors never take the native body on their own
    fa._override_impl = "sdpa"
    assert fa._want_native(q) is False
    fa._override_impl = "native"
    assert fa._want_native(q) is True
