"""
Attention entry points with the Flash-Attention call signature.

`flash_attn.flash_attn_func` (training / no cache) and
`flash_attn.flash_attn_with_kvcache` (prefill and decode against an in-place
updated cache) keep the argument conventions of the reference facade
(reference: nanochat/flash_attention.py:115-185): tensors are (B, T, H, D),
`window_size=(left, right)` with -1 = unlimited, a left window of w admits w+1
keys (the query's own position included).

Two bodies:
  * native — the sm_100a kernels (`ops.native`): tcgen05 flash forward/backward with
    causal + sliding-window tile skipping, and a split-KV decode kernel that appends
    the new K/V rows and reads positions from device memory (no host sync);
  * sdpa   — PyTorch SDPA with explicit masks; CPU path and numerical oracle.

`_override_impl` ('native' | 'sdpa' | None) lets tests pin either body.
"""

from types import SimpleNamespace


from nanochat_b200 import ops
from nanochat_b200.ops import reference as ref_ops

_override_impl = None  # 'native' | 'sdpa' | None (auto)
# The reference's flags for its prebuilt Hopper library; this package never loads it (the sm_100a kernels take its place).
HAS_FA3 = False
USE_FA3 = False


def _want_native(q):
    if _override_impl == "sdpa":
        return False
    if _override_impl == "native":
        return True
    return ops.use_native(q)


def flash_attn_func(q, k, v, causal=False, window_size=(-1, -1)):
    """Self-attention over whole sequences. q: (B,T,H,D); k,v: (B,T,Hkv,D). Returns (B,T,H,D)."""
    assert causal, "only causal attention is used by this model"
    if _want_native(q):
        return ops.native_module().attention(q, k, v, window_size[0])
    return ref_ops.attention(q, k, v, window_size[0])


def flash_attn_with_kvcache(q, k_cache, v_cache, k=None, v=None, cache_seqlens=None,
                            causal=False, window_size=(-1, -1)):
    """Append k,v at `cache_seqlens` (in place) and attend over the filled part of the cache.

    q: (B,Tn,H,D); caches: (B,Tmax,Hkv,D); k,v: (B,Tn,Hkv,D); cache_seqlens: (B,) int32.
    All rows are assumed to sit at the same position (the engine keeps them in lock-step).
    """
    if _want_native(q):
        return ops.native_module().attention_kvcache(q, k_cache, v_cache, k, v, cache_seqlens, window_size[0])
    B, Tn, H, D = q.shape
    pos = int(cache_seqlens[0].item())
    if k is not None and v is not None:
        k_cache[:, pos:pos + Tn] = k
        v_cache[:, pos:pos + Tn] = v
    end = pos + Tn
    return ref_ops.attention(q, k_cache[:, :end], v_cache[:, :end], window_size[0])


flash_attn = SimpleNamespace(
    flash_attn_func=flash_attn_func,
    flash_attn_with_kvcache=flash_attn_with_kvcache,
)
