"""
The allocation-free attention-backward entry point, called through its exported C symbol.

Some callers cannot allocate device memory where they need the backward pass (a fixed, pre-sized
memory pool; a host application that owns all buffers). For them the library keeps the kernel's
scratch vector inside its own image. This test calls `nc_attention_bwd_noalloc` twice in a row via
ctypes (two different shapes) and checks dq/dk/dv against the regular (caller-allocated scratch) entry
point, and that an oversized problem, a null or misaligned pointer and a stride that is not a whole
number of 16-byte vectors are refused with a clear error before anything is launched. It is collected
last on purpose.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

BF16 = torch.bfloat16


def _lib():
    from nanochat_b200.utils.build import build_cuda_extension
    from nanochat_b200.ops import native  # noqa: F401  (libtorch and the extension are loaded)
    lib = ctypes.CDLL(build_cuda_extension())
    fn = lib.nc_attention_bwd_noalloc
    P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    fn.argtypes = [P] * 9 + [I] * 5 + [L] * 9 + [I, ctypes.c_float, P]
    fn.restype = I
    lib.nc_noalloc_status.argtypes = [P]
    lib.nc_noalloc_status.restype = I
    lib.nc_noalloc_last_error.restype = ctypes.c_char_p
    return lib


def _problem(seed, B, T, H, Hkv):
    D = 128
    g = torch.Generator(device="cuda").manual_seed(seed)
    qkv = torch.randn(B, T, (H + 2 * Hkv) * D, device="cuda", generator=g).to(BF16)
    q = qkv[..., :H * D].view(B, T, H, D)
    k = qkv[..., H * D:(H + Hkv) * D].view(B, T, Hkv, D)
    v = qkv[..., (H + Hkv) * D:].view(B, T, Hkv, D)
    d_o = torch.randn(B, T, H, D, device="cuda", generator=g).to(BF16)
    return q, k, v, d_o


def _call(lib, q, k, v, o, lse, d_o, dq, dk, dv, window, scale):
    B, T, H, _ = q.shape
    Hkv = k.shape[2]
    stream = torch.cuda.current_stream().cuda_stream
    return lib.nc_attention_bwd_noalloc(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), d_o.data_ptr(),
        dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, T, T, H, Hkv,
        q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
        o.stride(0), o.stride(1), o.stride(2), window, scale, stream)


def test_noalloc_entry_matches_regular_entry_twice():
    from nanochat_b200.ops import native as nat
    lib = _lib()
    scale = 1.0 / math.sqrt(128)
    for call, (seed, B, T, H, Hkv, window) in enumerate([(1, 2, 384, 4, 2, 128), (2, 1, 512, 2, 2, -1)]):
        q, k, v, d_o = _problem(seed, B, T, H, Hkv)
        o = torch.empty(B, T, H, 128, dtype=BF16, device="cuda")
        lse = torch.empty(B, H, T, dtype=torch.float32, device="cuda")
        nat._C.attn_fwd(q, k, v, o, lse, window, scale)
        want = torch.zeros(B, T, (H + 2 * Hkv) * 128, dtype=BF16, device="cuda")
        got = torch.zeros_like(want)

        def views(buf):
            return (buf[..., :H * 128].view(B, T, H, 128), buf[..., H * 128:(H + Hkv) * 128].view(B, T, Hkv, 128),
                    buf[..., (H + Hkv) * 128:].view(B, T, Hkv, 128))
        delta = torch.empty(B, H, T, dtype=torch.float32, device="cuda")
        nat._C.attn_bwd(q, k, v, o, lse, d_o, *views(want), delta, window, scale)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = _call(lib, q, k, v, o, lse, d_o, *views(got), window, scale)
        assert rc == 0, lib.nc_noalloc_last_error().decode()
        assert lib.nc_noalloc_status(torch.cuda.current_stream().cuda_stream) == 0, lib.nc_noalloc_last_error().decode()
        assert torch.cuda.memory_allocated() == before
        err = ((got.float() - want.float()).norm() / want.float().norm()).item()
        assert err < 1e-2, f"call {call}: rel err {err}"
        nat.check_status(q)


def test_noalloc_entry_rejects_oversized_problem():
    lib = _lib()
    q, k, v, d_o = _problem(3, 1, 128, 2, 2)
    o = torch.empty(1, 128, 2, 128, dtype=BF16, device="cuda")
    lse = torch.empty(1, 2, 128, dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    # claim a batch so large that B*H*Tq exceeds the built-in scratch; nothing is launched
    rc = lib.nc_attention_bwd_noalloc(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), d_o.data_ptr(),
        q.data_ptr(), k.data_ptr(), v.data_ptr(), 8192, 128, 128, 2, 2,
        q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
        o.stride(0), o.stride(1), o.stride(2), -1, 0.1, stream)
    assert rc == 1
    assert b"exceeds" in lib.nc_noalloc_last_error()


def test_noalloc_entry_rejects_bad_pointers_and_strides():
    """Each of these must come back as code 2 from the host-side checks: nothing reaches the GPU."""
    from nanochat_b200.ops import native as nat
    lib = _lib()
    q, k, v, d_o = _problem(4, 1, 128, 2, 2)
    o = torch.empty(1, 128, 2, 128, dtype=BF16, device="cuda")
    lse = torch.empty(1, 2, 128, dtype=torch.float32, device="cuda")
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    stream = torch.cuda.current_stream().cuda_stream

    def call(ptrs, q_strides, kv_strides, o_strides):
        return lib.nc_attention_bwd_noalloc(*ptrs, 1, 128, 128, 2, 2, *q_strides, *kv_strides, *o_strides, -1, 0.1, stream)
    good = [t.data_ptr() for t in (q, k, v, o, lse, d_o, dq, dk, dv)]
    qs, ks, os_ = list(q.stride()[:3]), list(k.stride()[:3]), list(o.stride()[:3])
    null = list(good)
    null[3] = None
    assert call(null, qs, ks, os_) == 2 and b"null" in lib.nc_noalloc_last_error()
    odd = list(good)
    odd[0] += 2                                     # one bf16 element past a 16-byte boundary
    assert call(odd, qs, ks, os_) == 2 and b"aligned" in lib.nc_noalloc_last_error()
    assert call(good, [qs[0], qs[1] + 4, qs[2]], ks, os_) == 2 and b"strides" in lib.nc_noalloc_last_error()
    assert call(good, qs, [ks[0], ks[1], 0], os_) == 2
    assert call(good, qs, ks, [os_[0], os_[1], 64]) == 2 and b"head stride" in lib.nc_noalloc_last_error()
    torch.cuda.synchronize()
    nat.check_status(q)
