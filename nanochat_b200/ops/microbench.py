"""
Micro-benchmarks of the hand-written kernels, one operation per invocation:

    python -m nanochat_b200.ops.microbench gemm --m 32768 --n 4992 --k 1664 --layout fwd
    python -m nanochat_b200.ops.microbench attn_fwd --batch 16 --seq 2048 --heads 13 --window -1
    python -m nanochat_b200.ops.microbench attn_bwd --batch 2 --iters 1 --warmup 1      # small: profiler runs

Timing follows the usual hygiene: warm-up launches, a write larger than L2 between timed launches,
CUDA events on the launching stream, median of the timed launches. Prints one JSON line with the
time, the achieved TFLOP/s (useful FLOPs only: masked attention blocks are not counted) and, when a
`MEASURED_PEAKS.json` with this machine's measured cuBLAS bf16 rate lies in the working directory,
the fraction of that rate.
"""
import argparse
import json
import os

import torch


def _time(fn, iters, warmup, flush=True):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    scratch = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda") if flush else None
    times = []
    for _ in range(iters):
        if scratch is not None:
            scratch.zero_()                      # evict the previous launch's working set from L2
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2]


def _attn_pairs(T, window):
    if window < 0 or window >= T:
        return T * (T + 1) // 2
    return sum(min(i, window) + 1 for i in range(T))


def _operand(shape, dtype):
    """Random operand; 8-bit floats come with the de-quantisation scale of a per-tensor scaling."""
    x = torch.randn(shape, device="cuda")
    if dtype == "bf16":
        return x.to(torch.bfloat16), None
    t = torch.float8_e4m3fn
    scale = x.abs().max() / torch.finfo(t).max
    return (x / scale).to(t), scale.reshape(1).float()


def bench_gemm(args, nat):
    m, n, k = args.m, args.n, args.k
    bf16 = torch.bfloat16
    dev = "cuda"
    if args.dtype == "mxfp8":        # block-scaled fp8, y[m,n] = x[m,k] W[n,k]^T with both operands scaled along k
        assert args.layout == "fwd", "the block-scaled GEMM takes K-major operands: quantise along the reduction dim"
        A = torch.randn(m, k, device=dev).to(bf16)
        B = torch.randn(n, k, device=dev).to(bf16)
        (aq, asf), (bq, bsf) = nat.mx_quantize(A), nat.mx_quantize(B)
        C = torch.empty(m, n, device=dev, dtype=bf16)
        ms = _time(lambda: nat.gemm_mx(aq, asf, bq, bsf, C, bn=args.bn), args.iters, args.warmup)
        ms_q = _time(lambda: nat.mx_quantize(A), args.iters, args.warmup)
        return dict(op="gemm_mx/fwd", dtype="mxfp8", m=m, n=n, k=k, bn=args.bn, ms=ms, tflops=2.0 * m * n * k / ms / 1e9,
                    quantize_a_ms=ms_q, quantize_a_gbs=(m * k * 3 + m * k / 32) / ms_q / 1e6)
    if args.dtype == "fp8" or args.pair >= 0:
        shapes = {"fwd": ((m, k), (n, k)), "dgrad": ((m, k), (k, n)), "wgrad": ((k, m), (k, n))}[args.layout]
        (A, sa), (B, sb) = _operand(shapes[0], args.dtype), _operand(shapes[1], args.dtype)
        wg = args.layout == "wgrad"
        C = torch.zeros(m, n, device=dev, dtype=torch.float32 if wg else bf16)
        kw = dict(a_mn=wg, b_mn=args.layout != "fwd", bn=args.bn, pair=args.pair, scale_a=sa, scale_b=sb)
        if wg:
            kw.update(aux=C, beta=1.0)
        ms = _time(lambda: nat.gemm(A, B, C, **kw), args.iters, args.warmup)
        return dict(op=f"gemm/{args.layout}", dtype=args.dtype, pair=args.pair, m=m, n=n, k=k, bn=args.bn, ms=ms,
                    tflops=2.0 * m * n * k / ms / 1e9)
    if args.layout == "fwd":        # y[m,n] = x[m,k] W[n,k]^T
        A = torch.randn(m, k, device=dev).to(bf16)
        B = torch.randn(n, k, device=dev).to(bf16)
        C = torch.empty(m, n, device=dev, dtype=bf16)
        fn = lambda: nat.gemm(A, B, C, bn=args.bn)
    elif args.layout == "dgrad":    # dx[m,n] = dy[m,k] W[k,n]   (B is MN-major)
        A = torch.randn(m, k, device=dev).to(bf16)
        B = torch.randn(k, n, device=dev).to(bf16)
        C = torch.empty(m, n, device=dev, dtype=bf16)
        fn = lambda: nat.gemm(A, B, C, b_mn=True, bn=args.bn)
    elif args.layout == "wgrad":    # dW[m,n] (fp32) += dy[k,m]^T x[k,n]   (both MN-major)
        A = torch.randn(k, m, device=dev).to(bf16)
        B = torch.randn(k, n, device=dev).to(bf16)
        C = torch.zeros(m, n, device=dev, dtype=torch.float32)
        fn = lambda: nat.gemm(A, B, C, a_mn=True, b_mn=True, aux=C, beta=1.0, bn=args.bn)
    else:
        raise SystemExit(f"unknown layout {args.layout}")
    ms = _time(fn, args.iters, args.warmup)
    return dict(op=f"gemm/{args.layout}", m=m, n=n, k=k, bn=args.bn, ms=ms, tflops=2.0 * m * n * k / ms / 1e9)


def _attn_inputs(args):
    B, T, H, D = args.batch, args.seq, args.heads, 128
    qkv = torch.randn(B, T, 3 * H * D, device="cuda").to(torch.bfloat16)
    q = qkv[..., :H * D].view(B, T, H, D)
    k = qkv[..., H * D:2 * H * D].view(B, T, H, D)
    v = qkv[..., 2 * H * D:].view(B, T, H, D)
    return qkv, q, k, v


def bench_attn_fwd(args, nat):
    _, q, k, v = _attn_inputs(args)
    ms = _time(lambda: nat.attention_forward(q, k, v, args.window), args.iters, args.warmup)
    flops = 4.0 * args.batch * args.heads * _attn_pairs(args.seq, args.window) * 128
    return dict(op="attn_fwd", batch=args.batch, seq=args.seq, heads=args.heads, window=args.window, ms=ms,
                tflops=flops / ms / 1e9)


def bench_attn_bwd(args, nat):
    qkv, q, k, v = _attn_inputs(args)
    B, T, H, D = q.shape
    y, lse = nat.attention_forward(q, k, v, args.window)
    dy = torch.randn(B, T, H, D, device="cuda").to(torch.bfloat16)
    dqkv = torch.empty_like(qkv)
    views = (dqkv[..., :H * D].view(B, T, H, D), dqkv[..., H * D:2 * H * D].view(B, T, H, D),
             dqkv[..., 2 * H * D:].view(B, T, H, D))
    ms = _time(lambda: nat.attention_backward(dy, q, k, v, y, lse, args.window, views), args.iters, args.warmup)
    flops = 10.0 * B * H * _attn_pairs(T, args.window) * D
    return dict(op="attn_bwd", batch=B, seq=T, heads=H, window=args.window, ms=ms, tflops=flops / ms / 1e9)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("op", choices=["gemm", "attn_fwd", "attn_bwd"])
    ap.add_argument("--m", type=int, default=32768)
    ap.add_argument("--n", type=int, default=4992)
    ap.add_argument("--k", type=int, default=1664)
    ap.add_argument("--bn", type=int, default=0, help="N tile (0 = heuristic)")
    ap.add_argument("--layout", default="fwd", choices=["fwd", "dgrad", "wgrad"])
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp8", "mxfp8"], help="GEMM operand type")
    ap.add_argument("--pair", type=int, default=-1, help="GEMM: 1 = CTA-pair kernel, 0 = single-CTA kernel, -1 = library choice")
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=13)
    ap.add_argument("--window", type=int, default=-1)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    from nanochat_b200.ops import native as nat
    torch.manual_seed(0)
    res = {"gemm": bench_gemm, "attn_fwd": bench_attn_fwd, "attn_bwd": bench_attn_bwd}[args.op](args, nat)
    nat.check_status()
    if os.path.exists("MEASURED_PEAKS.json"):
        with open("MEASURED_PEAKS.json") as f:
            peak = json.load(f).get("bf16_tflops")
        if peak:
            res["frac_of_measured_bf16_peak"] = res["tflops"] / peak
    print(json.dumps(res))


if __name__ == "__main__":
    main()
