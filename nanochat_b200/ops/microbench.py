"""
Micro-benchmarks of the hand-written kernels, one operation per invocation:

    python -m nanochat_b200.ops.microbench gemm --m 32768 --n 4992 --k 1664 --layout fwd
    python -m nanochat_b200.ops.microbench attn_fwd --batch 16 --seq 2048 --heads 13 --window -1
    python -m nanochat_b200.ops.microbench attn_bwd --batch 2 --iters 1 --warmup 1      # small: profiler runs
    python -m nanochat_b200.ops.microbench sweep --m 32768     # the memory-bound kernels against their algorithmic bytes

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
        elif args.epi != "linear":     # the MLP's fused epilogues: relu^2 on the way out, or its derivative from the saved output
            kw.update(epi={"relu2": nat.EPI_RELU2, "mul2sqrt": nat.EPI_MUL2SQRT, "relu": nat.EPI_RELU,
                           "mulaux": nat.EPI_MULAUX, "residual": nat.EPI_LINEAR}[args.epi])
            if args.epi in ("mul2sqrt", "mulaux", "residual"):
                kw.update(aux=torch.rand(m, n, device=dev).to(bf16), beta=1.0)
        if args.amax:
            kw.update(amax_out=torch.zeros(1, device=dev))
        ms = _time(lambda: nat.gemm(A, B, C, **kw), args.iters, args.warmup)
        return dict(op=f"gemm/{args.layout}", dtype=args.dtype, pair=args.pair, epi=args.epi, m=m, n=n, k=k, bn=args.bn,
                    ms=ms, tflops=2.0 * m * n * k / ms / 1e9)
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


def bench_sweep(args, nat):
    """The memory-bound kernels of a training / decode step on d26-shaped operands (inputs larger than L2, about 2 GB
    held in total): device time per launch (CUDA events), algorithmic bytes per launch and the fraction of the measured
    copy bandwidth. Run the same command under `ncu -k regex:... --section SpeedOfLight` for the DRAM counters."""
    C_ = nat._C
    bf16 = torch.bfloat16
    dev = "cuda"
    M, C, H = args.m, 1664, 13
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape: torch.randn(*shape, device=dev, generator=g).to(bf16)
    rows = []

    def add(name, fn, nbytes):
        ms = _time(fn, args.iters, args.warmup)
        rows.append(dict(kernel=name, ms=round(ms, 4), algorithmic_mb=round(nbytes / 1e6, 1), gbs=round(nbytes / ms / 1e6, 1)))

    x, x0 = rnd(M, C), rnd(M, C)
    xm, xn = torch.empty_like(x), torch.empty_like(x)
    lam_r, lam_0 = torch.ones(26, device=dev), torch.full((26,), 0.1, device=dev)
    amax = torch.zeros(1, device=dev)
    add("mixnorm_fwd_kernel", lambda: C_.mixnorm_fwd(x, x0, lam_r, lam_0, 3, xm, xn, amax), 4 * M * C * 2)
    add("norm_fwd_kernel", lambda: C_.norm_fwd(x, xn, amax), 2 * M * C * 2)
    dxn, dres = rnd(M, C), rnd(M, C)
    dx, dx0 = torch.empty_like(x), torch.empty_like(x)
    dlr, dl0 = torch.zeros(26, device=dev), torch.zeros(26, device=dev)
    add("mixnorm_bwd_kernel", lambda: C_.mixnorm_bwd(dxn, dres, None, xm, x, x0, lam_r, lam_0, 3, dx, dx0, False, dlr, dl0, amax),
        7 * M * C * 2)
    add("normadd_bwd_kernel", lambda: C_.normadd_bwd(dxn, x, dres, dx, amax), 4 * M * C * 2)
    q8 = torch.empty(M, C, dtype=torch.float8_e4m3fn, device=dev)
    inv = torch.empty(1, device=dev)
    am = x.float().abs().max().reshape(1)
    add("quantize_bf16_kernel", lambda: C_.quantize_bf16(x, am, q8, inv), M * C * 3)
    add("amax_bf16_kernel", lambda: C_.amax_bf16(x, amax), M * C * 2)
    sfb = torch.full((nat.mx_scale_bytes(M, C),), 127, dtype=torch.uint8, device=dev)
    add("mx_quantize_bf16_kernel", lambda: C_.mx_quantize(x, q8, sfb), M * C * 3 + M * C // 32)
    # rotary + QK-norm on the fused QKV buffer
    T = 2048
    qkv = rnd(M, 3 * H * 128)
    cos, sin = rnd(T, 64), rnd(T, 64)
    rstd = torch.empty(M, 2 * H, device=dev)
    add("qkv_post_fwd_kernel", lambda: C_.qkv_post_fwd(qkv, H, H, cos, sin, T, rstd, None, None, None, None),
        2 * M * 2 * H * 128 * 2)
    dqkv = rnd(M, 3 * H * 128)
    add("qkv_post_bwd_kernel", lambda: C_.qkv_post_bwd(dqkv, qkv, H, H, cos, sin, T, rstd, None, None, None, None, None, None,
                                                      None, amax), 3 * M * 2 * H * 128 * 2)
    # loss head on a slice of the logits matrix (rows x 32768 bf16)
    R, V = max(2048, M // 8), 32768
    logits = (rnd(R, V) * 4)
    tgt = torch.randint(0, V, (R,), device=dev, generator=g)
    loss, lse = torch.empty(R, device=dev), torch.empty(R, device=dev)
    add("softcap_ce_fwd_kernel", lambda: C_.softcap_ce_fwd(logits, tgt, loss, lse, V, 15.0), R * V * 2)
    gs = torch.full((1,), 1.0 / R, device=dev)
    g8 = torch.empty(R, V, dtype=torch.float8_e5m2, device=dev)
    add("softcap_ce_bwd_fp8_kernel", lambda: C_.softcap_ce_bwd_fp8(logits, tgt, lse, gs, gs, g8, inv, V, 15.0), R * V * 3)
    # optimizer elementwise passes
    n = 32 * 1024 * 1024
    p32, g32 = torch.randn(n, device=dev), torch.randn(n, device=dev)
    m32, v32 = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    sh = torch.empty(n, dtype=bf16, device=dev)
    add("adamw_kernel<float,float>", lambda: C_.adamw_step(p32, g32, m32, v32, sh, 1e-3, 0.8, 0.95, 1e-10, 0.0, 3, 1.0),
        n * (4 * 4 + 3 * 4 + 2))
    k, r, c = 8, 1664, 1664
    P, X = torch.randn(k, r, c, device=dev), rnd(k, r, c)
    sec = torch.zeros(k, r, device=dev)
    ss, sc = torch.empty(k * r, device=dev), torch.empty(k * r, device=dev)
    shadow = torch.empty(k, r, c, dtype=bf16, device=dev)
    add("muon_finish (sumsq + stats + muon_apply_kernel)", lambda: C_.muon_finish(P, X, sec, ss, sc, shadow, 0.02, 0.1, 0.9),
        k * r * c * (2 + 2 + 4 + 4 + 2))
    # decode: weight-streaming GEMV and split-key attention
    W = rnd(4 * C, C)
    for B in (1, 8):
        xv, out = rnd(B, C), torch.empty(B, 4 * C, dtype=bf16, device=dev)
        add(f"gemv_rows_kernel<{B}>", lambda: C_.gemv_rows(xv, W, out, None, 0, False), W.numel() * 2)
    Bd, Tc = 8, 2048
    kc, vc = rnd(Bd, Tc, H, 128), rnd(Bd, Tc, H, 128)
    qd, yd = rnd(Bd, H * 128), torch.empty(Bd, H * 128, dtype=bf16, device=dev)
    seq = torch.full((Bd,), Tc - 1, dtype=torch.int32, device=dev)
    scratch = torch.zeros(C_.decode_attn_scratch(Bd, H), device=dev)
    add("decode_attn_kernel", lambda: C_.decode_attn(qd, kc, vc, seq, H, H, -1, 0.088, scratch, yd), 2 * kc.numel() * 2)
    peak = None
    if os.path.exists("MEASURED_PEAKS.json"):
        with open("MEASURED_PEAKS.json") as f:
            peak = json.load(f).get("hbm_gbs")
    for row in rows:
        if peak:
            row["frac_of_measured_hbm"] = round(row["gbs"] / peak, 3)
    return dict(op="sweep", rows_m=M, kernels=rows, measured_hbm_gbs=peak)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("op", choices=["gemm", "attn_fwd", "attn_bwd", "sweep"])
    ap.add_argument("--m", type=int, default=32768)
    ap.add_argument("--n", type=int, default=4992)
    ap.add_argument("--k", type=int, default=1664)
    ap.add_argument("--bn", type=int, default=0, help="N tile (0 = heuristic)")
    ap.add_argument("--layout", default="fwd", choices=["fwd", "dgrad", "wgrad"])
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp8", "mxfp8"], help="GEMM operand type")
    ap.add_argument("--pair", type=int, default=-1, help="GEMM: 1 = CTA-pair kernel, 0 = single-CTA kernel, -1 = library choice")
    ap.add_argument("--epi", default="linear", choices=["linear", "relu2", "mul2sqrt", "relu", "mulaux", "residual"], help="GEMM (fp8 / --pair): fused epilogue")
    ap.add_argument("--amax", type=int, default=0, help="GEMM (fp8 / --pair): 1 = the epilogue also reports max|output|")
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=13)
    ap.add_argument("--window", type=int, default=-1)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    from nanochat_b200.ops import native as nat
    torch.manual_seed(0)
    res = {"gemm": bench_gemm, "attn_fwd": bench_attn_fwd, "attn_bwd": bench_attn_bwd, "sweep": bench_sweep}[args.op](args, nat)
    nat.check_status()
    if os.path.exists("MEASURED_PEAKS.json"):
        with open("MEASURED_PEAKS.json") as f:
            peak = json.load(f).get("bf16_tflops")
        if peak and "tflops" in res:
            res["frac_of_measured_bf16_peak"] = res["tflops"] / peak
    print(json.dumps(res))


if __name__ == "__main__":
    main()
