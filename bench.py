"""
Headline benchmark: d26 pretraining throughput (tokens/sec over the whole job) on N B200s.

  python bench.py --gpus 1 --steps 3 --warmup 3
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
         --master-port P bench.py --gpus N --steps K --warmup W
  python bench.py --impl reference ...     # the unmodified reference from baseline/_ref

One "step" is a full optimizer step at the reference's d26 configuration: total batch
1,048,576 tokens = grad-accum x (device batch x 2048) x N, forward + backward for every
micro-batch, then MuonAdamW.step() (gradient averaging + Muon/AdamW updates) and gradient
reset. The total batch is fixed, so per-GPU work shrinks as N grows ("strong" scaling).

Two timed regions, both bracketed by barrier + cuda synchronize, CUDA events, max over ranks:
  value  - inputs already on the device (kernel-side throughput);
  e2e    - through the public API with, every micro-step, the host->device copy of that
           micro-batch from pinned memory, and every step a device->host read of the loss.
Data are uniform-random token ids, weights random-init (no network on the box).
"""

import argparse
import json
import os
import subprocess
import sys
import threading

ROOT = os.path.dirname(os.path.abspath(__file__))

PUBLISHED_TOK_PER_SEC = 764000.0   # reference d26 fp8, batch 1,048,576, 8xH100 (dev/LEADERBOARD.md run 3)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", type=str, default="ours", choices=["ours", "reference"])
    ap.add_argument("--depth", type=int, default=26)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--device-batch-size", type=int, default=16)
    ap.add_argument("--total-batch-size", type=int, default=1048576)
    ap.add_argument("--window-pattern", type=str, default="SSSL")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end region (debugging)")
    ap.add_argument("--no-decode", action="store_true",
                    help="skip the Engine decode sweep that is appended to the 1-GPU record")
    ap.add_argument("--decode-tokens", type=int, default=256)
    ap.add_argument("--comm", type=str, default="auto", choices=["auto", "fused", "nccl"],
                    help="optimizer collectives for N>1: fused peer-to-peer kernels or NCCL")
    ap.add_argument("--precision", type=str, default="fp8", choices=["fp8", "bf16", "mxfp8"],
                    help="our arm: fp8 = tensorwise e4m3/e5m2 linear layers (the reference's headline recipe); mxfp8 = "
                         "block-scaled fp8 on the hardware block-scaled GEMM (module path, not the fused layer path)")
    ap.add_argument("--ref-bf16", action="store_true", help="reference arm without --fp8")
    ap.add_argument("--ref-eager", action="store_true", help="reference arm without torch.compile")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks / throttle reasons of this rank's GPU with nvidia-smi during a timed region."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu_index), "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in self.rows:
            parts = [p.strip() for p in row.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def timed_region(torch, dist, world, steps, run_step):
    """Times `steps` calls of run_step() on the device; returns the max over ranks in milliseconds. The cyclic
    garbage collector is kept off inside the region, in both arms, as the reference's training loop does after its
    first step (scripts/base_train.py:588-594 there): a collection pausing one rank's host thread stalls every rank."""
    import gc
    gc.collect()
    gc.disable()
    try:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            run_step()
        t1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
    finally:
        gc.enable()
    ms = torch.tensor([t0.elapsed_time(t1)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms.item()


def shared_config(args, world, accum):
    """The benchmark configuration: the same keys and values in both arms."""
    return {"model": f"d{args.depth}", "global_batch": args.total_batch_size, "seq_len": args.seq_len,
            "device_batch": args.device_batch_size, "grad_accum": accum, "window_pattern": args.window_pattern,
            "parallelism": f"dp{world}",
            "l2": "inputs larger than L2 (activations of one micro-batch exceed 126 MB)"}


def losses_of(loss_log, args):
    """Last-micro-batch training loss of every step this process ran, in order: warm-up, timed, end-to-end
    (one extra untimed step opens the end-to-end region). Same seeds and data in both arms."""
    vals = [float(v) for v in loss_log]
    w, k = args.warmup, args.steps
    return {"warmup": vals[:w], "timed": vals[w:w + k], "e2e": vals[w + k:]}


def decode_sweep(args, impl):
    """Engine decode at the benchmark depth (bf16 random-init weights, 512-token prompt, temperature 1.0, top-k 50,
    batch 1/8/32/64) through scripts/infer_bench.py in a child process; returns its JSON record."""
    cmd = [sys.executable, "-m", "scripts.infer_bench", "--random-init", "--depth", str(args.depth),
           "--prompt-tokens", "512", "--decode-tokens", str(args.decode_tokens), "--batch-sizes", "1,8,32,64",
           "-t", "1.0", "-k", "50", "--impl", impl]
    env = dict(os.environ)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT"):
        env.pop(k, None)
    try:
        r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    except subprocess.TimeoutExpired:
        return {"unavailable": "decode sweep timed out"}
    lines = [ln for ln in r.stdout.strip().splitlines() if ln.startswith("{")]
    if r.returncode != 0 or not lines:
        return {"unavailable": f"decode sweep failed (exit {r.returncode}): {r.stderr.strip()[-300:]}"}
    rec = json.loads(lines[-1])
    keep = ("impl", "prompt_tokens", "decode_tokens", "temperature", "top_k", "prefill", "sweep", "unavailable")
    out = {k: rec[k] for k in keep if k in rec}
    out["command"] = " ".join(cmd[1:])
    return out


def build_ours(args, device):
    import torch
    from nanochat_b200.models.gpt import GPT, GPTConfig
    dim = -(-args.depth * 64 // 128) * 128
    cfg = GPTConfig(sequence_len=args.seq_len, vocab_size=32768, n_layer=args.depth, n_head=dim // 128,
                    n_kv_head=dim // 128, n_embd=dim, window_pattern=args.window_pattern)
    with torch.device("meta"):
        model = GPT(cfg)
    model.to_empty(device=device)
    model.init_weights()
    return model, cfg


def run_ours(args):
    import torch
    import torch.distributed as dist
    from nanochat_b200 import common, ops
    rank, local_rank, world = dist_env()
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    _, _, _, _, device = common.compute_init("cuda")
    assert common.COMPUTE_DTYPE == torch.bfloat16
    model, cfg = build_ours(args, device)
    dtype = "bf16"
    if args.precision == "fp8":
        from nanochat_b200.fp8 import Float8LinearConfig, convert_to_float8_training, default_fp8_filter
        convert_to_float8_training(model, config=Float8LinearConfig.from_recipe_name("tensorwise"),
                                   module_filter_fn=default_fp8_filter)
        dtype = "fp8 (tensorwise e4m3/e5m2 linears, bf16 elsewhere)"
    elif args.precision == "mxfp8":
        from nanochat_b200.fp8 import Float8LinearConfig, convert_to_float8_training, default_fp8_filter
        convert_to_float8_training(model, config=Float8LinearConfig.from_recipe_name("mxfp8"),
                                   module_filter_fn=default_fp8_filter)
        dtype = "mxfp8 (block-scaled e4m3/e5m2 linears on tcgen05 block_scale MMAs, bf16 elsewhere)"
    from nanochat_b200.train import TrainStep
    B, T = args.device_batch_size, args.seq_len
    assert args.total_batch_size % (B * T * world) == 0
    accum = args.total_batch_size // (B * T * world)
    # the object the training scripts drive (scripts/base_train.py, chat_sft.py, chat_rl.py): arena, collectives, step
    trainer = TrainStep(model, grad_accum=accum, comm=args.comm if world > 1 else None, matrix_lr=0.02, weight_decay=0.1,
                        log=lambda m: print(f"[bench] {m}", file=sys.stderr))
    comm_name = trainer.comm_name or "none (1 GPU)"
    flops_per_token = model.estimate_flops()

    gen = torch.Generator(device="cpu").manual_seed(1234 + rank)
    n_buf = min(accum, 8)
    host = [torch.randint(0, cfg.vocab_size, (2, B, T), generator=gen, dtype=torch.long).pin_memory()
            for _ in range(n_buf)]
    dev = [h.to(device) for h in host]
    staging = [torch.empty_like(dev[0]) for _ in range(2)]

    loss_log = []                     # device scalars; read back after the timed regions

    def step_device():
        loss_log.append(trainer.step(lambda i: (dev[i % n_buf][0], dev[i % n_buf][1])))

    last_loss = [None]

    def step_e2e():
        def fetch(i):
            buf = staging[i % 2]
            buf.copy_(host[i % n_buf], non_blocking=True)   # H2D from pinned memory, every micro-step
            return buf[0], buf[1]
        loss = trainer.step(fetch)
        last_loss[0] = loss.item()                           # D2H read of the step's loss
        loss_log.append(last_loss[0])

    for _ in range(args.warmup):
        step_device()
    nat = ops.native_module()
    nat.check_status()
    launches0 = nat.launch_count()
    trainer.timers.collect()               # NANOCHAT_TRACE=1: drop the warm-up intervals
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms = timed_region(torch, dist, world, args.steps, step_device)
    clocks = sampler.stop()
    # device time per phase and step (max over ranks); empty unless NANOCHAT_TRACE=1
    phases = {k: v / args.steps for k, v in trainer.timers.collect().items()}
    launches = nat.launch_count() - launches0
    nat.check_status()

    e2e = None
    if not args.no_e2e:
        step_e2e()
        e2e_ms = timed_region(torch, dist, world, args.steps, step_e2e)
        e2e = {"value": args.total_batch_size * args.steps / (e2e_ms / 1e3), "unit": "tokens/s",
               "ms_per_step": e2e_ms / args.steps,
               "h2d_bytes_per_step": accum * 2 * B * T * 8, "d2h_bytes_per_step": 4,
               "last_loss": last_loss[0]}
    # The optimizer step on its own (sharded Muon + AdamW with its gradient reduction and parameter write-back),
    # against the roofline of that step: the slower of its Newton-Schulz FLOPs at the measured GEMM rate and
    # its bytes over NVLink at the measured per-direction peer bandwidth.
    opt = None
    if world > 1:
        # two more real steps with an event pair around the update: what the update costs once the gradient
        # pushes have ridden on the backward pass (a bare optimizer.step() loop would pay them in the open)
        trainer.optimizer_events = []
        fused = trainer.comm is not None and hasattr(trainer.comm, "update_ms")
        if fused:
            trainer.comm.time_updates = True
        own = []
        for _ in range(2):
            step_device()
            if fused:
                own.append(trainer.comm.update_ms())
        torch.cuda.synchronize()
        outer = sum(a.elapsed_time(b) for a, b in trainer.optimizer_events) / len(trainer.optimizer_events)
        # `ms`: the update itself, from the moment every rank has arrived at it (fused path; the NCCL path has no
        # such mark and reports the whole call); `ms_with_arrival_skew`: the whole call, i.e. plus the wait for the
        # slowest rank's backward pass
        t = torch.tensor([sum(own) / len(own) if own else outer, outer], device=device)
        trainer.optimizer_events = None
        if fused:
            trainer.comm.time_updates = False
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        n_all = sum(p.numel() for p in model.parameters())
        ns_flops = 0.0
        for p in model.transformer.h.parameters():
            if p.dim() == 2 and min(p.shape) >= 8:
                n, m = min(p.shape), max(p.shape)
                # X X^T and A A are symmetric: half of their 2 n^2 m and 2 n^3 FLOPs are needed; B X is not
                ns_flops += 5 * (1.0 * n * n * m + 1.0 * n ** 3 + 2.0 * n * n * m)
        bytes_in = (world - 1) / world * n_all * 4          # fp32 gradient slices arriving from the peers: pushed by
        #                                                     the last micro-batch's backward pass, outside the update
        bytes_out = (world - 1) / world * n_all * 2         # bf16 parameters stored to the peers by the update kernels
        link_ms = bytes_out / 770e9 * 1e3                   # measured peer copy: 770 GB/s per direction
        push_ms = bytes_in / 770e9 * 1e3
        flop_ms = ns_flops / world / 1405e12 * 1e3          # measured sustained bf16 GEMM rate
        breakdown = None
        if trainer.comm is not None and hasattr(trainer.comm, "trace_report") and trainer.comm.trace.enabled:
            mine = trainer.comm.trace_report()       # stages of the last step, this rank's device time
            keys = list(mine)
            vals = torch.tensor([mine[k] for k in keys], device=device)
            dist.all_reduce(vals, op=dist.ReduceOp.MAX)
            breakdown = {k: round(v, 3) for k, v in zip(keys, vals.tolist())}
        opt = {"ms": t[0].item(), "ms_with_arrival_skew": t[1].item(), "breakdown_ms_max_over_ranks": breakdown, "roofline_ms": max(link_ms, flop_ms), "link_ms": link_ms, "newton_schulz_ms": flop_ms,
               "gradient_push_link_ms_under_backward": push_ms,
               "fraction_of_roofline": max(link_ms, flop_ms) / t[0].item()}
    tok_s = args.total_batch_size * args.steps / (ms / 1e3)
    peak_mem = torch.cuda.max_memory_allocated() / 2**30
    out = {
        "metric": "d26 pretrain tokens/sec (whole job)", "value": tok_s, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": tok_s / PUBLISHED_TOK_PER_SEC, "dtype": dtype, "data": "synthetic",
        "impl": "ours",
        "config": shared_config(args, world, accum),
        "arm": {"optimizer": "MuonAdamW (ZeRO-2 sharded)", "optimizer_comm": comm_name, "attention": nat.ATTENTION_IMPL,
                "step": "nanochat_b200.train.TrainStep (the loop body of scripts/base_train.py)",
                "fp8_layer_passes": nat.stats["fp8_layer_forward"], "bf16_layer_passes": nat.stats["bf16_layer_forward"]},
        "losses": losses_of(loss_log, args),
        "mfu_bf16_nominal": flops_per_token * tok_s / (world * 2.25e15),
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "peak_mem_gib": peak_mem,
        "optimizer_step": opt,
    }
    if phases:
        out["phases_ms_per_step"] = phases
    common.compute_cleanup()
    if rank == 0:
        if world == 1 and not args.no_decode:
            del trainer, model, dev, staging, host
            import gc
            gc.collect()
            torch.cuda.empty_cache()
            out["decode"] = decode_sweep(args, "ours")
        print(json.dumps(out))


def run_reference(args):
    """The unmodified reference (baseline/_ref) through its own GPT / fp8 / MuonAdamW / torch.compile."""
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "nanochat")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/nanochat not present on this box"}))
        return
    sys.path.insert(0, ref_root)
    os.environ.setdefault("PYTORCH_ALLOC_CONF", "expandable_segments:True")
    try:
        import torch
        import torch.distributed as dist
        import torch.nn as nn
        from nanochat.common import compute_init, compute_cleanup
        from nanochat.gpt import GPT, GPTConfig
    except Exception as e:  # dependency missing on this box
        print(json.dumps({"impl": "reference", "unavailable": f"import failed: {type(e).__name__}: {e}"}))
        return
    rank, local_rank, world = dist_env()
    _, _, _, _, device = compute_init("cuda")
    dim = -(-args.depth * 64 // 128) * 128
    cfg = GPTConfig(sequence_len=args.seq_len, vocab_size=32768, n_layer=args.depth, n_head=dim // 128,
                    n_kv_head=dim // 128, n_embd=dim, window_pattern=args.window_pattern)
    with torch.device("meta"):
        model = GPT(cfg)
    model.to_empty(device=device)
    model.init_weights()
    dtype = "bf16"
    if not args.ref_bf16:
        from nanochat.fp8 import Float8LinearConfig, convert_to_float8_training

        def fp8_filter(mod, fqn):   # the filter of the reference's training script
            if not isinstance(mod, nn.Linear):
                return False
            if mod.in_features % 16 != 0 or mod.out_features % 16 != 0:
                return False
            return min(mod.in_features, mod.out_features) >= 128
        convert_to_float8_training(model, config=Float8LinearConfig.from_recipe_name("tensorwise"),
                                   module_filter_fn=fp8_filter)
        dtype = "fp8 (tensorwise e4m3/e5m2 linears, bf16 elsewhere)"
    orig_model = model
    compiled = not args.ref_eager
    if compiled:
        model = torch.compile(model, dynamic=False)
    optimizer = orig_model.setup_optimizer(weight_decay=0.1)
    B, T = args.device_batch_size, args.seq_len
    accum = args.total_batch_size // (B * T * world)
    gen = torch.Generator(device="cpu").manual_seed(1234 + rank)
    n_buf = min(accum, 8)
    host = [torch.randint(0, cfg.vocab_size, (2, B, T), generator=gen, dtype=torch.long).pin_memory()
            for _ in range(n_buf)]
    dev = [h.to(device) for h in host]
    staging = [torch.empty_like(dev[0]) for _ in range(2)]

    def train_step(fetch):
        for i in range(accum):
            x, y = fetch(i)
            loss = model(x, y)
            (loss / accum).backward()
        optimizer.step()
        model.zero_grad(set_to_none=True)
        return loss.detach()

    loss_log = []

    def step_device():
        loss_log.append(train_step(lambda i: (dev[i % n_buf][0], dev[i % n_buf][1])))

    last_loss = [None]

    def step_e2e():
        def fetch(i):
            buf = staging[i % 2]
            buf.copy_(host[i % n_buf], non_blocking=True)
            return buf[0], buf[1]
        last_loss[0] = train_step(fetch).item()
        loss_log.append(last_loss[0])

    try:
        for _ in range(args.warmup):
            step_device()
    except Exception as e:
        if not compiled:
            raise
        # Inductor unavailable on this box: fall back to the reference's eager path and say so
        print(f"[bench] torch.compile failed ({type(e).__name__}); running the reference eagerly", file=sys.stderr)
        os.environ["TORCHDYNAMO_DISABLE"] = "1"
        import torch._dynamo
        torch._dynamo.reset()
        torch._dynamo.config.disable = True
        model = orig_model
        compiled = False
        model.zero_grad(set_to_none=True)
        del loss_log[:]
        for _ in range(args.warmup):
            step_device()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms = timed_region(torch, dist, world, args.steps, step_device)
    clocks = sampler.stop()
    e2e = None
    if not args.no_e2e:
        step_e2e()
        e2e_ms = timed_region(torch, dist, world, args.steps, step_e2e)
        e2e = {"value": args.total_batch_size * args.steps / (e2e_ms / 1e3), "unit": "tokens/s",
               "ms_per_step": e2e_ms / args.steps, "h2d_bytes_per_step": accum * 2 * B * T * 8,
               "d2h_bytes_per_step": 4, "last_loss": last_loss[0]}
    tok_s = args.total_batch_size * args.steps / (ms / 1e3)
    out = {
        "metric": "d26 pretrain tokens/sec (whole job)", "value": tok_s, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": tok_s / PUBLISHED_TOK_PER_SEC, "dtype": dtype, "data": "synthetic",
        "impl": "reference",
        "config": shared_config(args, world, accum),
        "arm": {"optimizer": "the reference's MuonAdamW / DistMuonAdamW", "optimizer_comm": "nccl" if world > 1 else "none (1 GPU)",
                "attention": "torch SDPA (the reference's path on a non-Hopper GPU)", "torch_compile": compiled},
        "losses": losses_of(loss_log, args),
        "mfu_bf16_nominal": orig_model.estimate_flops() * tok_s / (world * 2.25e15),
        "clocks": clocks, "e2e": e2e, "peak_mem_gib": torch.cuda.max_memory_allocated() / 2**30,
    }
    compute_cleanup()
    if rank == 0:
        if world == 1 and not args.no_decode:
            del model, orig_model, optimizer, dev, staging, host
            import gc
            gc.collect()
            torch.cuda.empty_cache()
            out["decode"] = decode_sweep(args, "reference")
        print(json.dumps(out))


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    else:
        if ROOT not in sys.path:
            sys.path.insert(0, ROOT)
        run_ours(a)
