"""
Inference benchmark: time to first token, time per output token, tokens/sec, memory-bandwidth
and compute utilisation over a sweep of decode batch sizes, through `Engine.generate`.

    python -m scripts.infer_bench -i base --batch-sizes 1,8,32,64
    python -m scripts.infer_bench --random-init --depth 26 --prompt-tokens 512 --decode-tokens 256 \
        --batch-sizes 1,8,32,64 -t 1.0 -k 50          # no checkpoint needed

TTFT is the first `next()` on the generator (batch-1 prefill + cache fork + first sample); TPOT
is the median later step; tok/s = batch x steps / total decode time; MBU = (weight bytes +
batch x KV bytes read at mid context) / TPOT / peak bandwidth; MFU analogous with decode FLOPs
(reference: scripts/infer_bench.py). The last stdout line is one JSON object with every number.
"""
import argparse
import json
import gc
import time

import torch

from nanochat_b200.common import (compute_init, compute_cleanup, autodetect_device_type, get_peak_bandwidth,
                                  get_peak_flops)
from nanochat_b200.engine import Engine


def weight_bytes(model):
    """Bytes a decode step has to read for the parameters, as they are consumed (bf16 shadows of the
    fp32 masters on the native path, the stored dtype otherwise)."""
    if hasattr(model, "transformer") and next(model.parameters()).is_cuda:
        # bf16 operand copies of the block matrices and lm_head; embedding tables are only touched by row
        dense = list(model.transformer.h.parameters()) + [model.lm_head.weight]
        return sum(p.numel() * 2 for p in dense)
    return sum(p.numel() * p.element_size() for p in model.parameters())


def bench_generate(engine, prompt_tokens, batch_size, decode_tokens, temperature, top_k=None):
    device = engine.model.get_device()
    # A cyclic collection landing inside a timed call reads as 0.1-0.5 s of TTFT or of one decode step (seen at batch 64,
    # where it halved the reported tokens/s): collect first, then keep the collector off for the timed generation.
    gc.collect()
    gc.disable()
    try:
        torch.cuda.reset_peak_memory_stats(device)
        torch.cuda.synchronize(device)
        gen = engine.generate(prompt_tokens, num_samples=batch_size, max_tokens=decode_tokens,
                              temperature=temperature, top_k=top_k)
        t0 = time.perf_counter()
        next(gen)
        torch.cuda.synchronize(device)
        ttft = time.perf_counter() - t0
        steps = []
        while True:
            t0 = time.perf_counter()
            try:
                next(gen)
            except StopIteration:
                break
            torch.cuda.synchronize(device)
            steps.append(time.perf_counter() - t0)
    finally:
        gc.enable()
    return dict(ttft=ttft, step_times=steps, peak_vram=torch.cuda.max_memory_allocated(device))


def build_prompt(tokenizer, n):
    text = ("The history of science is the study of the development of science, including both the natural "
            "and social sciences. Science is a body of empirical, theoretical, and practical knowledge about "
            "the natural world. ") * max(1, n // 10)
    ids = tokenizer.encode(text, prepend="<|bos|>")
    assert len(ids) >= n, "prompt text too short"
    return ids[:n]


class _SyntheticTokenizer:
    """Stands in for a trained tokenizer when benchmarking random-init weights: ids are what matter."""

    def __init__(self, vocab_size):
        self.vocab_size = vocab_size
        self._special = {"<|bos|>": vocab_size - 9, "<|python_start|>": vocab_size - 4,
                         "<|python_end|>": vocab_size - 3, "<|output_start|>": vocab_size - 2,
                         "<|output_end|>": vocab_size - 1, "<|assistant_end|>": vocab_size - 5}

    def encode_special(self, s):
        return self._special[s]

    def get_bos_token_id(self):
        return self._special["<|bos|>"]

    def encode(self, text, prepend=None):
        ids = [(b * 131 + i * 7) % (self.vocab_size - 9) for i, b in enumerate(text.encode())]
        return ([self.encode_special(prepend)] if prepend else []) + ids

    def decode(self, ids):
        return ""


def run_reference(args):
    """Decode rate of the UNMODIFIED reference (baseline/_ref: its GPT, its Engine, stock code path) on random-init
    weights of --depth, with the same prompt length, batch sizes and timing as the sweep below."""
    import os
    import sys
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
    if not os.path.isdir(os.path.join(root, "nanochat")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/nanochat not present on this box"}))
        return
    sys.path.insert(0, root)
    for name in [m for m in sys.modules if m == "nanochat" or m.startswith("nanochat.")]:
        del sys.modules[name]
    try:
        import rustbpe  # noqa: F401
    except ImportError:
        # the reference's tokenizer module imports its BPE trainer at import time; decode never calls it
        import types
        sys.modules["rustbpe"] = types.ModuleType("rustbpe")
    from nanochat.common import compute_init as ref_init, compute_cleanup as ref_cleanup
    from nanochat.gpt import GPT, GPTConfig
    from nanochat.engine import Engine as RefEngine
    _, _, _, _, device = ref_init("cuda")
    dim = -(-args.depth * 64 // 128) * 128
    cfg = GPTConfig(sequence_len=2048, vocab_size=32768, n_layer=args.depth, n_head=dim // 128, n_kv_head=dim // 128,
                    n_embd=dim)
    with torch.device("meta"):
        model = GPT(cfg)
    model.to_empty(device=device)
    model.init_weights()
    model.eval()
    engine = RefEngine(model, _SyntheticTokenizer(cfg.vocab_size))
    g = torch.Generator().manual_seed(0)
    prompt_len = min(args.prompt_tokens, cfg.sequence_len - args.decode_tokens)
    prompt = torch.randint(0, cfg.vocab_size - 9, (prompt_len,), generator=g).tolist()
    payload = {"impl": "reference", "prompt_tokens": prompt_len, "decode_tokens": args.decode_tokens, "sweep": []}
    for bs in [int(b) for b in args.batch_sizes.split(",")]:
        bench_generate(engine, prompt, bs, 8, args.temperature, args.top_k)
        res = bench_generate(engine, prompt, bs, args.decode_tokens, args.temperature, args.top_k)
        st = res["step_times"]
        if not st:
            continue
        tpot = sorted(st)[len(st) // 2]
        payload["sweep"].append({"batch_size": bs, "ttft_sec": round(res["ttft"], 6), "tpot_sec": round(tpot, 6),
                                 "tok_per_sec": round(bs * len(st) / sum(st), 1), "decode_steps": len(st)})
        print(f"reference batch {bs}: TPOT {tpot*1e3:.2f} ms, {payload['sweep'][-1]['tok_per_sec']:,.0f} tok/s")
    print(json.dumps(payload))
    ref_cleanup()


def main():
    ap = argparse.ArgumentParser(description="Inference benchmark")
    ap.add_argument("--impl", type=str, default="ours", choices=["ours", "reference"],
                    help="reference = the unmodified reference engine from baseline/_ref (random-init only)")
    ap.add_argument("-i", "--source", type=str, default="base")
    ap.add_argument("-g", "--model-tag", type=str, default=None)
    ap.add_argument("-s", "--step", type=int, default=None)
    ap.add_argument("--prompt-tokens", type=int, default=2048)
    ap.add_argument("--decode-tokens", type=int, default=256)
    ap.add_argument("--batch-sizes", type=str, default="1,8,32,128")
    ap.add_argument("-t", "--temperature", type=float, default=0.0)
    ap.add_argument("-k", "--top-k", type=int, default=None)
    ap.add_argument("--random-init", action="store_true", help="random weights of --depth instead of a checkpoint")
    ap.add_argument("--depth", type=int, default=26)
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    device_type = autodetect_device_type()
    assert device_type == "cuda", "infer_bench needs a CUDA GPU"
    _, _, _, world, device = compute_init(device_type)
    assert world == 1, "infer_bench is a single GPU benchmark, run without torchrun"
    if args.random_init:
        from nanochat_b200.models.gpt import GPT, GPTConfig
        from nanochat_b200.schedules import model_dims
        dim, heads = model_dims(args.depth)
        cfg = GPTConfig(sequence_len=2048, vocab_size=32768, n_layer=args.depth, n_head=heads, n_kv_head=heads,
                        n_embd=dim)
        with torch.device("meta"):
            model = GPT(cfg)
        model.to_empty(device=device)
        model.init_weights()
        model.eval()
        tokenizer = _SyntheticTokenizer(cfg.vocab_size)
        meta = {"step": 0, "model_config": vars(cfg).copy()}
        g = torch.Generator().manual_seed(0)
        prompt_source = lambda n: torch.randint(0, cfg.vocab_size - 9, (n,), generator=g).tolist()
    else:
        from nanochat_b200.checkpoint_manager import load_model
        model, tokenizer, meta = load_model(args.source, device, phase="eval", model_tag=args.model_tag,
                                            step=args.step)
        prompt_source = lambda n: build_prompt(tokenizer, n)
    cfg = model.config
    engine = Engine(model, tokenizer)
    prompt_len = min(args.prompt_tokens, cfg.sequence_len - args.decode_tokens)
    if prompt_len < args.prompt_tokens:
        print(f"note: clamping prompt to {prompt_len} tokens so prompt+decode fits sequence_len={cfg.sequence_len}")
    prompt = prompt_source(prompt_len)

    name = torch.cuda.get_device_name(device)
    peak_bw, peak_flops = get_peak_bandwidth(name), get_peak_flops(name)
    vram = torch.cuda.get_device_properties(device).total_memory
    w_bytes = weight_bytes(model)
    n_params = sum(p.numel() for p in model.parameters())
    kv_store = model.kv_bytes_per_token()
    ctx_mid = prompt_len + args.decode_tokens // 2
    kv_read = model.kv_read_bytes(ctx_mid)
    ceiling = peak_bw / (w_bytes + kv_read)
    max_rows = int((vram - w_bytes) / (kv_store * cfg.sequence_len))
    print("=" * 100)
    print(f"Model: {args.source} (step {meta['step']}) | depth {cfg.n_layer}, dim {cfg.n_embd}, heads {cfg.n_head}, "
          f"kv heads {cfg.n_kv_head}")
    print(f"GPU: {name} | peak bandwidth {peak_bw/1e12:.2f} TB/s | peak compute {peak_flops/1e12:.0f} TFLOPS | "
          f"VRAM {vram/2**30:.0f} GiB")
    print(f"Parameters: {n_params:,} | weight bytes as stored: {w_bytes/2**20:.0f} MiB")
    print(f"KV cache: {kv_store:,} bytes/token stored | {kv_read:,} bytes read/step at context {ctx_mid} "
          f"(window pattern {cfg.window_pattern})")
    print(f"Theoretical decode ceiling at batch 1: {ceiling:,.0f} tok/s | max ~{max_rows:,} full-context rows in VRAM")
    print("=" * 100)
    finite = lambda v: v if v != float("inf") else None
    payload = {"source": args.source, "step": meta["step"], "model_config": meta["model_config"], "gpu": name,
               "peak_bandwidth_bytes_per_sec": finite(peak_bw), "peak_flops_per_sec": finite(peak_flops),
               "total_vram_bytes": vram, "num_params": n_params, "weight_bytes": w_bytes,
               "kv_bytes_per_token": kv_store, "kv_read_bytes_per_step": kv_read, "context_mid": ctx_mid,
               "decode_flops_per_token": model.estimate_decode_flops(ctx_mid),
               "ceiling_bs1_tok_per_sec": finite(round(ceiling, 1)), "max_full_context_rows": max_rows,
               "prompt_tokens": prompt_len, "decode_tokens": args.decode_tokens, "temperature": args.temperature,
               "top_k": args.top_k, "sweep": []}

    bench_generate(engine, prompt, 1, 2, args.temperature, args.top_k)
    pre = bench_generate(engine, prompt, 1, 2, args.temperature, args.top_k)
    pre_mfu = 100 * model.estimate_prefill_flops(prompt_len) / pre["ttft"] / peak_flops
    print(f"Prefill (batch 1, {prompt_len} tokens): {prompt_len / pre['ttft']:,.0f} tok/s | MFU {pre_mfu:.1f}%")
    payload["prefill"] = {"tok_per_sec": round(prompt_len / pre["ttft"], 1), "mfu_percent": round(pre_mfu, 2),
                          "time_sec": round(pre["ttft"], 6)}

    header = f"{'batch':>6} {'TTFT ms':>9} {'TPOT ms':>9} {'tok/s':>10} {'MBU %':>7} {'MFU %':>7} {'VRAM GiB':>9} {'steps':>6}"
    print(header + "\n" + "-" * len(header))
    for bs in [int(b) for b in args.batch_sizes.split(",")]:
        bench_generate(engine, prompt, bs, 8, args.temperature, args.top_k)
        res = bench_generate(engine, prompt, bs, args.decode_tokens, args.temperature, args.top_k)
        st = res["step_times"]
        if not st:
            print(f"{bs:>6}  all rows terminated immediately, skipping")
            continue
        tpot = sorted(st)[len(st) // 2]
        tok_s = bs * len(st) / sum(st)
        mbu = 100 * ((w_bytes + bs * kv_read) / tpot) / peak_bw
        mfu = 100 * (bs * model.estimate_decode_flops(ctx_mid) / tpot) / peak_flops
        print(f"{bs:>6} {res['ttft']*1e3:>9.1f} {tpot*1e3:>9.2f} {tok_s:>10,.0f} {mbu:>7.1f} {mfu:>7.2f} "
              f"{res['peak_vram']/2**30:>9.2f} {len(st):>6}")
        payload["sweep"].append({"batch_size": bs, "ttft_sec": round(res["ttft"], 6), "tpot_sec": round(tpot, 6),
                                 "tok_per_sec": round(tok_s, 1), "mbu_percent": round(mbu, 2),
                                 "mfu_percent": round(mfu, 4), "peak_vram_bytes": res["peak_vram"],
                                 "decode_steps": len(st)})
    print("-" * len(header))
    print(json.dumps(payload))
    compute_cleanup()


if __name__ == "__main__":
    main()
