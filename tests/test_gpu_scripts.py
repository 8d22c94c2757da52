"""
The shipped entry points on a B200, through their command lines: the pretraining driver must run the
measured path (parameter arena, fused QKV, fp8 layer kernels, and with two ranks the fused peer-to-peer
optimizer), its loss must fall, its checkpoints must hold current weights on every back end, and a resumed
run must continue. The SFT driver is launched the same way on synthetic conversations.
"""
import os
import re
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

B, T, VOCAB, DEPTH = 4, 512, 4096, 4


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _launch(module, args, base_dir, world=1, extra_env=None, timeout=900):
    env = dict(os.environ, NANOCHAT_BASE_DIR=str(base_dir), OMP_NUM_THREADS="2", NCCL_NVLS_ENABLE="0")
    env.update(extra_env or {})
    if world == 1:
        cmd = [sys.executable, "-m", module, *args]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), "-m", module, *args]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, (r.stdout[-3000:], r.stderr[-3000:])
    dump = os.environ.get("NANOCHAT_TEST_DUMP_DIR", "")
    if dump and os.path.isdir(dump):
        with open(os.path.join(dump, f"{module.split('.')[-1]}_world{world}.log"), "a") as f:
            f.write(" ".join(cmd) + "\n" + r.stdout + "\n")
    return r.stdout


def _train_args(iters, tag, world, extra=()):
    # one fixed batch repeated (--synthetic-cycle 1) so a few steps are enough for the loss to fall
    return ["--synthetic-data", f"--depth={DEPTH}", "--fp8", f"--num-iterations={iters}", "--save-every=2",
            f"--device-batch-size={B}", f"--max-seq-len={T}", f"--total-batch-size={B * T * 2 * world}",
            f"--vocab-size={VOCAB}", "--eval-every=2", "--core-metric-every=-1", "--sample-every=-1",
            "--warmup-steps=0", "--synthetic-cycle=1", f"--model-tag={tag}", "--log-every=1", *extra]


def _step_losses(out):
    return [float(m) for m in re.findall(r"^step \d+/\d+ .*?\| loss: ([0-9.]+)", out, flags=re.M)]


def _val_losses(out):
    return {int(s): float(v) for s, v in re.findall(r"^Step (\d+) \| Validation loss: ([0-9.]+)", out, flags=re.M)}


def _path_counts(out):
    m = re.search(r"fp8 layer passes: ([\d,]+) \| bf16 layer passes: ([\d,]+) \| fused QKV: ([\d,]+)", out)
    assert m, out[-2000:]
    return tuple(int(g.replace(",", "")) for g in m.groups())


def _reload_and_eval(base_dir, tag, step, world):
    """The saved model on ONE rank, evaluated on the batches the `world` ranks of the run evaluated."""
    from nanochat_b200.checkpoint_manager import load_checkpoint
    from nanochat_b200.dataloader import synthetic_token_loader
    from nanochat_b200.models.gpt import GPT, GPTConfig
    ckpt = os.path.join(str(base_dir), "base_checkpoints", tag)
    model_data, _, meta = load_checkpoint(ckpt, step, torch.device("cuda"))
    with torch.device("meta"):
        model = GPT(GPTConfig(**meta["model_config"]))
    model.to_empty(device="cuda")
    model.init_weights()
    model.load_state_dict(model_data, strict=True, assign=True)
    model.eval()
    total, count = 0.0, 0
    with torch.no_grad():
        for r in range(world):
            gen = synthetic_token_loader(B, T, VOCAB, device="cuda", seed=r, cycle=1)   # rank r of the run drew these
            for _ in range(4):
                x, y, _ = next(gen)
                loss = model(x, y, loss_reduction="none")
                total += loss.double().sum().item()
                count += loss.numel()
    return total / count


@pytest.mark.parametrize("world", [1, 2])
def test_base_train_script_runs_the_fp8_arena_path_and_saves_current_weights(world, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    tag = f"script_w{world}"
    out = _launch("scripts.base_train", _train_args(6, tag, world), tmp_path, world)
    losses = _step_losses(out)
    assert len(losses) >= 6, out[-2000:]
    assert losses[-1] < losses[0] - 0.5, losses
    fp8_passes, bf16_passes, fused_qkv = _path_counts(out)
    micro_steps = 6 * 2
    assert fp8_passes >= micro_steps * DEPTH, (fp8_passes, bf16_passes)      # training layers ran the fp8 kernels
    assert fused_qkv >= fp8_passes                                           # one QKV GEMM per layer pass
    if world > 1:
        assert "fused peer-to-peer kernels" in out, out[-2000:]
    vals = _val_losses(out)
    assert 6 in vals and 0 in vals, vals
    for step in (2, 4, 6):
        assert os.path.exists(os.path.join(str(tmp_path), "base_checkpoints", tag, f"model_{step:06d}.pt"))
    # every rank's optimizer shard and the full model were written; the model reproduces the run's own evaluation
    for r in range(world):
        assert os.path.exists(os.path.join(str(tmp_path), "base_checkpoints", tag, f"optim_000006_rank{r}.pt"))
    reloaded = _reload_and_eval(tmp_path, tag, 6, world)
    assert abs(reloaded - vals[6]) < 5e-3 * max(1.0, vals[6]), (reloaded, vals[6])
    # ... which it would not with stale (initial) weights: the evaluated loss fell a long way since step 0
    assert vals[6] < vals[0] - 0.5, vals

    # resume from step 4: same horizon, the loss carries on from where it was, not from scratch
    out2 = _launch("scripts.base_train", _train_args(6, tag, world, ["--resume-from-step=4"]), tmp_path, world)
    vals2 = _val_losses(out2)
    assert 4 in vals2 and abs(vals2[4] - vals[4]) < 5e-3 * max(1.0, vals[4]), (vals2, vals)
    assert abs(vals2[6] - vals[6]) < 5e-2 * max(1.0, vals[6]), (vals2, vals)


def test_base_train_fused_and_nccl_collectives_agree(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    outs = {}
    for comm in ("fused", "nccl"):
        outs[comm] = _launch("scripts.base_train", _train_args(4, f"cmp_{comm}", 2, [f"--comm={comm}"]), tmp_path, 2)
    a, b = _step_losses(outs["fused"]), _step_losses(outs["nccl"])
    assert len(a) == len(b) >= 4
    for x, y in zip(a, b):
        assert abs(x - y) < 5e-2 * max(1.0, y), (a, b)
    va, vb = _val_losses(outs["fused"]), _val_losses(outs["nccl"])
    assert abs(va[4] - vb[4]) < 5e-2 * max(1.0, vb[4]), (va, vb)


@pytest.mark.parametrize("world", [1, 2])
def test_chat_sft_script_on_synthetic_conversations(world, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    # --num-iterations counts micro-batches, as in the reference: 8 of them at 2 per step are 4 optimizer steps
    args = ["--synthetic-data", f"--depth={DEPTH}", "--num-iterations=8", f"--device-batch-size={B}",
            f"--max-seq-len={T}", f"--total-batch-size={B * T * 2 * world}", "--eval-every=-1", "--chatcore-every=-1"]
    out = _launch("scripts.chat_sft", args, tmp_path, world)
    steps = re.findall(r"^step (\d+) .*?\| loss: ([0-9.]+)", out, flags=re.M)
    assert len(steps) >= 3, out[-2000:]
    assert all(float(v) == float(v) and float(v) < 20 for _, v in steps), steps
    if world > 1:
        assert "fused peer-to-peer kernels" in out, out[-2000:]
