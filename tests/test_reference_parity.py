"""Parity with the reference implementation run eagerly on CPU (skipped when no copy of it is present):
same seed -> same initial weights and loss trajectory; checkpoints (model + optimizer) load both ways."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CANDIDATES = [os.path.join(ROOT, "baseline", "_ref")] + (
    [os.environ["NANOCHAT_REFERENCE_DIR"]] if os.environ.get("NANOCHAT_REFERENCE_DIR") else [])
REF = next((c for c in CANDIDATES if os.path.isdir(os.path.join(c, "nanochat"))), None)
pytestmark = [pytest.mark.slow, pytest.mark.skipif(REF is None, reason="reference sources not available")]


def _run_ref(mode, path):
    r = subprocess.run([sys.executable, os.path.join(HERE, "_ref_worker.py"), REF, mode, path],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]


def _ours(blob=None):
    from nanochat_b200 import common
    from nanochat_b200.models.gpt import GPT, GPTConfig
    assert common.COMPUTE_DTYPE == torch.float32
    cfg = GPTConfig(sequence_len=128, vocab_size=1024, n_layer=4, n_head=2, n_kv_head=2, n_embd=256)
    torch.manual_seed(42)
    with torch.device("meta"):
        model = GPT(cfg)
    model.to_empty(device="cpu")
    model.init_weights()
    opt = model.setup_optimizer(weight_decay=0.1)
    if blob is not None:
        model.load_state_dict(blob["model"], strict=True, assign=True)
        opt = model.setup_optimizer(weight_decay=0.1)
        opt.load_state_dict(blob["optim"])
    g = torch.Generator().manual_seed(0)
    losses = []
    for _ in range(4):
        x = torch.randint(0, 1024, (4, 128), generator=g)
        y = torch.randint(0, 1024, (4, 128), generator=g)
        loss = model(x, y)
        loss.backward()
        opt.step()
        model.zero_grad(set_to_none=True)
        losses.append(loss.item())
    return losses, model, opt


def test_same_seed_same_trajectory_and_state_layout(tmp_path):
    path = str(tmp_path / "ref.pt")
    _run_ref("train", path)
    ref = torch.load(path)
    losses, model, opt = _ours()
    assert ref["losses"] == pytest.approx(losses, rel=0, abs=2e-5)
    ours_sd = model.state_dict()
    assert list(ours_sd.keys()) == list(ref["model"].keys())
    for k in ours_sd:
        assert ours_sd[k].shape == ref["model"][k].shape and ours_sd[k].dtype == ref["model"][k].dtype, k
        diff = (ours_sd[k] - ref["model"][k]).abs()
        assert (diff > 1e-4).float().mean().item() < 1e-3, k
    ours_opt, ref_opt = opt.state_dict(), ref["optim"]
    assert sorted(ours_opt["state"].keys()) == sorted(ref_opt["state"].keys())
    for idx, st in ref_opt["state"].items():
        assert set(st.keys()) == set(ours_opt["state"][idx].keys())
        for name, val in st.items():
            if torch.is_tensor(val):
                assert ours_opt["state"][idx][name].shape == val.shape, (idx, name)
    for g_ref, g_ours in zip(ref_opt["param_groups"], ours_opt["param_groups"]):
        assert g_ref["kind"] == g_ours["kind"] and g_ref["params"] == g_ours["params"]
        assert g_ref["lr"] == pytest.approx(g_ours["lr"])


def test_checkpoints_load_in_both_directions(tmp_path):
    # ours -> reference
    _, model, opt = _ours()
    ckpt = str(tmp_path / "ours.pt")
    torch.save({"model": model.state_dict(), "optim": opt.state_dict()}, ckpt)
    _run_ref("load", ckpt)
    ref_cont = torch.load(ckpt + ".out")
    cont_losses, _, _ = _ours(torch.load(ckpt))
    assert ref_cont["losses"] == pytest.approx(cont_losses, rel=0, abs=5e-5)
    # reference -> ours
    path = str(tmp_path / "ref.pt")
    _run_ref("train", path)
    blob = torch.load(path)
    losses, _, _ = _ours(blob)
    assert all(l == l for l in losses)


def _cli_flags(path):
    import re
    out = set()
    with open(path, encoding="utf-8") as f:
        src = f.read()
    for m in re.finditer(r"add_argument\(([^)]*)", src):
        out |= set(re.findall(r"""["'](--?[a-zA-Z][a-zA-Z0-9-]*)["']""", m.group(1)))
    return out


@pytest.mark.parametrize("script", ["base_train", "base_eval", "chat_sft", "chat_rl", "chat_eval", "chat_cli", "tok_train",
                                    "infer_bench"])
def test_entry_points_accept_every_flag_of_the_reference(script):
    ref_path = os.path.join(REF, "scripts", script + ".py")
    if not os.path.exists(ref_path):
        pytest.skip("the reference copy carries no scripts")
    ref = _cli_flags(ref_path)
    ours = _cli_flags(os.path.join(ROOT, "scripts", script + ".py"))
    assert ref and not (ref - ours), sorted(ref - ours)


def _public_names(path):
    import ast
    with open(path, encoding="utf-8") as f:
        tree = ast.parse(f.read())
    out = set()
    for node in tree.body:
        if isinstance(node, (ast.FunctionDef, ast.ClassDef)):
            out.add(node.name)
        elif isinstance(node, ast.Assign):
            out |= {t.id for t in node.targets if isinstance(t, ast.Name)}
    return {n for n in out if not n.startswith("_")}


@pytest.mark.parametrize("ref_mod,our_mod", [
    ("nanochat/common.py", "nanochat_b200.common"), ("nanochat/gpt.py", "nanochat_b200.models.gpt"),
    ("nanochat/flash_attention.py", "nanochat_b200.flash_attention"), ("nanochat/fp8.py", "nanochat_b200.fp8"),
    ("nanochat/optim.py", "nanochat_b200.optim"), ("nanochat/engine.py", "nanochat_b200.engine"),
    ("nanochat/execution.py", "nanochat_b200.execution"), ("nanochat/tokenizer.py", "nanochat_b200.tokenizer"),
    ("nanochat/dataset.py", "nanochat_b200.dataset"), ("nanochat/dataloader.py", "nanochat_b200.dataloader"),
    ("nanochat/core_eval.py", "nanochat_b200.core_eval"), ("nanochat/loss_eval.py", "nanochat_b200.loss_eval"),
    ("nanochat/checkpoint_manager.py", "nanochat_b200.checkpoint_manager"), ("tasks/common.py", "tasks.common"),
    ("tasks/arc.py", "tasks.arc"), ("tasks/mmlu.py", "tasks.mmlu"), ("tasks/gsm8k.py", "tasks.gsm8k"),
    ("tasks/humaneval.py", "tasks.humaneval"), ("tasks/smoltalk.py", "tasks.smoltalk")])
def test_every_public_name_of_the_reference_exists_here(ref_mod, our_mod, tmp_path, monkeypatch):
    import importlib
    path = os.path.join(REF, ref_mod)
    if not os.path.exists(path):
        pytest.skip("module not in the reference copy")
    monkeypatch.setenv("NANOCHAT_BASE_DIR", str(tmp_path))          # names resolved on access may touch the base dir
    ours = importlib.import_module(our_mod)
    missing = sorted(n for n in _public_names(path) if not hasattr(ours, n))
    assert not missing, missing
