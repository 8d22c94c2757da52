"""
CPU tests of the training-side plumbing: checkpoint files (round trip, per-rank optimizer shards, truncated
files, back-compat patches), depth-derived hyper-parameters and schedules, bits-per-byte evaluation, the SFT
packer's row rules and the fp8 module swapper.
"""
import json
import math
import os

import pytest
import torch
import torch.nn as nn

from nanochat_b200 import checkpoint_manager as cm
from nanochat_b200 import schedules
from nanochat_b200.loss_eval import evaluate_bpb
from nanochat_b200.sft_data import sft_batches


# ------------------------------------------------------------------------------ checkpoints

def test_checkpoint_round_trip_and_layout(tmp_path):
    d = str(tmp_path / "ck")
    model = {"w": torch.arange(6.0).view(2, 3), "b": torch.ones(3, dtype=torch.bfloat16)}
    meta = {"step": 7, "model_config": {"n_layer": 2}, "val_bpb": 0.9}
    cm.save_checkpoint(d, 7, model, {"state": {"0": torch.zeros(2)}}, meta, rank=0)
    cm.save_checkpoint(d, 7, None, {"state": {"0": torch.ones(2)}}, None, rank=1)      # other ranks: optimizer only
    assert sorted(os.listdir(d)) == ["meta_000007.json", "model_000007.pt", "optim_000007_rank0.pt",
                                     "optim_000007_rank1.pt"]
    m, o, md = cm.load_checkpoint(d, 7, "cpu", load_optimizer=True, rank=1)
    assert torch.equal(m["w"], model["w"]) and m["b"].dtype == torch.bfloat16
    assert torch.equal(o["state"]["0"], torch.ones(2)) and md == meta
    assert cm.find_last_step(d) == 7
    cm.save_checkpoint(d, 12, model, None, meta)
    assert cm.find_last_step(d) == 12


def test_truncated_or_missing_checkpoint_files_raise_checkpoint_error(tmp_path):
    d = str(tmp_path / "ck")
    cm.save_checkpoint(d, 3, {"w": torch.randn(64, 64)}, None, {"model_config": {}})
    path = os.path.join(d, "model_000003.pt")
    blob = open(path, "rb").read()
    with open(path, "wb") as f:
        f.write(blob[: len(blob) // 2])                          # a writer that died half way
    with pytest.raises(cm.CheckpointError, match="unreadable"):
        cm.load_checkpoint(d, 3, "cpu")
    with pytest.raises(cm.CheckpointError, match="missing"):
        cm.load_checkpoint(d, 4, "cpu")
    with open(path, "wb") as f:
        f.write(blob)
    os.remove(os.path.join(d, "meta_000003.json"))
    with pytest.raises(cm.CheckpointError, match="missing"):
        cm.load_checkpoint(d, 3, "cpu")
    assert not [f for f in os.listdir(d) if f.endswith(".tmp")]     # saves are atomic: no temp files left behind
    # optimizer shards: a resume on more ranks than the run that saved has no shard for the new rank; a torn one is unreadable
    cm.save_checkpoint(d, 5, {"w": torch.randn(4)}, {"state": {"0": torch.zeros(2)}}, {"model_config": {}}, rank=0)
    with pytest.raises(cm.CheckpointError, match="missing"):
        cm.load_checkpoint(d, 5, "cpu", load_optimizer=True, rank=1)
    shard = os.path.join(d, "optim_000005_rank0.pt")
    with open(shard, "r+b") as f:
        f.truncate(os.path.getsize(shard) // 3)
    with pytest.raises(cm.CheckpointError, match="unreadable"):
        cm.load_checkpoint(d, 5, "cpu", load_optimizer=True, rank=0)
    assert cm.load_checkpoint(d, 5, "cpu", load_optimizer=False)[1] is None      # the model alone still loads


def test_largest_model_tag_is_the_deepest(tmp_path):
    for tag in ("d4", "d12", "d8"):
        os.makedirs(tmp_path / tag)
    assert cm.find_largest_model(str(tmp_path)) == "d12"


# ---------------------------------------------------------------- depth-derived hyper-parameters

@pytest.mark.parametrize("depth,dim,heads", [(4, 256, 2), (12, 768, 6), (20, 1280, 10), (24, 1536, 12),
                                             (26, 1664, 13), (32, 2048, 16)])
def test_model_dims_from_depth(depth, dim, heads):
    assert schedules.model_dims(depth) == (dim, heads)


def test_derived_batch_size_lr_scale_and_weight_decay():
    ref = 1.0e8
    same = schedules.derive_hparams(ref, ref, ratio=10.0, weight_decay=0.2)
    assert same.total_batch_size == schedules.B_REF and same.batch_lr_scale == 1.0
    assert math.isclose(same.weight_decay, 0.2)
    big = schedules.derive_hparams(8 * ref, ref, ratio=10.0, weight_decay=0.2)
    assert big.total_batch_size == 2 ** round(math.log2(schedules.B_REF * 8 ** 0.383))     # power of two
    assert math.isclose(big.batch_lr_scale, math.sqrt(big.total_batch_size / schedules.B_REF))
    assert math.isclose(big.weight_decay, 0.2 * math.sqrt(big.total_batch_size / schedules.B_REF) / 8)
    forced = schedules.derive_hparams(8 * ref, ref, ratio=10.0, weight_decay=0.2, total_batch_size=2 ** 20)
    assert forced.total_batch_size == 2 ** 20 and forced.target_tokens == int(10.0 * 8 * ref)


def test_pretraining_schedules_have_the_reference_shape():
    n = 1000
    lr = [schedules.pretrain_lr_multiplier(i, n) for i in range(n + 1)]
    assert math.isclose(lr[0], 1 / 40) and math.isclose(lr[39], 1.0) and lr[200] == 1.0
    assert lr[350] == 1.0 and lr[351] < 1.0                     # warm-down covers the last 65 %
    assert all(a >= b for a, b in zip(lr[351:], lr[352:]))
    assert math.isclose(lr[n], 0.05)
    n2 = 2000                                                   # warm-down starts at 700, after the 400-step ramp
    mom = [schedules.pretrain_muon_momentum(i, n2) for i in range(n2 + 1)]
    assert math.isclose(mom[0], 0.85) and math.isclose(mom[400], 0.97) and mom[699] == 0.97
    assert math.isclose(mom[n2], 0.90) and all(a >= b for a, b in zip(mom[700:], mom[701:]))
    assert math.isclose(schedules.pretrain_weight_decay(0, n, 0.3), 0.3)
    assert abs(schedules.pretrain_weight_decay(n, n, 0.3)) < 1e-12
    assert schedules.sft_lr_multiplier(0.25) == 1.0 and math.isclose(schedules.sft_lr_multiplier(0.75), 0.5)
    assert math.isclose(schedules.sft_muon_momentum(150), 0.90) and schedules.sft_muon_momentum(900) == 0.95


# ------------------------------------------------------------------------------ bits per byte

class _FixedLossModel:
    """Returns a given per-token loss table; records what it was asked."""

    def __init__(self, loss):
        self.loss = loss

    def get_device(self):
        return torch.device("cpu")

    def __call__(self, x, y, loss_reduction="mean"):
        assert loss_reduction == "none"
        return self.loss[: y.numel()].clone()


def test_bits_per_byte_skips_special_and_ignored_targets():
    token_bytes = torch.tensor([1, 2, 0, 4], dtype=torch.int64)            # token 2 is a special token
    y = torch.tensor([[0, 1, 2, -1, 3]])
    loss = torch.tensor([0.5, 1.0, 9.0, 7.0, 2.0])
    bpb = evaluate_bpb(_FixedLossModel(loss), [(torch.zeros_like(y), y)], 1, token_bytes)
    assert math.isclose(bpb, (0.5 + 1.0 + 2.0) / (math.log(2) * (1 + 2 + 4)), rel_tol=1e-6)
    only_special = torch.tensor([[2, 2, -1]])
    assert evaluate_bpb(_FixedLossModel(loss), [(only_special, only_special)], 1, token_bytes) == float("inf")


# ---------------------------------------------------------------------------------- SFT packer

def test_sft_rows_are_padded_never_cropped_and_masked_by_target():
    BOS = 99
    convs = [list(range(1, 1 + n)) for n in (5, 3, 9, 4, 2, 7)]

    def render(ids):
        # odd tokens are "assistant" tokens (mask 1), even ones are prompt tokens (mask 0)
        return [BOS] + ids, [0] + [t % 2 for t in ids]

    gen = sft_batches(convs, render, BOS, B=2, T=10, buffer_size=3)
    x, y = next(gen)
    assert x.shape == (2, 10) and y.shape == (2, 10) and x.dtype == torch.int32 and y.dtype == torch.int64
    for row in range(2):
        starts = [i for i, t in enumerate(x[row].tolist()) if t == BOS]
        assert starts and starts[0] == 0                            # every row starts a conversation
        # targets are the next token where its mask is 1, else -1; a padded tail is all BOS with targets -1
        for i in range(10):
            t = y[row, i].item()
            assert t == -1 or (t % 2 == 1 and t != BOS)
    # no conversation is split: every maximal run between BOS tokens is one whole rendered conversation
    rendered = {tuple(render(c)[0]) for c in convs}
    for row in range(2):
        ids = x[row].tolist()
        # the row holds T+1 tokens of which the last has no input slot; re-attach it from the targets' view
        pieces, cur = [], []
        for t in ids:
            if t == BOS and cur:
                pieces.append(tuple(cur))
                cur = []
            cur.append(t)
        for piece in pieces:                                        # complete pieces only (the last may be cut by T)
            assert piece in rendered or set(piece) == {BOS}


# --------------------------------------------------------------------------------- fp8 swapper

def test_fp8_conversion_filter_and_disable_context():
    from nanochat_b200.fp8 import Float8Linear, convert_to_float8_training, default_fp8_filter, fp8_disabled
    torch.manual_seed(0)
    net = nn.Sequential(nn.Linear(256, 512, bias=False), nn.ReLU(), nn.Linear(512, 24, bias=False),
                        nn.Linear(24, 130, bias=False))
    w0 = net[0].weight
    convert_to_float8_training(net, module_filter_fn=default_fp8_filter)
    assert isinstance(net[0], Float8Linear) and net[0].weight is w0           # same parameter object
    assert not isinstance(net[2], Float8Linear)                               # 24 outputs: too small / not /16
    assert not isinstance(net[3], Float8Linear)
    x = torch.randn(8, 256)
    with fp8_disabled(net):
        exact = net(x)
        assert not net[0].fp8_enabled
    assert net[0].fp8_enabled
    ref = nn.functional.linear(nn.functional.relu(nn.functional.linear(x, w0)), net[2].weight)
    ref = nn.functional.linear(ref, net[3].weight)
    assert torch.allclose(exact, ref, atol=1e-5)
    json.dumps({"n_fp8": sum(isinstance(m, Float8Linear) for m in net.modules())})


def test_optimizer_shards_of_another_world_size_are_not_loaded(tmp_path, monkeypatch):
    monkeypatch.setenv("NANOCHAT_BASE_DIR", str(tmp_path))
    d = str(tmp_path / "base_checkpoints" / "d2")
    for rank in range(2):                                       # a two-rank run saved step 9
        cm.save_checkpoint(d, 9, {"w": torch.zeros(2)} if rank == 0 else None, {"state": {"0": torch.full((3,), float(rank))}},
                           {"model_config": {}} if rank == 0 else None, rank=rank)
    assert cm.optimizer_shard_count(d, 9) == 2 and cm.optimizer_shard_count(d, 8) == 0
    got = cm.load_optimizer_state("base", "cpu", rank=1, world_size=2)
    assert torch.equal(got["state"]["0"], torch.ones(3))
    for world in (1, 4):                                        # every rank of a run of another size gets None
        for rank in range(world):
            assert cm.load_optimizer_state("base", "cpu", rank=rank, world_size=world) is None
    assert cm.load_optimizer_state("base", "cpu", rank=0) is not None          # no world size given: as before
    assert cm.load_optimizer_state("base", "cpu", rank=5) is None
