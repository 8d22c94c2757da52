"""Runs the UNMODIFIED reference implementation (eager, fp32, CPU) for the parity tests.
usage: _ref_worker.py <ref_root> <mode> <path>"""
import os
import sys

os.environ["TORCHDYNAMO_DISABLE"] = "1"
os.environ["NANOCHAT_DTYPE"] = "float32"
ref_root, mode, path = sys.argv[1], sys.argv[2], sys.argv[3]
sys.path.insert(0, ref_root)

import torch                                      # noqa: E402
from nanochat.gpt import GPT, GPTConfig          # noqa: E402

cfg = GPTConfig(sequence_len=128, vocab_size=1024, n_layer=4, n_head=2, n_kv_head=2, n_embd=256)
torch.manual_seed(42)
with torch.device("meta"):
    model = GPT(cfg)
model.to_empty(device="cpu")
model.init_weights()
opt = model.setup_optimizer(weight_decay=0.1)
if mode == "load":      # continue from a checkpoint written by this repository
    blob = torch.load(path)
    model.load_state_dict(blob["model"], strict=True, assign=True)
    opt = model.setup_optimizer(weight_decay=0.1)
    opt.load_state_dict(blob["optim"])
g = torch.Generator().manual_seed(0)
losses = []
for step in range(4):
    x = torch.randint(0, 1024, (4, 128), generator=g)
    y = torch.randint(0, 1024, (4, 128), generator=g)
    loss = model(x, y)
    loss.backward()
    opt.step()
    model.zero_grad(set_to_none=True)
    losses.append(loss.item())
out = path if mode == "train" else path + ".out"
torch.save({"losses": losses, "model": model.state_dict(), "optim": opt.state_dict()}, out)
