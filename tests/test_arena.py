"""Parameter arena: same training result as separately allocated parameters, zero-copy Muon stacks."""
import torch

from nanochat_b200.models.gpt import GPT, GPTConfig
from nanochat_b200.optim import _stack_view
from nanochat_b200.parallel.arena import ParamArena
from nanochat_b200.train import TrainStep


def _model():
    cfg = GPTConfig(sequence_len=64, vocab_size=512, n_layer=4, n_head=2, n_kv_head=2, n_embd=256)
    torch.manual_seed(7)
    m = GPT(cfg)
    m.init_weights()
    with torch.no_grad():
        for blk in m.transformer.h:
            blk.attn.c_proj.weight.normal_(0, 0.02)
            blk.mlp.c_proj.weight.normal_(0, 0.02)
    return m, cfg


def test_arena_training_matches_plain_and_stacks_are_views():
    plain, cfg = _model()
    housed, _ = _model()
    arena = ParamArena(housed)
    for g in arena.muon_groups:
        st = _stack_view([p.data for p in g["params"]])
        assert st is not None and st.data_ptr() == g["master"].data_ptr()
        gs = _stack_view([p.grad for p in g["params"]])
        assert gs is not None and gs.data_ptr() == g["grad"].data_ptr()
    blk = housed.transformer.h[0].attn
    assert blk.c_k.weight.data_ptr() == blk.c_q.weight.data_ptr() + blk.c_q.weight.numel() * 4
    assert blk.c_v.weight.data_ptr() == blk.c_k.weight.data_ptr() + blk.c_k.weight.numel() * 4
    a = TrainStep(plain, grad_accum=2, use_arena=False, weight_decay=0.1)
    b = TrainStep(housed, grad_accum=2, weight_decay=0.1, use_arena=True)
    gen = torch.Generator().manual_seed(0)
    for _ in range(3):
        data = [(torch.randint(0, 512, (2, 64), generator=gen), torch.randint(0, 512, (2, 64), generator=gen))
                for _ in range(2)]
        la = a.step(lambda i: data[i])
        lb = b.step(lambda i: data[i])
        assert abs(la.item() - lb.item()) < 1e-5
    for (n, p), (_, q) in zip(plain.named_parameters(), housed.named_parameters()):
        diff = (p - q).abs()
        assert (diff > 1e-4).float().mean().item() < 1e-3, n
    sd = housed.state_dict()
    assert sd["transformer.h.0.attn.c_q.weight"].shape == (256, 256)
