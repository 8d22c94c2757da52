"""Sharded-optimizer logic with zero GPUs: ownership map, loopback collectives, N-rank == 1-rank."""
import copy

import pytest
import torch

from nanochat_b200.optim import MuonAdamW
from nanochat_b200.parallel.comm import LoopbackWorld, NullComm
from nanochat_b200.parallel.ownership import adamw_shard, muon_shard, muon_owner


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_ownership_formulae(world):
    for rank in range(world):
        s = adamw_shard((32768, 16), rank, world)
        if world == 1:
            assert s.replicated
        else:
            per = 32768 // world
            assert not s.replicated and (s.row_start, s.row_end) == (rank * per, (rank + 1) * per)
        assert adamw_shard((26,), rank, world).replicated
        assert adamw_shard((1, 24), rank, world).replicated
        for K in (2, 13, 26, 104):
            m = muon_shard(K, rank, world)
            chunk = (K + world - 1) // world
            assert m.chunk == chunk and m.padded == chunk * world and m.start == rank * chunk
            assert m.num_owned == min(chunk, max(0, K - rank * chunk))
    for K in (13, 26, 104):
        owners = [muon_owner(j, K, world) for j in range(K)]
        assert owners == sorted(owners) and max(owners) < world
        assert sum(muon_shard(K, r, world).num_owned for r in range(world)) == K
    if world > 1:
        with pytest.raises(ValueError):
            adamw_shard((1001, 8), 0, world)


def _toy_params(seed):
    g = torch.Generator().manual_seed(seed)
    big = torch.nn.Parameter(torch.randn(64, 32, generator=g))            # adamw, sharded by rows
    small = torch.nn.Parameter(torch.randn(7, generator=g))               # adamw, replicated
    mats = [torch.nn.Parameter(torch.randn(16, 24, generator=g)) for _ in range(5)]   # muon, wide
    tall = [torch.nn.Parameter(torch.randn(24, 16, generator=g)) for _ in range(3)]   # muon, tall
    return big, small, mats, tall


def _make_opt(params, comm):
    big, small, mats, tall = params
    return MuonAdamW([
        dict(kind="adamw", params=[big], lr=0.01, betas=(0.8, 0.95), eps=1e-10, weight_decay=0.01),
        dict(kind="adamw", params=[small], lr=0.02, betas=(0.8, 0.95), eps=1e-10, weight_decay=0.0),
        dict(kind="muon", params=mats, lr=0.02, momentum=0.9, ns_steps=5, beta2=0.9, weight_decay=0.1),
        dict(kind="muon", params=tall, lr=0.02, momentum=0.9, ns_steps=5, beta2=0.9, weight_decay=0.1),
    ], comm=comm)


def _flat(params):
    big, small, mats, tall = params
    return [big, small, *mats, *tall]


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_steps_equal_single_rank_with_mean_gradient(world):
    steps = 3
    grads = [[[torch.randn_like(p) for p in _flat(_toy_params(0))] for _ in range(world)] for _ in range(steps)]
    # single rank on the rank-mean gradient
    ref = _toy_params(0)
    opt = _make_opt(ref, NullComm())
    for s in range(steps):
        for i, p in enumerate(_flat(ref)):
            p.grad = sum(grads[s][r][i] for r in range(world)) / world
        opt.step()
    lw = LoopbackWorld(world)

    def rank_body(comm):
        mine = _toy_params(0)
        o = _make_opt(mine, comm)
        for s in range(steps):
            for i, p in enumerate(_flat(mine)):
                p.grad = grads[s][comm.rank][i].clone()
            o.step()
        return [p.detach().clone() for p in _flat(mine)], o.state_dict()

    results = lw.run(rank_body)
    for r in range(world):
        for got, want in zip(results[r][0], _flat(ref)):
            torch.testing.assert_close(got, want.detach(), rtol=2e-5, atol=2e-6)
    # state layout: AdamW slice on the big param, Muon state on the first param of each group
    sd = results[1][1]["state"]
    assert sd[0]["exp_avg"].shape == (64 // world, 32)
    assert sd[1]["exp_avg"].shape == (7,)
    chunk = -(-5 // world)
    assert sd[2]["momentum_buffer"].shape == (chunk, 16, 24)
    assert sd[2]["second_momentum_buffer"].shape == (chunk, 1, 24)
    assert sd[7]["second_momentum_buffer"].shape == (-(-3 // world), 24, 1)
    assert 3 not in sd and 8 not in sd


def test_adamw_matches_torch_adamw():
    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.randn(33, 17))
    q = torch.nn.Parameter(p.detach().clone())
    ours = MuonAdamW([dict(kind="adamw", params=[p], lr=0.01, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.05)])
    theirs = torch.optim.AdamW([q], lr=0.01, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.05)
    for _ in range(10):
        g = torch.randn_like(p)
        p.grad, q.grad = g.clone(), g.clone()
        ours.step()
        theirs.step()
    torch.testing.assert_close(p, q, rtol=1e-5, atol=1e-6)


def test_muon_first_update_is_nearly_orthogonal_and_deterministic():
    outs = []
    for _ in range(2):
        torch.manual_seed(1)
        p = torch.nn.Parameter(torch.zeros(32, 48))
        o = MuonAdamW([dict(kind="muon", params=[p], lr=1.0, momentum=0.95, ns_steps=5, beta2=0.9, weight_decay=0.0)])
        p.grad = torch.randn(32, 48)
        o.step()
        outs.append(p.detach().clone())
    assert torch.equal(outs[0], outs[1])
    s = torch.linalg.svdvals(outs[0])
    assert (s.max() / s.min()).item() < 4


def test_zero_copy_stack_views_for_contiguous_groups():
    from nanochat_b200.optim import _stack_view
    buf = torch.randn(4, 8, 6)
    views = [buf[i] for i in range(4)]
    st = _stack_view(views)
    assert st is not None and st.data_ptr() == buf.data_ptr() and st.shape == (4, 8, 6)
    assert _stack_view([torch.randn(8, 6) for _ in range(3)]) is None


def test_state_dict_round_trip_resumes_identically():
    torch.manual_seed(0)
    a = _toy_params(5)
    oa = _make_opt(a, NullComm())
    gs = [[torch.randn_like(p) for p in _flat(a)] for _ in range(4)]
    for s in range(2):
        for p, g in zip(_flat(a), gs[s]):
            p.grad = g.clone()
        oa.step()
    b = copy.deepcopy(a)
    ob = _make_opt(b, NullComm())
    ob.load_state_dict(copy.deepcopy(oa.state_dict()))
    for s in range(2, 4):
        for pa, pb, g in zip(_flat(a), _flat(b), gs[s]):
            pa.grad, pb.grad = g.clone(), g.clone()
        oa.step()
        ob.step()
    for pa, pb in zip(_flat(a), _flat(b)):
        assert torch.equal(pa, pb)


def test_functional_steps_with_the_reference_signatures():
    """`adamw_step_fused` / `muon_step_fused` take the reference's arguments (0-D tensors for the hyper-parameters)."""
    import torch
    from nanochat_b200.optim import adamw_step_fused, muon_step_fused
    torch.manual_seed(0)
    p = torch.randn(16, 8)
    q = p.clone().requires_grad_(True)
    oracle = torch.optim.AdamW([q], lr=0.01, betas=(0.8, 0.95), eps=1e-10, weight_decay=0.1)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    t = lambda x: torch.tensor(float(x))
    for step in range(1, 6):
        g = torch.randn(16, 8)
        q.grad = g.clone()
        oracle.step()
        adamw_step_fused(p, g, m, v, t(step), t(0.01), t(0.8), t(0.95), t(1e-10), t(0.1))
    assert torch.allclose(p, q.detach(), rtol=1e-5, atol=1e-6)

    grads = torch.randn(3, 32, 64)
    params = torch.randn(3, 32, 64)
    before = params.clone()
    mom, second = torch.zeros(3, 32, 64), torch.zeros(3, 32, 1)
    muon_step_fused(grads.clone(), params, mom, second, t(0.95), t(0.02), t(0.0), t(0.9), 5, -1)
    update = before - params
    s = torch.linalg.svdvals(update[0])
    assert s.max() / s.min() < 4 and mom.abs().sum() > 0 and second.abs().sum() > 0      # near semi-orthogonal step
