"""
MuonAdamW: one optimizer for the whole model — AdamW for embeddings, the
unembedding and scalars; Muon (Nesterov momentum -> row equilibration -> Polar
Express orthogonalisation -> Frobenius renorm -> NorMuon second-moment rescale ->
cautious weight decay) for every 2-D matrix of the transformer blocks.

Gradient averaging and ZeRO-2-style state sharding live here, not in a DDP
wrapper (reference: nanochat/optim.py:184-459). The ownership map is the
reference's (see parallel/ownership.py) so per-rank optimizer checkpoints are
interchangeable; `state_dict()` has the reference's layout: AdamW entries
{step, exp_avg, exp_avg_sq} per parameter (shaped like the rank's row slice),
Muon entries {momentum_buffer, second_momentum_buffer} on the FIRST parameter of
each group with a leading dim of ceil(K/world).

What is different by design:
  * A Muon group whose parameters (and gradients) already sit back to back in one
    buffer (see parallel/arena.py) is updated through zero-copy stack views: no
    torch.stack of gradients, no copy-back of parameters.
  * Collectives come from a `comm` object (parallel/comm.py). With `SymmComm` the
    reduce-scatter is a peer-to-peer pull fused into the update kernels and the
    all-gather is the update kernel's write-back to every peer; with
    `TorchDistComm` it is NCCL/gloo (baseline and CPU path).
  * Update math runs in the hand-written fused kernels on CUDA (`ops.native`) and in
    the PyTorch reference bodies elsewhere; no tracing compiler is involved.
"""

import torch

from nanochat_b200 import ops
from nanochat_b200.ops import reference as ref_ops
from nanochat_b200.parallel.comm import default_comm
from nanochat_b200.parallel.ownership import adamw_shard, muon_shard

polar_express_coeffs = list(ref_ops.POLAR_EXPRESS_COEFFS)


def _stack_view(tensors):
    """A (K, *shape) tensor aliasing `tensors` if they lie back to back in memory, else None."""
    first = tensors[0]
    if not first.is_contiguous():
        return None
    step = first.numel() * first.element_size()
    base = first.data_ptr()
    storage = first.untyped_storage().data_ptr()
    for j, t in enumerate(tensors):
        if (t.data_ptr() != base + j * step or not t.is_contiguous() or t.dtype != first.dtype
                or t.untyped_storage().data_ptr() != storage):
            return None
    try:
        return torch.as_strided(first, (len(tensors), *first.shape),
                                (first.numel(), *first.stride()))
    except RuntimeError:
        return None


def _use_native(t):
    return t.is_cuda and ops.get_kernel_mode() == "native"


def _scalar(v):
    return float(v.item()) if isinstance(v, torch.Tensor) else float(v)


def adamw_step_fused(p, grad, exp_avg, exp_avg_sq, step_t, lr_t, beta1_t, beta2_t, eps_t, wd_t):
    """One AdamW step in place on `p` and its moments, with the reference's functional signature
    (reference: nanochat/optim.py:24-63; hyper-parameters as 0-D tensors or numbers). On a B200 this is the fused
    kernel of `ops/csrc/optim.cu`, elsewhere the plain-PyTorch body."""
    args = (p, grad, exp_avg, exp_avg_sq, int(_scalar(step_t)), _scalar(lr_t), _scalar(beta1_t), _scalar(beta2_t),
            _scalar(eps_t), _scalar(wd_t))
    if _use_native(p):
        ops.native_module().adamw_update(*args)
    else:
        ref_ops.adamw_update(*args)


def muon_step_fused(stacked_grads, stacked_params, momentum_buffer, second_momentum_buffer, momentum_t, lr_t, wd_t,
                    beta2_t, ns_steps, red_dim):
    """One Muon step on stacked (k, r, c) tensors, in place on the parameters and both buffers, with the reference's
    functional signature (reference: nanochat/optim.py:112-180). `stacked_grads` is clobbered."""
    from nanochat_b200 import common
    args = (stacked_grads, stacked_params, momentum_buffer, second_momentum_buffer, _scalar(momentum_t), _scalar(lr_t),
            _scalar(wd_t), _scalar(beta2_t), int(ns_steps), int(red_dim))
    if _use_native(stacked_params):
        ops.native_module().muon_update(*args)
    else:
        ref_ops.muon_update(*args, use_bf16=(common.COMPUTE_DTYPE == torch.bfloat16))


class MuonAdamW(torch.optim.Optimizer):
    """param_groups: dicts with 'params', 'kind' ('adamw' | 'muon') and the kind's hyper-parameters
    (adamw: lr, betas, eps, weight_decay; muon: lr, momentum, ns_steps, beta2, weight_decay)."""

    def __init__(self, param_groups, comm=None):
        super().__init__(param_groups, defaults={})
        self.comm = comm

    # ------------------------------------------------------------ AdamW
    def _launch_adamw(self, group, comm):
        jobs = []
        for p in group["params"]:
            shard = adamw_shard(tuple(p.shape), comm.rank, comm.world)
            grad = p.grad
            grad32 = getattr(p, "grad32", None)   # fp32 accumulator kept by the native embedding kernels
            if grad32 is not None:
                grad = grad32
                if getattr(p, "_arena", None) is None:
                    self._consumed.append(grad32)     # an arena clears its own buffers
            if comm.world == 1:
                jobs.append((p, shard, grad, None))
            elif shard.replicated:
                jobs.append((p, shard, grad, comm.all_reduce_avg(grad)))
            else:
                g_slice = torch.empty_like(grad[:shard.rows])
                jobs.append((p, shard, g_slice, comm.reduce_scatter_avg(g_slice, grad)))
        return jobs

    def _finish_adamw(self, group, jobs, comm, gathers):
        beta1, beta2 = group["betas"]
        for p, shard, g, work in jobs:
            if work is not None:
                work.wait()
            p_slice = p if shard.replicated else p[shard.row_start:shard.row_end]
            state = self.state[p]
            if not state:
                state["step"] = 0
                state["exp_avg"] = torch.zeros_like(p_slice)
                state["exp_avg_sq"] = torch.zeros_like(p_slice)
            state["step"] += 1
            args = (p_slice, g, state["exp_avg"], state["exp_avg_sq"], state["step"],
                    group["lr"], beta1, beta2, group["eps"], group["weight_decay"])
            if _use_native(p):
                ops.native_module().adamw_update(*args, master=p)
            else:
                ref_ops.adamw_update(*args)
            if not shard.replicated:
                gathers.append((comm.all_gather(p, p_slice), None, None))
                if _use_native(p) and p.dtype == torch.float32:
                    # the other ranks' rows arrive behind autograd's back: the bf16 operand copy must be re-cast
                    self._stale_shadows.append(p)

    # ------------------------------------------------------------- Muon
    def _launch_muon(self, group, comm):
        params = group["params"]
        shard = muon_shard(len(params), comm.rank, comm.world)
        grads = [p.grad for p in params]
        stacked = _stack_view(grads)
        if comm.world == 1:
            if stacked is None:
                stacked = torch.stack(grads)
            return dict(shard=shard, work=None, grad_chunk=stacked, gather_buf=None)
        p0 = params[0]
        if stacked is not None and shard.padded == len(params):
            full = stacked
        else:
            full = torch.empty(shard.padded, *p0.shape, dtype=p0.dtype, device=p0.device)
            if stacked is not None:
                full[:len(params)].copy_(stacked)
            else:
                torch.stack(grads, out=full[:len(params)])
            if shard.padded > len(params):
                full[len(params):].zero_()
        chunk = torch.empty(shard.chunk, *p0.shape, dtype=p0.dtype, device=p0.device)
        work = comm.reduce_scatter_avg(chunk, full)
        return dict(shard=shard, work=work, grad_chunk=chunk, gather_buf=full)

    def _finish_muon(self, group, info, comm, gathers):
        if info["work"] is not None:
            info["work"].wait()
        params = group["params"]
        shard = info["shard"]
        p0 = params[0]
        r, c = p0.shape[-2], p0.shape[-1]
        state = self.state[p0]
        if "momentum_buffer" not in state:
            state["momentum_buffer"] = torch.zeros(shard.chunk, r, c, dtype=p0.dtype, device=p0.device)
        if "second_momentum_buffer" not in state:
            sshape = (shard.chunk, r, 1) if r >= c else (shard.chunk, 1, c)
            state["second_momentum_buffer"] = torch.zeros(sshape, dtype=p0.dtype, device=p0.device)
        red_dim = -1 if r >= c else -2

        owned = params[shard.start:shard.start + shard.num_owned]
        owned_stack, aliased = None, False
        if shard.num_owned > 0:
            owned_stack = _stack_view([p.data for p in owned])
            aliased = owned_stack is not None
            if not aliased:
                owned_stack = torch.stack([p.data for p in owned])
            lr = group["lr"] * max(1.0, r / c) ** 0.5
            n = shard.num_owned
            args = (info["grad_chunk"][:n], owned_stack, state["momentum_buffer"][:n],
                    state["second_momentum_buffer"][:n], group["momentum"], lr,
                    group["weight_decay"], group["beta2"], group["ns_steps"], red_dim)
            if _use_native(p0) and p0.dtype == torch.float32:
                ops.native_module().muon_update(*args, params=owned)
            else:
                from nanochat_b200 import common
                ref_ops.muon_update(*args, use_bf16=(common.COMPUTE_DTYPE == torch.bfloat16))

        if comm.world == 1:
            if not aliased and owned_stack is not None:
                torch._foreach_copy_([p.data for p in params], list(owned_stack.unbind(0)))
            return
        send = torch.zeros(shard.chunk, r, c, dtype=p0.dtype, device=p0.device)
        if shard.num_owned > 0:
            send[:shard.num_owned].copy_(owned_stack)
        out = info["gather_buf"]
        if out.data_ptr() == p0.grad.data_ptr():
            # the reduce input aliased the live gradient stack; gather into a scratch stack instead
            out = torch.empty(shard.padded, r, c, dtype=p0.dtype, device=p0.device)
        gathers.append((comm.all_gather(out, send), out, params))

    # ------------------------------------------------------------- step
    @torch.no_grad()
    def step(self):
        if torch.cuda.is_available() and ops.get_kernel_mode() == "native":
            ops.native_module().sync_wgrad_stream()     # weight gradients are produced on a side stream
        comm = self.comm if self.comm is not None else default_comm()
        if getattr(comm, "fused", False):
            return comm.fused_step(self)
        launched = []
        self._consumed = []
        self._stale_shadows = []
        for group in self.param_groups:
            if group["kind"] == "adamw":
                launched.append(self._launch_adamw(group, comm))
            elif group["kind"] == "muon":
                launched.append(self._launch_muon(group, comm))
            else:
                raise ValueError(f"Unknown optimizer kind: {group['kind']}")
        gathers = []
        for group, info in zip(self.param_groups, launched):
            if group["kind"] == "adamw":
                self._finish_adamw(group, info, comm, gathers)
            else:
                self._finish_muon(group, info, comm, gathers)
        for work, stacked, params in gathers:
            work.wait()
            if params is not None:
                torch._foreach_copy_([p.data for p in params], list(stacked[:len(params)].unbind(0)))
        for g in self._consumed:
            g.zero_()
        self._consumed = []
        if self._stale_shadows:
            table = ops.native_module()._shadow
            for p in self._stale_shadows:
                ent = table.get(p)
                if ent is not None:
                    table.set(p, -1, ent[1])     # keep the buffer, force a refresh on next use
            self._stale_shadows = []
