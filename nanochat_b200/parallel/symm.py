"""
Fused peer-to-peer optimizer path for one NVSwitch domain (2-8 GPUs).

Replaces the optimizer's NCCL collectives (reference: nanochat/optim.py:274-318 reduces,
:359,407-417 gathers) by kernels that read and write the other ranks' memory directly. Ownership,
optimizer state layout and hyper-parameters are the reference's, so per-rank optimizer
checkpoints remain interchangeable with the NCCL path.

Reduce-scatter = a PUSH that rides on the last micro-batch's backward pass. Every rank has a
staging pool (symmetric memory: same layout on every rank) with, for each sharded tensor, one slot
per source rank the size of the owner's slice. On the last micro-batch of a step
  * the weight-gradient GEMM of a matrix owned by another rank writes its result
    (accumulated gradient + this micro-batch's product, fp32) straight into the owner's slot
    for this rank: the GEMM's epilogue stores ARE the transfer, tile by tile, under the rest of
    the backward pass (lm_head: one GEMM per owner's row slice);
  * embedding-table gradients (scatter-adds) are pushed by a copy kernel on a side stream as soon
    as the layer that produces them has run.
The owner then sums its W slots from LOCAL memory inside the update kernels (rank order, so the
result does not depend on timing).

All-gather = the update kernels' write-back: AdamW (`p2p_adamw`) and the Muon update
(`p2p_muon_apply`) store the new bf16 values into every rank's shadow / table from registers.

A step is bracketed by two device-side barriers (bounded waits, status word). Between them the slot
sums, AdamW updates and write-backs and the Muon groups' Newton-Schulz GEMMs run on the caller's stream
(NANOCHAT_OPT_OVERLAP=1 moves the memory-bound kernels to a second stream with a capped number of CTAs;
measured at 2 and 4 GPUs it gains nothing, so it is off by default). The fp32 masters stay with their owners; `sync_masters()` makes every replica's masters
consistent on demand (checkpointing), using NCCL broadcasts since that is rare and off the hot path.

If a step's gradients were not produced through that last-micro-batch path (a driver that calls
backward itself), the missing pushes are made by the copy kernel at the start of the step.
"""

import torch
import torch.distributed as dist

from nanochat_b200.parallel.ownership import adamw_shard, muon_shard

_ALIGN = 256


class _StepTrace:
    """Device time of each stage of a fused step (CUDA events on the launching stream), kept when
    NANOCHAT_OPT_TRACE=1; `SymmComm.trace_report()` returns the milliseconds of the last traced step."""

    def __init__(self, enabled):
        self.enabled = enabled
        self.marks = []

    def begin(self):
        self.marks = []
        self.mark("start")

    def mark(self, name):
        if self.enabled:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.marks.append((name, ev))

    def report(self):
        if len(self.marks) < 2:
            return {}
        torch.cuda.synchronize()
        out = {}
        for (_, a), (name, b) in zip(self.marks, self.marks[1:]):
            out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        return out


class _Pool:
    """A symmetric byte pool with a bump allocator; `peer_ptrs` are the N mapped base addresses."""

    def __init__(self, nbytes, device, group):
        import torch.distributed._symmetric_memory as symm_mem
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.buf, group=group.group_name if hasattr(group, "group_name") else group)
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.used = 0

    def take(self, shape, dtype):
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        start = (self.used + _ALIGN - 1) // _ALIGN * _ALIGN
        assert start + nbytes <= self.buf.numel(), "symmetric pool exhausted"
        self.used = start + nbytes
        return self.buf[start:start + nbytes].view(dtype).view(*shape)

    def offset_of(self, t, dtype_size):
        """Offset of tensor `t` from the pool base, in elements of `dtype_size` bytes."""
        off = t.data_ptr() - self.buf.data_ptr()
        assert 0 <= off < self.buf.numel() and off % dtype_size == 0
        return off // dtype_size


def _pool_sizes(model):
    """Bytes needed in the gradient pool (fp32) and the bf16 pool (shadows + tables + pad)."""
    grad = bf16 = 0
    pad = lambda n: (n + _ALIGN - 1) // _ALIGN * _ALIGN + _ALIGN
    matrix_params = list(model.transformer.h.parameters())
    for shape in {p.shape for p in matrix_params}:
        k = sum(1 for p in matrix_params if p.shape == shape)
        n = k * shape[0] * shape[1]
        grad += pad(4 * n)
        bf16 += pad(2 * n)
    big = [model.lm_head.weight, model.transformer.wte.weight] + [ve.weight for ve in model.value_embeds.values()]
    for p in big:
        grad += pad(4 * p.numel())
        bf16 += pad(2 * p.numel())
    seen = {id(p) for p in matrix_params} | {id(p) for p in big}
    for p in model.parameters():
        if id(p) not in seen:
            grad += pad(4 * p.numel())
    return grad + 4096, bf16 + 4096


def _stage_plan(model, world):
    """Staging regions: {key: (offset in fp32 elements, slice elements)} and the pool size in bytes. Keys are
    ('muon', shape) for a Muon stack and id(param) for a row-sharded AdamW tensor; a region is `world` slots of
    one owner's slice."""
    plan, off = {}, 0
    align = _ALIGN // 4
    matrix_params = list(model.transformer.h.parameters())
    for shape in sorted({tuple(p.shape) for p in matrix_params}):
        if shape[0] % 8 or shape[1] % 8:
            continue
        k = sum(1 for p in matrix_params if tuple(p.shape) == shape)
        slice_elems = -(-k // world) * shape[0] * shape[1]
        plan[("muon", shape)] = (off, slice_elems)
        off = (off + world * slice_elems + align - 1) // align * align
    big = [model.lm_head.weight, model.transformer.wte.weight] + [ve.weight for ve in model.value_embeds.values()]
    for p in big:
        assert p.shape[0] % world == 0, "row-sharded tensors need rows divisible by the world size"
        slice_elems = p.shape[0] // world * p.shape[1]
        plan[id(p)] = (off, slice_elems)
        off = (off + world * slice_elems + align - 1) // align * align
    return plan, off * 4 + 4096


class SymmComm:
    """Communicator whose `fused_step` runs the whole sharded optimizer step with in-kernel NVLink traffic."""

    fused = True

    def __init__(self, model, group=None):
        from nanochat_b200 import ops
        from nanochat_b200.parallel.arena import ParamArena
        assert dist.is_initialized() and dist.get_world_size(group) > 1
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        assert self.world <= 8, "one NVSwitch domain: at most 8 ranks"
        self.nat = ops.native_module()
        dev = model.get_device()
        grad_bytes, bf16_bytes = _pool_sizes(model)
        self.grad_pool = _Pool(grad_bytes, dev, self.group)
        self.bf16_pool = _Pool(bf16_bytes, dev, self.group)
        self.pad_pool = _Pool(4096, dev, self.group)
        self.pad_pool.buf.zero_()
        self.stage_plan, stage_bytes = _stage_plan(model, self.world)
        self.stage_pool = _Pool(stage_bytes, dev, self.group)
        # each rank's staging pool as an fp32 tensor in this process (peer memory for the others): slices of these
        # are the `out` operands of the last micro-batch's weight-gradient GEMMs
        self.stage_peer = [self.stage_pool.handle.get_buffer(o, (stage_bytes // 4,), torch.float32, 0)
                           for o in range(self.world)]
        self._targets = {}            # id(param) -> [(row_lo, row_hi, remote out tensor or None)]
        self._pushed = set()          # ids of parameters / table entries whose final gradient reached its owners
        self._sink_on = False
        self.epoch = 0
        import os
        self.trace = _StepTrace(os.environ.get("NANOCHAT_OPT_TRACE", "0") == "1")
        # NANOCHAT_OPT_OVERLAP=1 runs the slot sums + AdamW kernels on a second stream beside the Newton-Schulz GEMMs
        # (default off: since the gradients arrive by push those kernels read local memory and take ~2 ms; measured
        # at 2 and 4 GPUs the overlap gives nothing and slows the GEMMs); NANOCHAT_OPT_LINK_CTAS caps their grid then
        self.overlap = os.environ.get("NANOCHAT_OPT_OVERLAP", "0") != "0"
        self.link_ctas = int(os.environ.get("NANOCHAT_OPT_LINK_CTAS", "296")) if self.overlap else 0
        self._link_stream = torch.cuda.Stream(device=dev)
        self.time_updates = False     # benchmarks: keep an event pair per step, read with `update_ms()`

        def alloc(shape, dtype, device, role="master"):
            if role == "grad":
                return self.grad_pool.take(shape, dtype)
            if role in ("shadow", "table"):
                return self.bf16_pool.take(shape, dtype)
            return torch.empty(shape, dtype=dtype, device=device)

        self.arena = ParamArena(model, alloc=alloc, with_shadows=True)
        self._fallback = None
        self._plan_targets()
        torch.cuda.synchronize()
        dist.barrier(group)

    @classmethod
    def create(cls, model, group=None):
        return cls(model, group)

    # TorchDistComm surface for the pieces that stay on NCCL (tiny Muon groups)
    def _nccl(self):
        if self._fallback is None:
            from nanochat_b200.parallel.comm import TorchDistComm
            self._fallback = TorchDistComm(None if self.group is dist.group.WORLD else self.group)
        return self._fallback

    # ------------------------------------------------------------------ gradient pushes
    def _plan_targets(self):
        """Where each non-owned gradient goes: a view of the owner's slot for this rank."""
        W, me = self.world, self.rank
        for g in self.arena.muon_groups:
            r, c = g["shape"]
            if r % 8 or c % 8:
                continue
            off, slice_elems = self.stage_plan[("muon", (r, c))]
            chunk = -(-len(g["params"]) // W)
            for j, p in enumerate(g["params"]):
                owner = j // chunk
                if owner == me:
                    continue
                at = off + me * slice_elems + (j % chunk) * r * c
                self._targets[id(p)] = [(0, r, self.stage_peer[owner][at:at + r * c].view(r, c))]
        for d in self.arena.adamw_big:
            p = d["param"]
            if p.dtype != torch.float32:
                continue                      # bf16 tables: scatter-added gradients, pushed by the copy kernel
            off, slice_elems = self.stage_plan[id(p)]
            rows, cols = p.shape[0] // W, p.shape[1]
            at = off + me * slice_elems
            self._targets[id(p)] = [
                (o * rows, (o + 1) * rows,
                 None if o == me else self.stage_peer[o][at:at + slice_elems].view(rows, cols)) for o in range(W)]

    # surface used by ops.native while the last micro-batch's backward runs
    def targets(self, w):
        return self._targets.get(id(w))

    def mark_pushed(self, w):
        self._pushed.add(id(w))

    def table_grad_final(self, p):
        """Called by the backward pass right after the kernel that completes a table's gradient: push it to the
        owners on the link stream, under the rest of the backward pass."""
        d = self._entry_of(p)
        if d is None or id(p) in self._pushed:
            return
        main = torch.cuda.current_stream()
        self._link_stream.wait_stream(main)
        with torch.cuda.stream(self._link_stream):
            self._push_sharded(d["grad"], self.stage_plan[id(p)], 148)    # few CTAs: it shares the GPU with the backward pass
        self._pushed.add(id(p))

    def begin_last_microbatch(self):
        """From here to `end_last_microbatch()` gradients are final when written: deliver them to their owners."""
        self._sink_on = True
        self.nat.set_grad_sink(self)

    def end_last_microbatch(self):
        self._sink_on = False
        self.nat.set_grad_sink(None)

    def _push_sharded(self, grad, plan_entry, max_ctas=0):
        off, slice_elems = plan_entry
        self.nat._C.p2p_push_slices(grad.view(-1), slice_elems, self.stage_pool.peer_ptrs,
                                    off + self.rank * slice_elems, self.rank, max_ctas)

    def _push_missing(self):
        """Gradients that did not travel with the backward pass (a driver that runs its own backward calls)."""
        W, me = self.world, self.rank
        for g in self.arena.muon_groups:
            r, c = g["shape"]
            if r % 8 or c % 8:
                continue
            remote = [p for p in g["params"] if id(p) in self._targets]
            missing = [p for p in remote if id(p) not in self._pushed]
            if not missing:
                continue
            if len(missing) == len(remote):
                self._push_sharded(g["grad"], self.stage_plan[("muon", (r, c))])
            else:
                for p in missing:
                    dst = self._targets[id(p)][0][2]
                    self.nat._C.p2p_copy_f32(p.grad, dst.data_ptr())
        for d in self.arena.adamw_big:
            p = d["param"]
            if id(p) not in self._pushed:
                self._push_sharded(d["grad"], self.stage_plan[id(p)])
        self._pushed.clear()

    def _slots(self, plan_entry, own_grad_ptr):
        """The W addresses an owner sums: its slot for every source rank, and its own gradient where it lies."""
        off, slice_elems = plan_entry
        base = self.stage_pool.peer_ptrs[self.rank]
        ptrs = [base + 4 * (off + s * slice_elems) for s in range(self.world)]
        ptrs[self.rank] = own_grad_ptr
        return ptrs

    def barrier(self):
        self.epoch += 1
        self.nat._C.p2p_barrier(self.pad_pool.peer_ptrs, self.rank, self.epoch, self.pad_pool.buf)

    # ------------------------------------------------------------------ the fused step
    def _entry_of(self, p):
        for d in self.arena.adamw_big:
            if d["param"] is p:
                return d
        return None

    @torch.no_grad()
    def fused_step(self, opt):
        """The whole sharded update between two device barriers. The gradients are already in their owners' staging
        slots (pushed by the last micro-batch's weight-gradient GEMM epilogues and by the table copy kernels), so
        after the first barrier everything reads local memory: per Muon group the owner sums its W slots inside the
        momentum kernel, orthogonalises the stack on the tensor cores and stores the updated bf16 matrices to every
        rank from the update kernel; the AdamW kernels do the same for the row-sharded tables and lm_head. With
        `self.overlap` (off by default: measured no gain) the slot sums and AdamW kernels run on a second stream
        beside the Newton-Schulz GEMMs; otherwise everything is issued on the caller's stream."""
        C = self.nat._C
        gp, bp = self.grad_pool, self.bf16_pool
        tr = self.trace
        main = torch.cuda.current_stream()
        link = self._link_stream if self.overlap else main
        tr.begin()
        main.wait_stream(self._link_stream)              # table pushes issued during the backward pass
        self._push_missing()
        tr.mark("late pushes")
        self.barrier()                                   # every rank's gradients have landed in their owners' slots
        tr.mark("barrier_in")
        if self.time_updates:                            # from "every rank has arrived" to the end of the step
            self._t0 = torch.cuda.Event(enable_timing=True)
            self._t0.record()
        link.wait_stream(main)
        muon = [g for g in opt.param_groups if g["kind"] == "muon"]
        adamw = [g for g in opt.param_groups if g["kind"] == "adamw"]
        jobs = []
        with torch.cuda.stream(link):
            for group in muon:
                job = self._muon_pull(opt, group, C, gp)
                if job is not None:
                    job["pulled"] = torch.cuda.Event()
                    job["pulled"].record(link)
                    jobs.append(job)
                    if not self.overlap:
                        tr.mark(job["tag"] + "pull+momentum")
            for group in adamw:
                self._adamw_group(opt, group, C, gp, bp)
                if not self.overlap:
                    tr.mark("adamw " + "x".join(str(d) for d in group["params"][0].shape) + f" n={len(group['params'])}")
        for group in muon:
            r, c = group["params"][0].shape
            if r % 8 or c % 8:
                self._muon_tiny(opt, group)              # NCCL on the caller's stream while the link stream pulls
                tr.mark(f"muon {r}x{c} (nccl)")
        for job in jobs:
            main.wait_event(job["pulled"])
            self._muon_update(opt, job, C, bp)
        main.wait_stream(link)
        tr.mark("link stream tail")
        self.barrier()                                   # write-backs landed; peers are done reading my grads
        tr.mark("barrier_out")
        if self.time_updates:
            self._t1 = torch.cuda.Event(enable_timing=True)
            self._t1.record()
        for g in self.arena.muon_groups:
            if g["shadow"] is not None:
                for p in g["params"]:
                    self.nat.mark_shadow_fresh(p)
        for d in self.arena.adamw_big:
            if d["shadow"] is not None:
                self.nat.mark_shadow_fresh(d["param"])

    def _adamw_group(self, opt, group, C, gp, bp):
        b1, b2 = group["betas"]
        for p in group["params"]:
            shard = adamw_shard(tuple(p.shape), self.rank, self.world)
            state = opt.state[p]
            if shard.replicated:
                if not state:
                    state["step"] = 0
                    state["exp_avg"] = torch.zeros_like(p)
                    state["exp_avg_sq"] = torch.zeros_like(p)
                state["step"] += 1
                C.p2p_small_adamw(gp.peer_ptrs, gp.offset_of(p.grad, 4), p.data, state["exp_avg"], state["exp_avg_sq"],
                                  group["lr"], b1, b2, group["eps"], group["weight_decay"], state["step"])
                continue
            entry = self._entry_of(p)
            cols = p.shape[1]
            p_slice = p.data[shard.row_start:shard.row_end]
            if not state:
                state["step"] = 0
                state["exp_avg"] = torch.zeros_like(p_slice)
                state["exp_avg_sq"] = torch.zeros_like(p_slice)
            state["step"] += 1
            slots = self._slots(self.stage_plan[id(p)], entry["grad"][shard.row_start:shard.row_end].data_ptr())
            if p.dtype == torch.bfloat16:      # the table itself is the bf16 tensor every rank reads
                out_off = bp.offset_of(p.data, 2) + shard.row_start * cols
                write_local = False            # the kernel already wrote p_slice in place
            else:
                out_off = bp.offset_of(entry["shadow"], 2) + shard.row_start * cols
                write_local = True
            C.p2p_adamw(slots, 0, self.rank, p_slice, state["exp_avg"], state["exp_avg_sq"],
                        bp.peer_ptrs, out_off, write_local, group["lr"], b1, b2, group["eps"],
                        group["weight_decay"], state["step"], self.link_ctas)

    def _muon_tiny(self, opt, group):
        """The value-embedding gate matrices (a few KB): averaged with NCCL, generic sharded update."""
        info = opt._launch_muon(group, self._nccl())
        gathers = []
        opt._finish_muon(group, info, self._nccl(), gathers)
        for work, stacked, ps in gathers:
            work.wait()
            torch._foreach_copy_([p.data for p in ps], list(stacked[:len(ps)].unbind(0)))

    def _muon_pull(self, opt, group, C, gp):
        """Link-stream half of a Muon group: pull and average the gradients of the matrices this rank owns inside the
        momentum kernel. Returns the job the compute stream continues with (None for tiny or unowned groups)."""
        params = group["params"]
        p0 = params[0]
        r, c = p0.shape
        if r % 8 or c % 8:
            return None
        entry = next(g for g in self.arena.muon_groups if g["params"][0] is p0)
        shard = muon_shard(len(params), self.rank, self.world)
        state = opt.state[p0]
        if "momentum_buffer" not in state:
            state["momentum_buffer"] = torch.zeros(shard.chunk, r, c, dtype=p0.dtype, device=p0.device)
            sshape = (shard.chunk, r, 1) if r >= c else (shard.chunk, 1, c)
            state["second_momentum_buffer"] = torch.zeros(sshape, dtype=p0.dtype, device=p0.device)
        n = shard.num_owned
        tag = f"muon {r}x{c}: "
        if n == 0:
            if not self.overlap:
                self.trace.mark(tag + "pull+momentum")
            for stage in ("equilibrate", "newton-schulz", "finish+write-back"):
                self.trace.mark(tag + stage)          # same keys on every rank (the report is reduced over ranks)
            return None
        nat = self.nat
        dev = p0.device
        key = f"_{r}x{c}"                             # scratch is per group: all groups' pulls are in flight at once
        job = dict(group=group, entry=entry, shard=shard, state=state, n=n, r=r, c=c, tag=tag,
                   X=nat._scratch("muon_X" + key, (n, r, c), torch.bfloat16, dev),
                   rowss=nat._scratch("muon_rowss" + key, (n * r,), torch.float32, dev),
                   rowss2=nat._scratch("muon_rowss2" + key, (n * r,), torch.float32, dev),
                   total=nat._scratch("muon_total" + key, (n,), torch.float32, dev),
                   total2=nat._scratch("muon_total2" + key, (n,), torch.float32, dev))
        slots = self._slots(self.stage_plan[("muon", (r, c))], entry["grad"][shard.start:shard.start + n].data_ptr())
        C.p2p_muon_momentum(slots, 0, state["momentum_buffer"][:n], job["X"], job["rowss"], job["total"],
                            group["momentum"], self.link_ctas)
        return job

    def _muon_update(self, opt, job, C, bp):
        """Compute-stream half: equilibrate, polar iteration on the tensor cores, update + write-back to every rank."""
        group, entry, shard, state = job["group"], job["entry"], job["shard"], job["state"]
        n, r, c, tag = job["n"], job["r"], job["c"], job["tag"]
        nat = self.nat
        dev = job["X"].device
        C.muon_equilibrate(job["X"], job["rowss"], job["total"], job["rowss2"], job["total2"])
        self.trace.mark(tag + "equilibrate")
        Xo = nat.polar_express_native(job["X"], group["ns_steps"])
        self.trace.mark(tag + "newton-schulz")
        m = max(r, c)
        ss = nat._scratch("muon_ss", (n * m,), torch.float32, dev)
        scale = nat._scratch("muon_scale", (n * m,), torch.float32, dev)
        lr = group["lr"] * max(1.0, r / c) ** 0.5
        master = entry["master"][shard.start:shard.start + n]
        out_off = bp.offset_of(entry["shadow"], 2) + shard.start * r * c
        C.p2p_muon_finish(master, Xo, state["second_momentum_buffer"][:n].view(n, -1), ss, scale, bp.peer_ptrs, out_off,
                          lr, group["weight_decay"], group["beta2"])
        self.trace.mark(tag + "finish+write-back")

    def trace_report(self):
        return self.trace.report()

    def update_ms(self):
        """Device time of the last step from the moment every rank had arrived (after the first barrier's wait, which
        is the ranks' skew, not work) to the end of the second barrier. Synchronises."""
        self._t1.synchronize()
        return self._t0.elapsed_time(self._t1)

    # ---------------------------------------------------------------- master consistency
    @torch.no_grad()
    def sync_masters(self):
        """Make every rank's fp32 masters equal to their owners' (before saving a full-model checkpoint)."""
        for g in self.arena.muon_groups:
            K = len(g["params"])
            if g["shape"][0] % 8 or g["shape"][1] % 8:
                continue                     # tiny groups are gathered by the NCCL path every step
            chunk = -(-K // self.world)
            for owner in range(self.world):
                lo, hi = owner * chunk, min(K, (owner + 1) * chunk)
                if lo < hi:
                    dist.broadcast(g["master"][lo:hi], src=dist.get_global_rank(self.group, owner), group=self.group)
        for d in self.arena.adamw_big:
            p = d["param"]
            if p.dtype != torch.float32:
                continue                     # bf16 tables are written on every rank by the update kernel
            rows = p.shape[0] // self.world
            for owner in range(self.world):
                dist.broadcast(p.data[owner * rows:(owner + 1) * rows],
                               src=dist.get_global_rank(self.group, owner), group=self.group)
