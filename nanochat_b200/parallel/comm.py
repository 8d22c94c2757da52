"""
Collective back ends behind the sharded optimizer.

The optimizer needs three primitives: average a small tensor on every rank,
reduce-scatter-average a tensor along dim 0, and all-gather slices along dim 0.
Back ends:

  * `NullComm`      — world size 1, nothing to do.
  * `TorchDistComm` — `torch.distributed`: NCCL on GPUs (the measured baseline for
                      the fused kernels and the bootstrap channel), gloo on CPU.
                      gloo has neither ReduceOp.AVG nor reduce-scatter, so the CPU
                      path sums with all_reduce, scales by 1/N and slices.
  * `LoopbackWorld` — N logical ranks inside one process (threads + barriers) doing
                      the reductions in fixed rank order; lets the sharding logic be
                      tested with zero GPUs and zero sockets.
  * `SymmComm` (parallel/symm.py) — in-kernel peer-to-peer loads/stores over NVLink
                      on a symmetric heap; the product path on multi-GPU B200.

Reductions in `LoopbackWorld` and `SymmComm` add in rank order 0..N-1 in fp32 and
multiply by 1/N once, so results are bitwise reproducible run to run.

Reference for the call sites being served: nanochat/optim.py:274-318 (reduces) and
:359,407-417 (gathers).
"""

import threading

import torch.distributed as dist


class _Done:
    def wait(self):
        return None


class _DistWork:
    def __init__(self, works, after=None):
        self.works = works
        self.after = after

    def wait(self):
        for w in self.works:
            w.wait()
        if self.after is not None:
            self.after()
            self.after = None


class NullComm:
    rank = 0
    world = 1
    fused = False

    def all_reduce_avg(self, t):
        return _Done()

    def reduce_scatter_avg(self, out, full):
        out.copy_(full)
        return _Done()

    def all_gather(self, full, part):
        if full.data_ptr() != part.data_ptr():
            full.copy_(part)
        return _Done()

    def barrier(self):
        pass


class TorchDistComm:
    """torch.distributed collectives (NCCL or gloo) with the optimizer's averaging semantics."""
    fused = False

    def __init__(self, group=None):
        assert dist.is_initialized()
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.backend = dist.get_backend(group)

    def all_reduce_avg(self, t):
        if self.backend == "nccl":
            return _DistWork([dist.all_reduce(t, op=dist.ReduceOp.AVG, group=self.group, async_op=True)])
        w = dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        return _DistWork([w], after=lambda: t.div_(self.world))

    def reduce_scatter_avg(self, out, full):
        if self.backend == "nccl":
            return _DistWork([dist.reduce_scatter_tensor(out, full, op=dist.ReduceOp.AVG,
                                                         group=self.group, async_op=True)])
        # gloo: sum everything everywhere, keep our rows
        w = dist.all_reduce(full, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        rows = out.shape[0]

        def finish():
            out.copy_(full[self.rank * rows:(self.rank + 1) * rows])
            out.div_(self.world)
        return _DistWork([w], after=finish)

    def all_gather(self, full, part):
        if self.backend == "nccl":
            return _DistWork([dist.all_gather_into_tensor(full, part, group=self.group, async_op=True)])
        rows = part.shape[0]
        pieces = [full[r * rows:(r + 1) * rows] for r in range(self.world)]
        src = part.clone() if part.data_ptr() == pieces[self.rank].data_ptr() else part
        return _DistWork([dist.all_gather(pieces, src, group=self.group, async_op=True)])

    def barrier(self):
        dist.barrier(group=self.group)


class LoopbackWorld:
    """N logical ranks in one process. `run(fn)` calls fn(comm) on N threads and returns the results."""

    def __init__(self, world: int):
        self.world = world
        self._barrier = threading.Barrier(world)
        self._slots = [None] * world
        self._lock = threading.Lock()

    def comm(self, rank: int):
        return _LoopbackComm(self, rank)

    def run(self, fn):
        results = [None] * self.world
        errors = []

        def body(r):
            try:
                results[r] = fn(self.comm(r))
            except BaseException as e:  # surface the first failure, release the others
                errors.append(e)
                self._barrier.abort()
        threads = [threading.Thread(target=body, args=(r,)) for r in range(self.world)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if errors:
            raise errors[0]
        return results

    def _exchange(self, rank, value):
        self._slots[rank] = value
        self._barrier.wait()
        snapshot = list(self._slots)
        self._barrier.wait()
        return snapshot


class _LoopbackComm:
    fused = False

    def __init__(self, world_obj, rank):
        self._w = world_obj
        self.rank = rank
        self.world = world_obj.world

    def _ordered_mean(self, tensors):
        acc = tensors[0].float().clone()
        for t in tensors[1:]:
            acc += t.float()
        return acc * (1.0 / self.world)

    def all_reduce_avg(self, t):
        everyone = self._w._exchange(self.rank, t.detach().clone())
        t.copy_(self._ordered_mean(everyone).to(t.dtype))
        return _Done()

    def reduce_scatter_avg(self, out, full):
        rows = out.shape[0]
        everyone = self._w._exchange(self.rank, full.detach().clone())
        mine = [f[self.rank * rows:(self.rank + 1) * rows] for f in everyone]
        out.copy_(self._ordered_mean(mine).to(out.dtype))
        return _Done()

    def all_gather(self, full, part):
        rows = part.shape[0]
        everyone = self._w._exchange(self.rank, part.detach().clone())
        for r, piece in enumerate(everyone):
            full[r * rows:(r + 1) * rows].copy_(piece)
        return _Done()

    def barrier(self):
        self._w._barrier.wait()


def default_comm():
    """The communicator implied by the process state: torch.distributed if initialised, else none."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        return TorchDistComm()
    return NullComm()
