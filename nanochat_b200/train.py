"""
One optimizer step as a callable, shared by every training driver (pretraining, SFT, RL, the
benchmark): gradient accumulation over micro-batches, the sharded MuonAdamW update, gradient reset,
and the two things a driver needs around it: a full-model state_dict that is right on every back
end, and the choice of optimizer collectives.

The loop body it replaces is reference scripts/base_train.py:510-540 (and the same block of
scripts/chat_sft.py / scripts/chat_rl.py). What it adds on a B200:

  * the parameter arena (parallel/arena.py) is always built on the CUDA bf16 path, so the layer runs
    one fused QKV GEMM, the fp8 layer path is reachable, and gradients are persistent buffers that
    are re-armed (`arena.zero_grads()`), never dropped;
  * with more than one rank the fused peer-to-peer optimizer (`parallel/symm.py`) is the default;
    its fp32 masters are complete only on their owners, so `model_state_dict()` first makes every
    replica consistent (`sync_masters`) and only then walks the parameters.
"""

import torch
import torch.distributed as dist

from nanochat_b200 import common
from nanochat_b200.utils.trace import PhaseTimers


def native_bf16_path(device_type):
    """True when the model runs on the hand-written kernels (CUDA, bf16 compute, native kernel mode)."""
    from nanochat_b200 import ops
    return (device_type == "cuda" and common.COMPUTE_DTYPE == torch.bfloat16
            and ops.get_kernel_mode() == "native")


def make_comm(model, mode="auto", log=None):
    """Optimizer collectives for this job. mode: 'auto' (fused peer-to-peer kernels when more than one CUDA
    rank runs the native path, else torch.distributed), 'fused' (required: errors propagate) or 'nccl'.
    Returns (comm or None, description). None means "the optimizer's default" (NCCL / gloo / single rank)."""
    world = dist.get_world_size() if dist.is_initialized() else 1
    if world == 1:
        return None, "none (1 rank)"
    device_type = model.get_device().type
    want_fused = mode == "fused" or (mode == "auto" and native_bf16_path(device_type))
    if want_fused:
        try:
            from nanochat_b200.parallel.symm import SymmComm
            return SymmComm.create(model), "fused peer-to-peer kernels (symmetric memory over NVLink)"
        except Exception as e:          # peer access unavailable: stay on torch.distributed and say so
            if mode == "fused":
                raise
            if log is not None:
                log(f"fused peer-to-peer optimizer path unavailable ({type(e).__name__}: {e}); using NCCL")
    return None, "nccl" if device_type == "cuda" else "gloo"


class TrainStep:
    """`comm` is a communicator object, None, or one of the `make_comm` modes ('auto', 'fused', 'nccl')."""

    def __init__(self, model, grad_accum=1, comm=None, optimizer=None, use_arena=None, timers=None, scaler=None,
                 log=None, **optimizer_kwargs):
        self.model = model
        device_type = model.get_device().type
        # phase timers are inert (no events, no extra launches) unless NANOCHAT_TRACE=1 or one is passed in
        self.timers = timers if timers is not None else PhaseTimers(device_type=device_type)
        self.comm_name = None
        if isinstance(comm, str):
            comm, self.comm_name = make_comm(model, comm, log=log)
        self.comm = comm
        if use_arena is None:
            use_arena = native_bf16_path(device_type)
        if use_arena and getattr(model, "_arena", None) is None:
            from nanochat_b200.parallel.arena import ParamArena
            ParamArena(model)
        self.grad_accum = grad_accum
        self.scaler = scaler            # torch.amp.GradScaler for fp16 compute, else None
        self.optimizer = optimizer if optimizer is not None else model.setup_optimizer(comm=comm, **optimizer_kwargs)
        if optimizer is not None and comm is not None:
            self.optimizer.comm = comm
        self.steps_done = 0
        # set to a list to collect a (start, end) CUDA event pair around every optimizer update (benchmarks: the
        # update's exposed device time inside real steps, after whatever it overlapped with the backward pass)
        self.optimizer_events = None

    # ------------------------------------------------------------------------------ one step
    def backward(self, loss):
        """Backward pass of one (already scaled) micro-batch loss."""
        with self.timers.phase("backward"):
            if self.scaler is not None:
                self.scaler.scale(loss).backward()
            else:
                loss.backward()

    def optimizer_step(self):
        """Sharded optimizer update on the accumulated gradients, then gradient reset."""
        events = None
        if self.optimizer_events is not None and self.model.get_device().type == "cuda":
            events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            events[0].record()
        with self.timers.phase("optimizer"):
            if self.scaler is not None:
                self.scaler.unscale_(self.optimizer)
                if dist.is_initialized() and dist.get_world_size() > 1:     # every rank must agree on skipping
                    for v in self.scaler._found_inf_per_device(self.optimizer).values():
                        dist.all_reduce(v, op=dist.ReduceOp.MAX)
                self.scaler.step(self.optimizer)
                self.scaler.update()
            else:
                self.optimizer.step()
        if events is not None:
            events[1].record()
            self.optimizer_events.append(events)
        self.zero_grads()
        self.steps_done += 1

    def zero_grads(self):
        arena = getattr(self.model, "_arena", None)
        if arena is not None:
            arena.zero_grads()      # persistent gradient buffers: re-arm "first write overwrites"
        else:
            # dropping the buffers lets the first wgrad of the next step write instead of read-modify-write
            self.model.zero_grad(set_to_none=True)

    def step(self, fetch, loss_scale=None, after_backward=None, before_update=None):
        """`fetch(i)` returns the (inputs, targets) of micro-batch i; `after_backward(i)` runs once its backward
        pass is queued (the drivers fetch the next batch there, so host-side packing overlaps the GPU work);
        `before_update()` runs after the last backward and before the update (schedules that depend on how much
        data the step consumed). Returns the last micro-batch's loss (detached, on device)."""
        scale = (1.0 / self.grad_accum) if loss_scale is None else loss_scale
        loss = None
        comm = self.comm if self.comm is not None else getattr(self.optimizer, "comm", None)
        sink = comm if hasattr(comm, "begin_last_microbatch") else None
        for i in range(self.grad_accum):
            x, y = fetch(i)
            with self.timers.phase("forward"):
                loss = self.model(x, y)
            last = sink is not None and i == self.grad_accum - 1
            if last:
                sink.begin_last_microbatch()      # gradients written from here on are final: they go to their owners
            try:
                self.backward(loss * scale)
            finally:
                if last:
                    sink.end_last_microbatch()
            if after_backward is not None:
                after_backward(i)
        if before_update is not None:
            before_update()
        self.optimizer_step()
        return loss.detach()

    # ------------------------------------------------------------------------- checkpoints
    def sync_masters(self):
        """Collective: after it every rank's fp32 parameters equal their owners'. A no-op on back ends that
        all-gather the parameters every step."""
        comm = self.comm if self.comm is not None else getattr(self.optimizer, "comm", None)
        if comm is not None and hasattr(comm, "sync_masters"):
            comm.sync_masters()

    def model_state_dict(self):
        """Collective on every rank: the model's `state_dict()` with every parameter current. With the fused
        optimizer path only the owner of a matrix (or row slice) updates its fp32 master; the others hold the
        bf16 copy their kernels consume, so the masters are synchronised before the parameters are walked."""
        self.sync_masters()
        return self.model.state_dict()

    def load_model_state(self, state_dict, strict=True):
        """Copy a state_dict into the live parameters (arena views stay where they are) and re-cast the bf16
        operand copies; the collective-free counterpart of `model_state_dict()`."""
        with torch.no_grad():
            own = dict(self.model.state_dict())
            missing = [k for k in own if k not in state_dict]
            unexpected = [k for k in state_dict if k not in own]
            if strict and (missing or unexpected):
                raise KeyError(f"state_dict mismatch: missing {missing}, unexpected {unexpected}")
            for k, v in state_dict.items():
                if k in own:
                    own[k].copy_(v)
        self.refresh_operands()

    def refresh_operands(self):
        """After parameters were written behind the optimizer's back (checkpoint load): re-cast bf16 shadows and
        drop cached fp8 weights."""
        arena = getattr(self.model, "_arena", None)
        if arena is not None and arena.with_shadows:
            arena.refresh_shadows()
        from nanochat_b200 import ops
        if self.model.get_device().type == "cuda" and ops.get_kernel_mode() == "native":
            ops.native_module().bump_weights_epoch()
