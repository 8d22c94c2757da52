"""
One optimizer step as a callable: gradient accumulation over micro-batches, the sharded
MuonAdamW update, gradient reset. This is the loop body of the pretraining / SFT drivers
(reference: scripts/base_train.py:510-540) packaged so benchmarks and scripts share it.
"""

from nanochat_b200.utils.trace import PhaseTimers


class TrainStep:
    def __init__(self, model, grad_accum=1, comm=None, optimizer=None, use_arena=None, timers=None,
                 **optimizer_kwargs):
        self.model = model
        # phase timers are inert (no events, no extra launches) unless NANOCHAT_TRACE=1 or one is passed in
        self.timers = timers if timers is not None else PhaseTimers(device_type=model.get_device().type)
        if use_arena is None:
            use_arena = model.get_device().type == "cuda"
        if use_arena and getattr(model, "_arena", None) is None:
            from nanochat_b200.parallel.arena import ParamArena
            ParamArena(model)
        self.grad_accum = grad_accum
        self.optimizer = optimizer if optimizer is not None else model.setup_optimizer(comm=comm, **optimizer_kwargs)

    def step(self, fetch, loss_scale=None):
        """`fetch(i)` returns the (inputs, targets) of micro-batch i. Returns the last micro-batch loss
        (detached, on device)."""
        scale = (1.0 / self.grad_accum) if loss_scale is None else loss_scale
        loss = None
        for i in range(self.grad_accum):
            x, y = fetch(i)
            with self.timers.phase("forward"):
                loss = self.model(x, y)
            with self.timers.phase("backward"):
                (loss * scale).backward()
        with self.timers.phase("optimizer"):
            self.optimizer.step()
        arena = getattr(self.model, "_arena", None)
        if arena is not None:
            arena.zero_grads()      # persistent gradient buffers: re-arm "first write overwrites"
        else:
            # dropping the buffers lets the first wgrad of the next step write instead of read-modify-write
            self.model.zero_grad(set_to_none=True)
        return loss.detach()
