"""
One optimizer step as a callable: gradient accumulation over micro-batches, the sharded
MuonAdamW update, gradient reset. This is the loop body of the pretraining / SFT drivers
(reference: scripts/base_train.py:510-540) packaged so benchmarks and scripts share it.
"""

import torch


class TrainStep:
    def __init__(self, model, grad_accum=1, comm=None, optimizer=None, **optimizer_kwargs):
        self.model = model
        self.grad_accum = grad_accum
        self.optimizer = optimizer if optimizer is not None else model.setup_optimizer(comm=comm, **optimizer_kwargs)

    def step(self, fetch, loss_scale=None):
        """`fetch(i)` returns the (inputs, targets) of micro-batch i. Returns the last micro-batch loss
        (detached, on device)."""
        scale = (1.0 / self.grad_accum) if loss_scale is None else loss_scale
        loss = None
        for i in range(self.grad_accum):
            x, y = fetch(i)
            loss = self.model(x, y)
            (loss * scale).backward()
        self.optimizer.step()
        # dropping the buffers lets the first wgrad of the next step write instead of read-modify-write
        self.model.zero_grad(set_to_none=True)
        return loss.detach()
