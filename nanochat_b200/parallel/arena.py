"""
Parameter arena: the model's large tensors re-homed into a few contiguous buffers.

For every Muon shape group (all (C,C) matrices, all (4C,C) matrices, ...) the arena owns
  master  (K, r, c) fp32   the parameters themselves (`p.data` become views of it)
  shadow  (K, r, c) bf16   the GEMM operands (registered with `ops.native` as the weights' shadows)
  grad    (K, r, c) fp32   `p.grad` views; written by the wgrad GEMM epilogues
and for the large AdamW tensors (lm_head, wte, value embeddings) a gradient accumulator (and a
bf16 shadow for fp32 masters). Consequences:
  * the optimizer sees each Muon group as ONE stacked tensor without copying (no torch.stack of
    gradients, no copy-back of parameters: reference optim.py:300-312,426 become no-ops);
  * q, k and v of a layer are adjacent rows of the (C,C) stack, so the layer runs one fused QKV
    GEMM forward, one dgrad and one wgrad instead of three each;
  * gradients are persistent buffers: `zero_grads()` only re-arms a per-parameter "first write
    overwrites" flag (and clears the small atomically-accumulated buffers) instead of
    re-allocating or memsetting gigabytes every step;
  * with a symmetric allocator (parallel/symm.py) every rank has the same layout at the same
    offsets, which is what the peer-to-peer optimizer kernels address.

`state_dict()` is unaffected (it walks parameters), so checkpoints keep the reference layout.
"""

import torch


def _default_alloc(shape, dtype, device, role="master"):
    """role: 'master' (fp32 parameters), 'grad' (fp32 accumulators), 'shadow' (bf16 GEMM operands),
    'table' (bf16 embedding tables). A symmetric allocator places grad/shadow/table in peer-mapped pools."""
    return torch.empty(shape, dtype=dtype, device=device)


class ParamArena:
    def __init__(self, model, alloc=None, with_shadows=None):
        alloc = alloc or _default_alloc
        self.model = model
        dev = model.get_device()
        self.device = dev
        if with_shadows is None:
            with_shadows = dev.type == "cuda"
        self.with_shadows = with_shadows
        self.muon_groups = []      # dicts: shape, params, master, shadow, grad
        self.adamw_big = []        # dicts: param, grad (fp32), shadow (or None)
        self.small = []            # small fp32 params with ordinary grads
        matrix_params = list(model.transformer.h.parameters())
        for shape in sorted({p.shape for p in matrix_params}):
            ps = [p for p in matrix_params if p.shape == shape]
            K = len(ps)
            master = alloc((K, *shape), ps[0].dtype, dev, "master")
            grad = alloc((K, *shape), torch.float32, dev, "grad")
            shadow = (alloc((K, *shape), torch.bfloat16, dev, "shadow")
                      if (with_shadows and ps[0].dtype == torch.float32) else None)
            with torch.no_grad():
                for j, p in enumerate(ps):
                    master[j].copy_(p.data)
                    p.data = master[j]
                if shadow is not None:
                    shadow.copy_(master)
            self.muon_groups.append(dict(shape=tuple(shape), params=ps, master=master, shadow=shadow, grad=grad))
        big = [model.lm_head.weight, model.transformer.wte.weight] + [ve.weight for ve in model.value_embeds.values()]
        for p in big:
            grad = alloc(tuple(p.shape), torch.float32, dev, "grad")
            shadow = None
            if p.dtype == torch.float32:
                store = alloc(tuple(p.shape), p.dtype, dev, "master")
                with torch.no_grad():
                    store.copy_(p.data)
                    p.data = store
                if with_shadows:
                    shadow = alloc(tuple(p.shape), torch.bfloat16, dev, "shadow")
                    with torch.no_grad():
                        shadow.copy_(p.data)
            else:
                store = alloc(tuple(p.shape), p.dtype, dev, "table")
                with torch.no_grad():
                    store.copy_(p.data)
                    p.data = store
            p._arena = True
            self.adamw_big.append(dict(param=p, grad=grad, shadow=shadow))
        seen = {id(p) for g in self.muon_groups for p in g["params"]} | {id(d["param"]) for d in self.adamw_big}
        self.small = [p for p in model.parameters() if id(p) not in seen]
        self.small_grads = {}
        for p in self.small:     # scalars and the smear gate: fp32 gradients in the same pool as the others
            self.small_grads[id(p)] = alloc(tuple(p.shape), torch.float32, dev, "grad")
        self._register_shadows()
        self.bind_grads()
        model._arena = self

    def _register_shadows(self):
        if not self.with_shadows:
            return
        from nanochat_b200 import ops
        table = ops.native_module()._shadow
        for g in self.muon_groups:
            if g["shadow"] is not None:
                for j, p in enumerate(g["params"]):
                    table.set(p, p._version, g["shadow"][j])
        for d in self.adamw_big:
            if d["shadow"] is not None:
                table.set(d["param"], d["param"]._version, d["shadow"])

    def bind_grads(self):
        """Point every parameter's gradient at its arena slot and arm the first-write flags."""
        for g in self.muon_groups:
            for j, p in enumerate(g["params"]):
                p.grad = g["grad"][j]
        for d in self.adamw_big:
            p = d["param"]
            if p.dtype == torch.float32:
                p.grad = d["grad"]
            else:
                p.grad32 = d["grad"]     # fp32 accumulator of a bf16 table (see ops.native._grad_buffer)
                p.grad = None
        for p in self.small:
            p.grad = self.small_grads[id(p)]
        self.zero_grads()

    @torch.no_grad()
    def zero_grads(self):
        from nanochat_b200 import ops
        if self.device.type != "cuda" or ops.get_kernel_mode() != "native":
            # autograd accumulates into the bound views: they must start from zero
            for g in self.muon_groups:
                g["grad"].zero_()
            for d in self.adamw_big:
                d["grad"].zero_()
            for p in self.small:
                if p.grad is not None:
                    p.grad.zero_()
            return
        for g in self.muon_groups:
            for p in g["params"]:
                if p.shape[-1] % 8 == 0 and p.shape[0] % 8 == 0:
                    p._grad_fresh = True          # next wgrad GEMM overwrites
                else:
                    p.grad.zero_()                # tiny matrices accumulate atomically
        for d in self.adamw_big:
            p = d["param"]
            if p.dtype == torch.float32:
                p._grad_fresh = True
            else:
                d["grad"].zero_()                 # scatter-added embedding gradients need a zero base
        for p in self.small:
            if p.grad is not None:
                p.grad.zero_()

    def refresh_shadows(self):
        """Re-cast every shadow from its master (after a checkpoint load or a master sync)."""
        with torch.no_grad():
            for g in self.muon_groups:
                if g["shadow"] is not None:
                    g["shadow"].copy_(g["master"])
            for d in self.adamw_big:
                if d["shadow"] is not None:
                    d["shadow"].copy_(d["param"].data)
        self._register_shadows()
