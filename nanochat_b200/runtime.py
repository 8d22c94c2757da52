"""
Execution runtime: CUDA-graph replay of the single-token decode step.

A decode step of the reference engine is one `model.forward` on a (B, 1) batch: a few hundred
small library kernels whose launch cost, not their work, sets the token rate
(reference: nanochat/engine.py:186-190). Here the step is a fixed sequence of purpose-built
kernels (`ops/csrc/decode.cu`: weight-streaming GEMV with fused residual / relu^2, rotary +
QK-norm + value-embedding gate + cache append, split-key attention) over static buffers. Every
position-dependent quantity is read from device memory (`KVCache.cache_seqlens`), so the whole
step is captured once per (engine, cache) and replayed with a single launch per token.

`decode_graph_for(engine, kv_cache)` returns the `DecodeGraph` of a cache, or None when the
fast path does not apply (CPU, kernels disabled, more than 64 rows, head dim != 128).
"""

import os

import torch

from nanochat_b200 import common, ops
from nanochat_b200.ops import reference as ref_ops

LM_HEAD_PREFETCH_ROWS = 16384     # rows of lm_head (54 MB at 1664 wide) the last layer prefetches: what L2 can hold
MAX_ROWS = 64          # rows of one decode graph; up to GEMV_ROWS of them use the weight-streaming GEMV
GEMV_ROWS = 8
# Up to this many rows the layer's mix + norm is folded into the QKV GEMV (one launch fewer per layer). Every CTA of
# that GEMV redoes the mix for its rows, which is free while the kernel waits on memory (few rows) and costs more
# than the launch it saves once the rows make it arithmetic-bound. Measured on d26: 1 row +4.8 %, 2 rows +2 %,
# 4 rows -5 %, 8 rows -4 % tokens per second.
FOLD_MIX_ROWS = int(os.environ.get("NANOCHAT_DECODE_FOLD_ROWS", "2"))
# every GEMV of the step prefetches the next kernel's weight matrix into L2 (NANOCHAT_DECODE_PREFETCH=0: off, A/B runs)
PREFETCH_NEXT = os.environ.get("NANOCHAT_DECODE_PREFETCH", "1") != "0"


class DecodeGraph:
    def __init__(self, model, kv_cache):
        nat = ops.native_module()
        self.nat, self.C_ = nat, nat._C
        self.model, self.cache = model, kv_cache
        cfg = model.config
        dev = kv_cache.cache_seqlens.device
        self.paged = getattr(kv_cache, "paged", False)
        self.pool_version = getattr(kv_cache, "pool_version", 0)
        B, C = kv_cache.batch_size, cfg.n_embd
        self.B, self.C = B, C
        self.H, self.Hkv = cfg.n_head, cfg.n_kv_head
        nq, nkv = self.H * 128, self.Hkv * 128
        bf16 = torch.bfloat16
        e = lambda *shape, dtype=bf16: torch.empty(*shape, dtype=dtype, device=dev)
        self.ids = torch.zeros(B, 1, dtype=torch.long, device=dev)
        self.prev = torch.zeros(B, C, dtype=bf16, device=dev)
        self.xm, self.xn, self.xa, self.xn2 = e(B, C), e(B, C), e(B, C), e(B, C)
        self.xs = [e(B, C), e(B, C)]                       # residual stream ping-pong
        self.x_in = e(B, C)                                # embedding + smear: the stream's input and the x0 of every layer
        self.x_backout = e(B, C)
        self.qkv, self.y, self.h = e(B, nq + 2 * nkv), e(B, nq), e(B, 4 * C)
        self.logits_bf16 = e(B, model.lm_head.weight.shape[0])
        self.logits = e(B, cfg.vocab_size, dtype=torch.float32)
        self.scratch = torch.zeros(self.C_.decode_attn_scratch(B, self.H), dtype=torch.float32, device=dev)
        self.cos = model.cos.reshape(-1, 64).contiguous()
        self.sin = model.sin.reshape(-1, 64).contiguous()
        self.use_gemv = B <= GEMV_ROWS     # more rows: the tcgen05 GEMM (rows padded to a 128-row tile) inside the graph
        self.weights_epoch = None
        self.w = None
        self.graph = None
        self.warm = False

    # ------------------------------------------------------------------ weights
    def _refresh_weights(self):
        """bf16 operand copies laid out for the step (fused QKV); re-copied in place when the parameters moved,
        so a captured graph keeps pointing at valid buffers."""
        nat = self.nat
        m = self.model
        fresh = []
        for blk in m.transformer.h:
            a = blk.attn
            fresh.append(dict(
                qkv=[nat.shadow_of(a.c_q.weight), nat.shadow_of(a.c_k.weight), nat.shadow_of(a.c_v.weight)],
                o=nat.shadow_of(a.c_proj.weight), fc=nat.shadow_of(blk.mlp.c_fc.weight),
                pr=nat.shadow_of(blk.mlp.c_proj.weight),
                wg=a.ve_gate.weight if a.ve_gate is not None else None))
        lm_head = nat.shadow_of(m.lm_head.weight)
        epoch = nat._weights_epoch            # read after the shadows: a re-cast above moves it
        if self.w is not None and self.weights_epoch == epoch:
            return
        first = self.w is None
        if first:
            self.w = []
        for i, f in enumerate(fresh):
            if first:
                self.w.append(dict(qkv=torch.cat(f["qkv"]).contiguous(),
                                   wg=f["wg"].detach().float().contiguous() if f["wg"] is not None else None))
            else:
                torch.cat(f["qkv"], out=self.w[i]["qkv"])
                if f["wg"] is not None:
                    self.w[i]["wg"].copy_(f["wg"].detach().float())
            # the other matrices are used where they live (bf16 parameters or their persistent shadows)
            self.w[i].update(o=f["o"], fc=f["fc"], pr=f["pr"])
        self.lm_head = lm_head
        self.weights_epoch = epoch
        # tensors the step reads where they live: if any of them was re-homed since the capture (a parameter arena
        # built later, a checkpoint loaded with assign=True) the captured addresses are stale and the graph is dropped
        where = tuple(t.data_ptr() for w in self.w for t in (w["o"], w["fc"], w["pr"])) + (
            lm_head.data_ptr(), m.transformer.wte.weight.data_ptr(),
            *[ve.weight.data_ptr() for ve in m.value_embeds.values()])
        if where != getattr(self, "_captured_where", where):
            self.graph, self.warm = None, False
        self._captured_where = where

    # --------------------------------------------------------------------- step
    def _linear(self, x, w, out, aux=None, relu2=False, norm_input=False, next_w=None):
        """out = epi(norm?(x) @ w^T) (+ aux): GEMV for a few rows, tensor-core GEMM otherwise. `next_w`: the weight
        matrix the following kernel will stream; the GEMV's CTAs prefetch it into L2 (decode is latency-bound per
        kernel, so keeping HBM busy across kernel boundaries is what raises the weight-streaming rate)."""
        if self.use_gemv:
            self.C_.gemv_rows(x, w, out, aux, 1 if relu2 else 0, norm_input, next_w if PREFETCH_NEXT else None)
            return
        nat = self.nat
        if norm_input:
            self.C_.norm_fwd(x, self.xn2, None)
            x = self.xn2
        nat.gemm(x, w, out, aux=aux, beta=1.0 if aux is not None else 0.0,
                 epi=nat.EPI_RELU2 if relu2 else nat.EPI_LINEAR)

    def _forward(self):
        m, C_ = self.model, self.C_
        B, H, Hkv = self.B, self.H, self.Hkv
        nq = H * 128
        cache = self.cache
        idx = self.ids[:, 0]
        # embedding gather, norm, smear with the previous token's embedding and the update of that state: one kernel
        C_.decode_embed(self.ids, m.transformer.wte.weight, m.smear_gate.weight.detach().float().contiguous().view(-1),
                        m.smear_lambda.detach().float().view(1), self.prev, self.x_in)
        x0 = x = self.x_in
        backout_layer = m.config.n_layer // 2
        scale = 1.0 / (128 ** 0.5)
        for i, w in enumerate(self.w):
            # what the kernel after this layer's last GEMV streams: the next layer's QKV weights, or the head of lm_head
            after = self.w[i + 1]["qkv"] if i + 1 < len(self.w) else self.lm_head[:LM_HEAD_PREFETCH_ROWS]
            if self.use_gemv and B <= FOLD_MIX_ROWS:
                # mix + norm folded into the QKV GEMV; its first CTA writes xm and the gate's slice of xn
                C_.gemv_rows_mix(x, x0, m.resid_lambdas, m.x0_lambdas, i, w["qkv"], self.qkv, self.xm, self.xn,
                                 w["o"] if PREFETCH_NEXT else None)
            else:
                C_.mixnorm_fwd(x, x0, m.resid_lambdas, m.x0_lambdas, i, self.xm, self.xn, None)
                self._linear(self.xn, w["qkv"], self.qkv, next_w=w["o"])
            ve = m.value_embeds[str(i)].weight if str(i) in m.value_embeds else None
            kc, vc = cache.get_layer_cache(i)
            # a paged cache: one layer's page pools + the rows' page table; the row capacity bounds the append
            table = cache.table if self.paged else None
            t_max = cache.max_seq_len if self.paged else 0
            C_.decode_qkv_post(self.qkv, H, Hkv, self.cos, self.sin, cache.cache_seqlens,
                               self.xn if ve is not None else None, w["wg"] if ve is not None else None, ve,
                               idx if ve is not None else None, kc, vc, table, t_max)
            window = m.window_sizes[i][0]
            window = window if 0 <= window < cache.max_seq_len else -1
            C_.decode_attn(self.qkv[:, :nq], kc, vc, cache.cache_seqlens, H, Hkv, window, scale, self.scratch, self.y,
                           table)
            self._linear(self.y, w["o"], self.xa, aux=self.xm, next_w=w["fc"])
            self._linear(self.xa, w["fc"], self.h, relu2=True, norm_input=True, next_w=w["pr"])   # GEMV: norm(xa) folded in
            out = self.x_backout if i == backout_layer else self.xs[i & 1]
            self._linear(self.h, w["pr"], out, aux=self.xa, next_w=after)
            x = out
        C_.backout_norm_fwd(x, self.x_backout, m.backout_lambda.detach().float(), self.xn)
        self._linear(self.xn, self.lm_head, self.logits_bf16)
        C_.softcap_logits(self.logits_bf16, self.logits, m.config.vocab_size, ref_ops.SOFTCAP)
        cache.cache_seqlens.add_(1)

    def begin(self):
        """Start of a generation: take over the smear state the prefill left in the cache."""
        prev = self.cache.prev_embedding
        if prev is None:
            self.prev.zero_()
        else:
            self.prev.copy_(prev.reshape(self.B, self.C))
        self._refresh_weights()

    @torch.inference_mode()
    def step(self, ids):
        """ids: (B, 1) token ids of the new position; returns (B, V) fp32 logits (a static buffer, valid until
        the next step)."""
        self.ids.copy_(ids)
        if self.weights_epoch != self.nat._weights_epoch or self.w is None:
            self._refresh_weights()
        if self.graph is not None:
            self.graph.replay()
        elif not self.warm:
            self._forward()                      # first step runs eagerly: kernels get configured outside capture
            self.warm = True
        else:
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._forward()
            self.graph = g
            g.replay()
        self.cache._pos += 1
        return self.logits


def graph_path_applies(model, rows):
    """True when `rows` sample rows of this model decode through the captured-graph kernels."""
    from nanochat_b200.models.gpt import GPT
    if not isinstance(model, GPT) or ops.get_kernel_mode() != "native":
        return False
    cfg = model.config
    wte = model.transformer.wte.weight
    return (wte.is_cuda and cfg.n_embd // cfg.n_head == 128 and rows <= MAX_ROWS and cfg.n_embd % 8 == 0
            and common.COMPUTE_DTYPE == torch.bfloat16 and wte.dtype == torch.bfloat16)


def decode_graph_for(engine, kv_cache):
    """The DecodeGraph bound to `kv_cache` (created on first use), or None when the fast path does not apply."""
    model = engine.model
    if (not getattr(kv_cache, "pooled", False) or not kv_cache.cache_seqlens.is_cuda
            or not graph_path_applies(model, kv_cache.batch_size)):
        return None
    graphs = engine._decode_graphs
    g = graphs.get(id(kv_cache))
    if g is None or g.cache is not kv_cache or g.pool_version != getattr(kv_cache, "pool_version", 0):
        g = DecodeGraph(model, kv_cache)       # first use, or the page pool moved: capture on the new addresses
        graphs[id(kv_cache)] = g
    return g
