"""
Depth-dialed decoder-only transformer, expressed over the fused-op surface in
`nanochat_b200.ops` so the same module runs on the PyTorch reference bodies (CPU)
and on the hand-written sm_100a kernels (B200).

Architecture (reference: nanochat/gpt.py:28-555): rotary position embedding
(half-split, base 1e5), parameter-free RMSNorm, QK-norm with a 1.2 gain on q and
k, untied embedding / lm_head, ReLU^2 MLP (4x), per-layer residual / x0 mixing
scalars, previous-token "smear" gate, mid-depth "backout" subtraction, gated value
embeddings on alternating layers, per-layer sliding windows ("SSSL" pattern, last
layer always long), logits soft-capped at 15, optional GQA.

The module tree and parameter names match the reference's `state_dict` layout
(gpt.py:173-192) so checkpoints load in either code base. What differs is the
execution: the per-layer loop issues a handful of fused ops (mix+norm, fused
rope+qk-norm, flash attention with window tile skipping, add+norm, GEMM with
ReLU^2 epilogue, fused soft-capped cross entropy) instead of dozens of elementwise
kernels produced by a tracing compiler.
"""

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from nanochat_b200 import common
from nanochat_b200 import ops
from nanochat_b200.common import print0
from nanochat_b200.flash_attention import flash_attn
from nanochat_b200.ops import reference as ref_ops


@dataclass
class GPTConfig:
    sequence_len: int = 2048
    vocab_size: int = 32768
    n_layer: int = 12
    n_head: int = 6
    n_kv_head: int = 6
    n_embd: int = 768
    # per-layer window pattern tiled over depth: L = full context, S = quarter context
    window_pattern: str = "SSSL"


def norm(x):
    return ops.rms_norm(x)


def has_ve(layer_idx, n_layer):
    """Value embeddings sit on every other layer, phase chosen so the last layer has one."""
    return layer_idx % 2 == (n_layer - 1) % 2


def apply_rotary_emb(x, cos, sin):
    assert x.ndim == 4
    return ref_ops._rope(x, cos, sin)


class Linear(nn.Linear):
    """Bias-free linear whose fp32 master weight is consumed in the activation dtype.

    On the native path the bf16 operand comes from a shadow copy refreshed when the
    optimizer writes the parameter, not from a per-call cast (reference: gpt.py:45-50).
    """

    def forward(self, x):
        return ops.linear(x, self.weight)


class CausalSelfAttention(nn.Module):
    def __init__(self, config, layer_idx):
        super().__init__()
        self.layer_idx = layer_idx
        self.n_head = config.n_head
        self.n_kv_head = config.n_kv_head
        self.n_embd = config.n_embd
        assert config.n_embd % config.n_head == 0
        assert config.n_kv_head <= config.n_head and config.n_head % config.n_kv_head == 0
        self.head_dim = config.n_embd // config.n_head
        self.c_q = Linear(self.n_embd, self.n_head * self.head_dim, bias=False)
        self.c_k = Linear(self.n_embd, self.n_kv_head * self.head_dim, bias=False)
        self.c_v = Linear(self.n_embd, self.n_kv_head * self.head_dim, bias=False)
        self.c_proj = Linear(self.n_embd, self.n_embd, bias=False)
        self.ve_gate_channels = ref_ops.VE_GATE_CHANNELS
        self.ve_gate = (Linear(self.ve_gate_channels, self.n_kv_head, bias=False)
                        if has_ve(layer_idx, config.n_layer) else None)

    def forward(self, xn, idx, ve_weight, cos_sin, window_size, kv_cache):
        B, T, _ = xn.shape
        q = self.c_q(xn).view(B, T, self.n_head, self.head_dim)
        k = self.c_k(xn).view(B, T, self.n_kv_head, self.head_dim)
        v = self.c_v(xn).view(B, T, self.n_kv_head, self.head_dim)
        if ve_weight is not None:
            v = ops.ve_gate_add(v, xn, self.ve_gate.weight, ve_weight, idx)
        q, k = ops.rope_qknorm(q, k, cos_sin[0], cos_sin[1])
        if kv_cache is None:
            y = flash_attn.flash_attn_func(q, k, v, causal=True, window_size=window_size)
        else:
            k_cache, v_cache = kv_cache.get_layer_cache(self.layer_idx)
            y = flash_attn.flash_attn_with_kvcache(
                q, k_cache, v_cache, k=k, v=v, cache_seqlens=kv_cache.cache_seqlens,
                causal=True, window_size=window_size)
            if self.layer_idx == kv_cache.n_layers - 1:
                kv_cache.advance(T)
        return self.c_proj(y.contiguous().view(B, T, -1))


class MLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.c_fc = Linear(config.n_embd, 4 * config.n_embd, bias=False)
        self.c_proj = Linear(4 * config.n_embd, config.n_embd, bias=False)

    def forward(self, xn):
        # relu(.)^2 rides in the epilogue of the c_fc GEMM on the native path
        if type(self.c_fc) is Linear:
            h = ops.linear_relu2(xn, self.c_fc.weight)
        else:
            h = F.relu(self.c_fc(xn)).square()
        return self.c_proj(h)


class Block(nn.Module):
    def __init__(self, config, layer_idx):
        super().__init__()
        self.attn = CausalSelfAttention(config, layer_idx)
        self.mlp = MLP(config)

    def forward(self, x, xn, idx, ve_weight, cos_sin, window_size, kv_cache):
        """`x` is the mixed residual stream, `xn` its norm; returns the new stream."""
        x, xn = ops.add_norm(x, self.attn(xn, idx, ve_weight, cos_sin, window_size, kv_cache))
        return x + self.mlp(xn)


class GPT(nn.Module):
    def __init__(self, config, pad_vocab_size_to=64):
        """Shapes only: construction may happen under `torch.device('meta')`; values come from
        `init_weights()` (reference: gpt.py:157-201)."""
        super().__init__()
        self.config = config
        self.window_sizes = self._compute_window_sizes(config)
        padded_vocab = -(-config.vocab_size // pad_vocab_size_to) * pad_vocab_size_to
        if padded_vocab != config.vocab_size:
            print0(f"Padding vocab_size from {config.vocab_size} to {padded_vocab} for efficiency")
        self.padded_vocab_size = padded_vocab
        self.transformer = nn.ModuleDict({
            "wte": nn.Embedding(padded_vocab, config.n_embd),
            "h": nn.ModuleList([Block(config, i) for i in range(config.n_layer)]),
        })
        self.lm_head = Linear(config.n_embd, padded_vocab, bias=False)
        self.resid_lambdas = nn.Parameter(torch.ones(config.n_layer))
        self.x0_lambdas = nn.Parameter(torch.zeros(config.n_layer))
        self.smear_gate = Linear(ref_ops.SMEAR_CHANNELS, 1, bias=False)
        self.smear_lambda = nn.Parameter(torch.zeros(1))
        self.backout_lambda = nn.Parameter(0.2 * torch.ones(1))
        head_dim = config.n_embd // config.n_head
        kv_dim = config.n_kv_head * head_dim
        self.value_embeds = nn.ModuleDict({
            str(i): nn.Embedding(padded_vocab, kv_dim)
            for i in range(config.n_layer) if has_ve(i, config.n_layer)})
        # rotary tables cover 10x the training length; decode may run past sequence_len
        self.rotary_seq_len = config.sequence_len * 10
        cos, sin = self._precompute_rotary_embeddings(self.rotary_seq_len, head_dim)
        self.register_buffer("cos", cos, persistent=False)
        self.register_buffer("sin", sin, persistent=False)

    # ------------------------------------------------------------------ init
    @torch.no_grad()
    def init_weights(self):
        """Draws follow the same order and distributions as the reference (gpt.py:203-268),
        so a given torch seed yields the same initial model in both code bases."""
        cfg = self.config
        nn.init.normal_(self.transformer.wte.weight, mean=0.0, std=0.8)
        nn.init.normal_(self.lm_head.weight, mean=0.0, std=0.001)
        bound = 3 ** 0.5 * cfg.n_embd ** -0.5  # uniform with the std of N(0, 1/C)
        for block in self.transformer.h:
            nn.init.uniform_(block.attn.c_q.weight, -bound, bound)
            nn.init.uniform_(block.attn.c_k.weight, -bound, bound)
            nn.init.uniform_(block.attn.c_v.weight, -bound, bound)
            nn.init.zeros_(block.attn.c_proj.weight)
            nn.init.uniform_(block.mlp.c_fc.weight, -0.4 * bound, 0.4 * bound)
            nn.init.zeros_(block.mlp.c_proj.weight)
        L = cfg.n_layer
        span = max(L - 1, 1)
        for i in range(L):
            self.resid_lambdas.data[i] = 1.15 - 0.10 * i / span
        for i in range(L):
            self.x0_lambdas.data[i] = 0.20 - 0.15 * i / span
        nn.init.zeros_(self.smear_lambda)
        nn.init.constant_(self.backout_lambda, 0.2)
        nn.init.uniform_(self.smear_gate.weight, 0.0, 0.02)
        for ve in self.value_embeds.values():
            nn.init.uniform_(ve.weight, -bound, bound)
        for block in self.transformer.h:
            if block.attn.ve_gate is not None:
                nn.init.uniform_(block.attn.ve_gate.weight, 0.0, 0.02)
        head_dim = cfg.n_embd // cfg.n_head
        self.cos, self.sin = self._precompute_rotary_embeddings(self.rotary_seq_len, head_dim)
        # embeddings live in the compute dtype (fp16 keeps fp32: its GradScaler needs fp32 grads)
        if common.COMPUTE_DTYPE != torch.float16:
            self.transformer.wte.to(dtype=common.COMPUTE_DTYPE)
            for ve in self.value_embeds.values():
                ve.to(dtype=common.COMPUTE_DTYPE)

    def _precompute_rotary_embeddings(self, seq_len, head_dim, base=100000, device=None):
        if device is None:
            device = self.transformer.wte.weight.device
        chan = torch.arange(0, head_dim, 2, dtype=torch.float32, device=device)
        inv_freq = 1.0 / (base ** (chan / head_dim))
        t = torch.arange(seq_len, dtype=torch.float32, device=device)
        freqs = torch.outer(t, inv_freq)
        cos = freqs.cos().to(common.COMPUTE_DTYPE)[None, :, None, :]
        sin = freqs.sin().to(common.COMPUTE_DTYPE)[None, :, None, :]
        return cos, sin

    def _compute_window_sizes(self, config):
        """(left, right) per layer: L -> (seq, 0); S -> (ceil(seq/4 to 128), 0); last layer L
        (reference: gpt.py:287-314)."""
        pattern = config.window_pattern.upper()
        assert all(c in "SL" for c in pattern), f"Invalid window_pattern: {pattern}. Use only S and L."
        long_w = config.sequence_len
        short_w = -(-long_w // 4 // 128) * 128
        table = {"L": (long_w, 0), "S": (short_w, 0)}
        sizes = [table[pattern[i % len(pattern)]] for i in range(config.n_layer)]
        sizes[-1] = (long_w, 0)
        return sizes

    def get_device(self):
        return self.transformer.wte.weight.device

    # ------------------------------------------------------- cost accounting
    def num_matmul_params(self):
        return sum(m.weight.numel() for m in self.modules() if isinstance(m, nn.Linear))

    def estimate_flops(self):
        """Training FLOPs per token: 6 per matmul weight + 12*h*d*min(window, T) per layer
        (reference: gpt.py:319-339)."""
        h, d, t = self.config.n_head, self.config.n_embd // self.config.n_head, self.config.sequence_len
        attn = 0
        for left, _ in self.window_sizes:
            attn += 12 * h * d * (t if left < 0 else min(left, t))
        return 6 * self.num_matmul_params() + attn

    def estimate_decode_flops(self, context_len):
        h, d = self.config.n_head, self.config.n_embd // self.config.n_head
        attn = sum(4 * h * d * min(context_len, w) for w, _ in self.window_sizes)
        return 2 * self.num_matmul_params() + attn

    def estimate_prefill_flops(self, num_tokens):
        h, d = self.config.n_head, self.config.n_embd // self.config.n_head
        attn = 0
        for w, _ in self.window_sizes:
            w = min(w, num_tokens)
            attn += 4 * h * d * (w * (w + 1) // 2 + (num_tokens - w) * w)
        return 2 * self.num_matmul_params() * num_tokens + attn

    def kv_bytes_per_token(self):
        d = self.config.n_embd // self.config.n_head
        return self.config.n_layer * 2 * self.config.n_kv_head * d * common.COMPUTE_DTYPE.itemsize

    def kv_read_bytes(self, context_len):
        d = self.config.n_embd // self.config.n_head
        per_tok = 2 * self.config.n_kv_head * d * common.COMPUTE_DTYPE.itemsize
        return sum(per_tok * min(context_len, w) for w, _ in self.window_sizes)

    def num_scaling_params(self):
        wte = sum(p.numel() for p in self.transformer.wte.parameters())
        value_embeds = sum(p.numel() for p in self.value_embeds.parameters())
        lm_head = sum(p.numel() for p in self.lm_head.parameters())
        matrices = sum(p.numel() for p in self.transformer.h.parameters())
        scalars = (self.resid_lambdas.numel() + self.x0_lambdas.numel() + self.smear_gate.weight.numel()
                   + self.smear_lambda.numel() + self.backout_lambda.numel())
        total = wte + value_embeds + lm_head + matrices + scalars
        assert total == sum(p.numel() for p in self.parameters()), "Parameter count mismatch"
        return {"wte": wte, "value_embeds": value_embeds, "lm_head": lm_head,
                "transformer_matrices": matrices, "scalars": scalars, "total": total}

    # -------------------------------------------------------------- optimizer
    def setup_optimizer(self, unembedding_lr=0.004, embedding_lr=0.2, matrix_lr=0.02, weight_decay=0.0,
                        scalar_lr=0.5, comm=None):
        """Group layout and hyper-parameters of reference gpt.py:419-457; group order fixes the
        parameter indices of the optimizer checkpoint."""
        from nanochat_b200.optim import MuonAdamW
        matrix_params = list(self.transformer.h.parameters())
        ve_params = list(self.value_embeds.parameters())
        emb_params = list(self.transformer.wte.parameters())
        head_params = list(self.lm_head.parameters())
        smear_params = [self.smear_gate.weight, self.smear_lambda, self.backout_lambda]
        n_all = (len(matrix_params) + len(ve_params) + len(emb_params) + len(head_params) + 2 + len(smear_params))
        assert len(list(self.parameters())) == n_all
        s = (self.config.n_embd / 768) ** -0.5
        print0(f"Scaling the LR for the AdamW parameters ∝1/√({self.config.n_embd}/768) = {s:.6f}")
        adam = dict(kind="adamw", eps=1e-10)
        groups = [
            dict(adam, params=head_params, lr=unembedding_lr * s, betas=(0.8, 0.96), weight_decay=0.01),
            dict(adam, params=emb_params, lr=embedding_lr * s, betas=(0.8, 0.995), weight_decay=0.001),
            dict(adam, params=ve_params, lr=embedding_lr * s * 0.5, betas=(0.8, 0.995), weight_decay=0.01),
            dict(adam, params=[self.resid_lambdas], lr=scalar_lr * 0.01, betas=(0.8, 0.95), weight_decay=0.05),
            dict(adam, params=[self.x0_lambdas], lr=scalar_lr, betas=(0.96, 0.95), weight_decay=0.0),
            dict(adam, params=smear_params, lr=0.2, betas=(0.8, 0.95), weight_decay=0.0),
        ]
        for shape in sorted({p.shape for p in matrix_params}):
            groups.append(dict(kind="muon", params=[p for p in matrix_params if p.shape == shape],
                               lr=matrix_lr, momentum=0.95, ns_steps=5, beta2=0.9, weight_decay=weight_decay))
        optimizer = MuonAdamW(groups, comm=comm)
        for g in optimizer.param_groups:
            g["initial_lr"] = g["lr"]
        return optimizer

    # ---------------------------------------------------------------- forward
    def _embed(self, idx, kv_cache):
        """Embedding + norm + smear for the three regimes of reference gpt.py:471-492."""
        wte = self.transformer.wte.weight
        T = idx.size(1)
        if kv_cache is None:
            assert T > 1, "Training forward pass should have T > 1"
            x, _ = ops.embed_norm_smear(idx, wte, self.smear_gate.weight, self.smear_lambda,
                                        common.COMPUTE_DTYPE)
            return x
        prev = kv_cache.prev_embedding
        if T > 1:
            x, last = ops.embed_norm_smear(idx, wte, self.smear_gate.weight, self.smear_lambda,
                                           common.COMPUTE_DTYPE)
            kv_cache.prev_embedding = last
            return x
        x = norm(F.embedding(idx, wte).to(common.COMPUTE_DTYPE))
        kv_cache.prev_embedding = x[:, -1:, :]
        if prev is not None:
            gate = self.smear_lambda.to(x.dtype) * torch.sigmoid(
                F.linear(x[:, :, :ref_ops.SMEAR_CHANNELS], self.smear_gate.weight.to(x.dtype)))
            x = x + gate * prev
        return x

    def forward(self, idx, targets=None, kv_cache=None, loss_reduction="mean"):
        B, T = idx.size()
        assert T <= self.cos.size(1), f"Sequence length grew beyond the rotary embeddings cache: {T} > {self.cos.size(1)}"
        assert idx.device == self.cos.device, f"Rotary embeddings and idx are on different devices: {idx.device} != {self.cos.device}"
        assert self.cos.dtype == common.COMPUTE_DTYPE, f"Rotary embeddings must be in {common.COMPUTE_DTYPE}, got {self.cos.dtype}"
        T0 = 0 if kv_cache is None else kv_cache.get_pos()
        cos_sin = self.cos[:, T0:T0 + T], self.sin[:, T0:T0 + T]

        if (kv_cache is None and common.COMPUTE_DTYPE == torch.bfloat16 and ops.use_native(self.transformer.wte.weight)
                and not getattr(self, "_fp8_module_path", False)):
            return self._forward_native(idx, targets, cos_sin, loss_reduction)

        if (kv_cache is not None and T > 1 and T0 == 0 and kv_cache.prev_embedding is None
                and not torch.is_grad_enabled() and common.COMPUTE_DTYPE == torch.bfloat16
                and self.config.n_embd // self.config.n_head == 128 and T <= kv_cache.max_seq_len
                and ops.use_native(self.transformer.wte.weight)):
            return self._prefill_native(idx, cos_sin, kv_cache)

        x = self._embed(idx, kv_cache)
        x0 = x
        backout_layer = self.config.n_layer // 2
        x_backout = None
        for i, block in enumerate(self.transformer.h):
            x, xn = ops.resid_mix_norm(x, x0, self.resid_lambdas, self.x0_lambdas, i)
            ve_w = self.value_embeds[str(i)].weight if str(i) in self.value_embeds else None
            x = block(x, xn, idx, ve_w, cos_sin, self.window_sizes[i], kv_cache)
            if i == backout_layer:
                x_backout = x
        x = ops.backout_norm(x, x_backout, self.backout_lambda)

        if targets is not None:
            loss = ops.softcap_cross_entropy(x, self.lm_head.weight, targets, self.config.vocab_size,
                                             reduction=loss_reduction)
            if loss_reduction == "none":
                loss = loss.view(-1)
            return loss
        return ops.softcap_logits(x, self.lm_head.weight, self.config.vocab_size)

    def _forward_native(self, idx, targets, cos_sin, loss_reduction):
        """Whole-sequence forward on the sm_100a kernels: one fused autograd node per layer."""
        nat = ops.native_module()
        assert idx.size(1) > 1, "Training forward pass should have T > 1"
        if idx.dtype != torch.long:          # the SFT loader yields int32 inputs (reference: scripts/chat_sft.py); the
            idx = idx.long()                 # gather kernels index with 64-bit ids
        if targets is not None and targets.dtype != torch.long:
            targets = targets.long()
        if nat.fp8_enabled():
            nat.begin_microstep(idx.device)
        x, _ = nat.embed_norm_smear(idx, self.transformer.wte.weight, self.smear_gate.weight, self.smear_lambda)
        x0 = x
        backout_layer = self.config.n_layer // 2
        x_backout = None
        for i, block in enumerate(self.transformer.h):
            ve_w = self.value_embeds[str(i)].weight if str(i) in self.value_embeds else None
            x = nat.layer_forward(block, x, x0, idx, ve_w, cos_sin, self.window_sizes[i],
                                  self.resid_lambdas, self.x0_lambdas, i)
            if i == backout_layer:
                x_backout = x
        if targets is not None:
            loss = nat.head_loss(x, x_backout, self.backout_lambda, self.lm_head.weight, targets,
                                 self.config.vocab_size, loss_reduction)
            return loss.view(-1) if loss_reduction == "none" else loss
        x = ops.backout_norm(x, x_backout, self.backout_lambda)
        return nat.softcap_logits(x, self.lm_head.weight, self.config.vocab_size)

    def _prefill_native(self, idx, cos_sin, kv_cache):
        """Prompt into an empty cache on the fused per-layer path of training (one QKV GEMM, rotary / QK-norm / VE
        gate in place, the whole-sequence attention kernel), each layer's keys and values copied into its cache.
        The op-by-op cached forward launches about twice as many kernels and is bound by their launch cost."""
        nat = ops.native_module()
        T = idx.size(1)
        x, last = nat.embed_norm_smear(idx, self.transformer.wte.weight, self.smear_gate.weight, self.smear_lambda)
        kv_cache.prev_embedding = last
        x0 = x
        backout_layer = self.config.n_layer // 2
        x_backout = None
        for i, block in enumerate(self.transformer.h):
            ve_w = self.value_embeds[str(i)].weight if str(i) in self.value_embeds else None
            x = nat.layer_forward(block, x, x0, idx, ve_w, cos_sin, self.window_sizes[i],
                                  self.resid_lambdas, self.x0_lambdas, i, kv_sink=kv_cache.get_layer_cache(i))
            if i == backout_layer:
                x_backout = x
        kv_cache.advance(T)
        x = ops.backout_norm(x, x_backout, self.backout_lambda)
        return nat.softcap_logits(x, self.lm_head.weight, self.config.vocab_size)

    @torch.inference_mode()
    def generate(self, tokens, max_tokens, temperature=1.0, top_k=None, seed=42):
        """Naive batch-1 streaming sampler that recomputes the whole prefix per token; the
        Engine must agree with it token for token at temperature 0 (reference: gpt.py:526-555)."""
        assert isinstance(tokens, list)
        device = self.get_device()
        rng = None
        if temperature > 0:
            rng = torch.Generator(device=device)
            rng.manual_seed(seed)
        ids = torch.tensor([tokens], dtype=torch.long, device=device)
        for _ in range(max_tokens):
            logits = self.forward(ids)[:, -1, :]
            if top_k is not None and top_k > 0:
                kth, _ = torch.topk(logits, min(top_k, logits.size(-1)))
                logits[logits < kth[:, [-1]]] = -float("inf")
            if temperature > 0:
                probs = F.softmax(logits / temperature, dim=-1)
                nxt = torch.multinomial(probs, num_samples=1, generator=rng)
            else:
                nxt = torch.argmax(logits, dim=-1, keepdim=True)
            ids = torch.cat((ids, nxt), dim=1)
            yield nxt.item()
