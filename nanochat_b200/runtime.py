"""
Execution runtime: CUDA-graph capture of shape-static inner loops and device-side timers.

`decode_graph_for(engine, kv_cache)` returns a `DecodeGraph` that replays one
captured decode step of a `GPT` (positions live in device memory, so replays need
no host-side position), or None when capture does not apply (CPU, non-GPT model,
kernels disabled).
"""

import torch


def decode_graph_for(engine, kv_cache):
    from nanochat_b200.models.gpt import GPT
    model = engine.model
    if not isinstance(model, GPT) or not kv_cache.k_cache.is_cuda:
        return None
    return None  # graph capture is wired in by runtime_graph once the decode kernels are loaded
