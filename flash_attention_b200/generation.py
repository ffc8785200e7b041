"""The decode caller path: what sits between a model's attention layer and flash_attn_with_kvcache while
generating.

Covers, for this one path, what the reference spreads over three places:
  - the per-layer KV cache and its bookkeeping: InferenceParams (flash_attn/utils/generation.py:19-36) and
    _update_kv_cache (flash_attn/modules/mha.py:296-322);
  - the attention core of an MHA layer during generation: prefill writes the cache and runs the training
    kernel, every later step is ONE fused call that rotates q and the new k, appends k / v to the cache and
    attends (MHA._update_kvcache_attention / _apply_rotary_update_kvcache_attention, mha.py:442-507);
  - capture of a decode step in a CUDA graph and its replay with new inputs (update_graph_cache /
    capture_graph, generation.py:604-737).

InferenceParams keeps the reference's field names, so the reference's own modules can be driven with it and
this module's layer with theirs.  Nothing here launches a kernel of its own: the work is the C ABI's.
"""
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, Optional, Sequence, Tuple

import torch

from flash_attention_b200.flash_attn_interface import flash_attn_kvpacked_func, flash_attn_with_kvcache
from flash_attention_b200.layers.rotary import RotaryEmbedding


@dataclass
class InferenceParams:
    """State of one generation: cache capacity, how far every sequence has come, one cache tensor per layer.

    key_value_memory_dict[layer_idx]: (max_batch_size, max_seqlen, 2, nheads_k, head_dim), K at [:, :, 0].
    seqlen_offset: tokens already in the cache when all sequences move in step (0 = prefill).
    lengths_per_sample: (max_batch_size,) int32 on the device, per-sequence lengths; when set it takes the
        place of seqlen_offset in the fused step (and is what a captured graph reads, so that one graph serves
        every position)."""

    max_seqlen: int
    max_batch_size: int
    seqlen_offset: int = 0
    batch_size_offset: int = 0
    key_value_memory_dict: Dict[int, torch.Tensor] = field(default_factory=dict)
    lengths_per_sample: Optional[torch.Tensor] = None

    def reset(self, max_seqlen, max_batch_size):
        self.max_seqlen, self.max_batch_size, self.seqlen_offset = max_seqlen, max_batch_size, 0
        if self.lengths_per_sample is not None:
            self.lengths_per_sample.zero_()

    def allocate(self, layers: Sequence[int], nheads_k: int, head_dim: int, dtype, device):
        """One cache per layer, up front: a decode step must not allocate (it may be inside a graph)."""
        shape = (self.max_batch_size, self.max_seqlen, 2, nheads_k, head_dim)
        for i in layers:
            self.key_value_memory_dict[i] = torch.empty(shape, dtype=dtype, device=device)
        return self

    def cache_seqlens(self, batch: int):
        return self.seqlen_offset if self.lengths_per_sample is None else self.lengths_per_sample[:batch]


def update_kv_cache(kv: torch.Tensor, inference_params: InferenceParams, layer_idx: int) -> torch.Tensor:
    """Stores kv (batch, seqlen, 2, nheads_k, head_dim) at rows [seqlen_offset, seqlen_offset + seqlen) of the
    layer's cache (created on first use) and returns the cache of these sequences up to the last row written."""
    cache = inference_params.key_value_memory_dict.get(layer_idx)
    if cache is None:
        inference_params.allocate([layer_idx], kv.shape[3], kv.shape[4], kv.dtype, kv.device)
        cache = inference_params.key_value_memory_dict[layer_idx]
    b0, s0 = inference_params.batch_size_offset, inference_params.seqlen_offset
    b1, s1 = b0 + kv.shape[0], s0 + kv.shape[1]
    if b1 > cache.shape[0] or s1 > cache.shape[1]:
        raise ValueError(f"KV cache of layer {layer_idx} holds {cache.shape[0]} x {cache.shape[1]} rows, "
                         f"asked to write up to {b1} x {s1}")
    cache[b0:b1, s0:s1].copy_(kv)
    return cache[b0:b1, :s1]


class CachedSelfAttention(torch.nn.Module):
    """Attention core of one decoder layer while generating.

    forward(q, kv, inference_params) with q (batch, seqlen, nheads, head_dim) and kv (batch, seqlen, 2,
    nheads_k, head_dim), both fresh from the projections, returns the context (batch, seqlen, nheads, head_dim).
    Prefill (inference_params.seqlen_offset == 0): rotary on q and k in place, kv stored, causal attention
    with the training kernel.  Afterwards: one fused call per step (rotary at the cache positions, append,
    attention over the cache).  rotary_dim 0 switches the embedding off; the fused step needs rotary_dim % 16
    == 0, other values rotate with the stand-alone op first."""

    def __init__(self, layer_idx: int, head_dim: int, causal=True, softmax_scale=None, rotary_dim=0, rotary_base=10000.0,
                 rotary_interleaved=False, device=None):
        super().__init__()
        self.layer_idx, self.head_dim, self.causal, self.softmax_scale = layer_idx, head_dim, causal, softmax_scale
        self.rotary_dim = rotary_dim
        self.rotary_emb = (RotaryEmbedding(rotary_dim, base=rotary_base, interleaved=rotary_interleaved, device=device)
                           if rotary_dim > 0 else None)

    def _tables(self, inference_params, like):
        self.rotary_emb._update_cos_sin_cache(inference_params.max_seqlen, device=like.device, dtype=like.dtype)
        return self.rotary_emb._cos_cached, self.rotary_emb._sin_cached

    def forward(self, q, kv, inference_params: InferenceParams):
        batch = q.shape[0]
        fused_rotary = self.rotary_dim > 0 and self.rotary_dim % 16 == 0
        first = inference_params.seqlen_offset == 0
        if self.rotary_dim > 0 and (first or not fused_rotary):
            q, kv = self.rotary_emb(q, kv, seqlen_offset=inference_params.cache_seqlens(batch) if not first else 0,
                                    max_seqlen=inference_params.max_seqlen)
        if first:
            kv_all = update_kv_cache(kv, inference_params, self.layer_idx)
            return flash_attn_kvpacked_func(q, kv_all, softmax_scale=self.softmax_scale, causal=self.causal)
        b0 = inference_params.batch_size_offset
        cache = inference_params.key_value_memory_dict[self.layer_idx][b0:b0 + batch]
        cos, sin = self._tables(inference_params, q) if fused_rotary else (None, None)
        return flash_attn_with_kvcache(
            q, cache[:, :, 0], cache[:, :, 1], kv[:, :, 0], kv[:, :, 1], rotary_cos=cos, rotary_sin=sin,
            cache_seqlens=inference_params.cache_seqlens(batch), softmax_scale=self.softmax_scale, causal=self.causal,
            rotary_interleaved=self.rotary_emb.interleaved if fused_rotary else False)


class DecodeGraphs:
    """Decode steps captured once per (batch, tokens per step) and replayed with new inputs.

    step(inference_params, *inputs) -> tensor is the work of one step (a layer, a stack of layers, a model);
    it must read positions from inference_params.lengths_per_sample, allocate nothing that has to outlive
    the call, and pick its kernels from sizes alone.  The fused KV-cache call does: its split plan depends on
    the cache capacity, never on the lengths, so the step captured at the last position is the step for
    every position.

    run(*inputs, seqlen=...) copies the inputs into the captured buffers, sets every sequence's length to
    `seqlen` (an int, or a (batch,) tensor), replays, and returns the captured output buffer -- valid until
    the next run of the same key; clone it to keep it."""

    def __init__(self, step: Callable, inference_params: InferenceParams, n_warmups: int = 2):
        self.step, self.params, self.n_warmups = step, inference_params, n_warmups
        self.pool = None
        self._graphs: Dict[Tuple, Tuple] = {}
        if inference_params.lengths_per_sample is None:
            raise ValueError("a captured step reads positions from inference_params.lengths_per_sample: allocate it first")

    def _capture(self, inputs):
        params = self.params
        static_in = [torch.zeros_like(x) for x in inputs]
        tokens = inputs[0].shape[1]
        keep_offset, keep_lengths = params.seqlen_offset, params.lengths_per_sample.clone()
        # capture at the last position the cache can hold: the largest problem the step will ever see
        params.seqlen_offset = params.max_seqlen - tokens
        params.lengths_per_sample.fill_(params.seqlen_offset)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(self.n_warmups):  # first calls load kernels, build tables, set per-device attributes
                self.step(params, *static_in)
        side.synchronize()
        torch.cuda.current_stream().wait_stream(side)
        if self.pool is None:
            self.pool = torch.cuda.graphs.graph_pool_handle()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, pool=self.pool):
            static_out = self.step(params, *static_in)
        params.seqlen_offset = keep_offset
        params.lengths_per_sample.copy_(keep_lengths)
        return graph, static_in, static_out

    def run(self, *inputs, seqlen):
        key = tuple((tuple(x.shape), x.dtype) for x in inputs)
        if key not in self._graphs:
            self._graphs[key] = self._capture(inputs)
        graph, static_in, static_out = self._graphs[key]
        batch = inputs[0].shape[0]
        if torch.is_tensor(seqlen):
            self.params.lengths_per_sample[:batch].copy_(seqlen)
        else:
            self.params.lengths_per_sample[:batch].fill_(seqlen)
        for dst, src in zip(static_in, inputs):
            dst.copy_(src)
        graph.replay()
        return static_out

    def release(self):
        """Drops the graphs (before the process group or the allocator they were captured under goes away)."""
        self._graphs.clear()
        self.pool = None


def host_time_per_call_us(fn: Callable, iters: int = 200) -> float:
    """Host time to ENQUEUE one call of fn (wall clock around a run of calls with no synchronisation inside;
    the device is idle before and drained after): the per-step launch overhead that a graph replay removes."""
    fn()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(iters):
        fn()
    t1 = time.perf_counter()
    torch.cuda.synchronize()
    return (t1 - t0) / iters * 1e6
