"""Public attention API with the names, arguments and semantics of FlashAttention v2.3.3's
flash_attn/flash_attn_interface.py (functions at :551-1042, autograd Functions at :193-548).

The reference's own interface file also works unchanged on top of this repository's
`flash_attn_2_cuda` module; this file is the same surface for users who do not have the reference
tree on their path.  One autograd Function serves all six packings: the packed tensors are sliced
into strided q/k/v views on the way in (never copied) and gradients are written straight into views
of one packed gradient tensor on the way out, as the reference does (:199-201, :218-232).
"""
from typing import Optional, Tuple, Union

import torch

import flash_attn_2_cuda as _ext

__all__ = [
    "flash_attn_func", "flash_attn_kvpacked_func", "flash_attn_qkvpacked_func",
    "flash_attn_varlen_func", "flash_attn_varlen_kvpacked_func", "flash_attn_varlen_qkvpacked_func",
    "flash_attn_with_kvcache",
]


def _unit_stride(x):
    return x if x is None or x.stride(-1) == 1 else x.contiguous()


def _split(packing, tensors, varlen):
    """q, k, v views of the user's tensors for packing in {'qkv', 'kv', 'none'}."""
    ax = 1 if varlen else 2  # axis that holds the 3 (or 2) packed operands
    if packing == "qkv":
        (qkv,) = tensors
        return tuple(qkv.select(ax, i) for i in range(3))
    if packing == "kv":
        q, kv = tensors
        return q, kv.select(ax, 0), kv.select(ax, 1)
    return tensors


class _Attention(torch.autograd.Function):
    """forward/backward through flash_attn_2_cuda.{fwd,varlen_fwd,bwd,varlen_bwd}."""

    @staticmethod
    def forward(ctx, packing, seq, dropout_p, softmax_scale, causal, window_size, return_softmax, deterministic, *tensors):
        # seq is None for padded batches, else (cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k)
        varlen = seq is not None
        q, k, v = (_unit_stride(t) for t in _split(packing, tensors, varlen))
        if softmax_scale is None:
            softmax_scale = q.shape[-1] ** (-0.5)
        want_probs = return_softmax and dropout_p > 0
        if varlen:
            cu_q, cu_k, max_q, max_k = seq
            out, q, k, v, out_padded, lse, s_dmask, rng_state = _ext.varlen_fwd(
                q, k, v, None, cu_q, cu_k, max_q, max_k, dropout_p, softmax_scale, False, causal,
                window_size[0], window_size[1], want_probs, None)
            ctx.save_for_backward(q, k, v, out_padded, lse, cu_q, cu_k, rng_state)
            ctx.max_seqlens = (max_q, max_k)
        else:
            out, q, k, v, out_padded, lse, s_dmask, rng_state = _ext.fwd(
                q, k, v, None, dropout_p, softmax_scale, causal, window_size[0], window_size[1], want_probs, None)
            ctx.save_for_backward(q, k, v, out_padded, lse, rng_state)
        ctx.packing, ctx.varlen, ctx.deterministic = packing, varlen, bool(deterministic)
        ctx.dropout_p, ctx.softmax_scale, ctx.causal, ctx.window_size = dropout_p, softmax_scale, causal, window_size
        return out if not return_softmax else (out, lse, s_dmask)

    @staticmethod
    def backward(ctx, dout, *unused):
        if ctx.varlen:
            q, k, v, out, lse, cu_q, cu_k, rng_state = ctx.saved_tensors
        else:
            q, k, v, out, lse, rng_state = ctx.saved_tensors
        ax = 1 if ctx.varlen else 2
        lead_q, lead_k = q.shape[:-2], k.shape[:-2]
        # one packed gradient tensor per packed input; dq/dk/dv are views into it
        if ctx.packing == "qkv":
            dqkv = torch.empty(lead_q + (3,) + q.shape[-2:], dtype=q.dtype, device=q.device)
            dq, dk, dv = (dqkv.select(ax, i) for i in range(3))
            grads = (dqkv,)
        elif ctx.packing == "kv":
            dq = torch.empty_like(q)
            dkv = torch.empty(lead_k + (2,) + k.shape[-2:], dtype=k.dtype, device=k.device)
            dk, dv = dkv.select(ax, 0), dkv.select(ax, 1)
            grads = (dq, dkv)
        else:
            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            grads = (dq, dk, dv)
        dout, q, k, v, out = (_unit_stride(t) for t in (dout, q, k, v, out))
        if ctx.varlen:
            _ext.varlen_bwd(dout, q, k, v, out, lse, dq, dk, dv, cu_q, cu_k, ctx.max_seqlens[0], ctx.max_seqlens[1],
                            ctx.dropout_p, ctx.softmax_scale, False, ctx.causal, ctx.window_size[0],
                            ctx.window_size[1], None, rng_state, deterministic=ctx.deterministic)
        else:
            _ext.bwd(dout, q, k, v, out, lse, dq, dk, dv, ctx.dropout_p, ctx.softmax_scale, ctx.causal,
                     ctx.window_size[0], ctx.window_size[1], None, rng_state, deterministic=ctx.deterministic)
        d = dout.shape[-1]  # the head dim may have been padded to a multiple of 8
        grads = tuple(g[..., :d] for g in grads)
        return (None,) * 8 + grads


def _call(packing, seq, dropout_p, softmax_scale, causal, window_size, return_attn_probs, deterministic, *tensors):
    return _Attention.apply(packing, seq, dropout_p, softmax_scale, causal, tuple(window_size), return_attn_probs,
                            deterministic, *tensors)


# Every function below also takes `deterministic` (not in this version of the reference): the backward's dq is then
# bit-reproducible from run to run whichever kernel the call takes.  The tensor-core kernels always are; the
# any-shape kernel (dropout, operands TMA cannot address) otherwise adds its dq tiles with fp32 atomics.
def flash_attn_qkvpacked_func(qkv, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                              return_attn_probs=False, deterministic=False):
    """qkv: (batch, seqlen, 3, nheads, headdim) -> out (batch, seqlen, nheads, headdim).
    Same contract as flash_attn_interface.py:551-590 of the reference."""
    return _call("qkv", None, dropout_p, softmax_scale, causal, window_size, return_attn_probs, deterministic, qkv)


def flash_attn_kvpacked_func(q, kv, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                             return_attn_probs=False, deterministic=False):
    """q: (batch, seqlen_q, nheads, d), kv: (batch, seqlen_k, 2, nheads_k, d) (reference :593-649).
    MQA/GQA by nheads_k dividing nheads; causal mask aligned to the bottom-right corner."""
    return _call("kv", None, dropout_p, softmax_scale, causal, window_size, return_attn_probs, deterministic, q, kv)


def flash_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                    return_attn_probs=False, deterministic=False):
    """q: (batch, seqlen_q, nheads, d); k, v: (batch, seqlen_k, nheads_k, d) (reference :652-707).
    Query i attends keys in [i + sk - sq - window_size[0], i + sk - sq + window_size[1]]; rows with no
    visible key give zeros.  With return_attn_probs also returns softmax_lse (batch, nheads, seqlen_q)
    and the dropout-sign-encoded probabilities (testing only)."""
    return _call("none", None, dropout_p, softmax_scale, causal, window_size, return_attn_probs, deterministic, q, k, v)


def flash_attn_varlen_qkvpacked_func(qkv, cu_seqlens, max_seqlen, dropout_p=0.0, softmax_scale=None, causal=False,
                                     window_size=(-1, -1), return_attn_probs=False, deterministic=False):
    """qkv: (total, 3, nheads, headdim), cu_seqlens: (batch + 1,) int32 (reference :710-761)."""
    seq = (cu_seqlens, cu_seqlens, max_seqlen, max_seqlen)
    return _call("qkv", seq, dropout_p, softmax_scale, causal, window_size, return_attn_probs, deterministic, qkv)


def flash_attn_varlen_kvpacked_func(q, kv, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p=0.0,
                                    softmax_scale=None, causal=False, window_size=(-1, -1), return_attn_probs=False,
                                    deterministic=False):
    """q: (total_q, nheads, d), kv: (total_k, 2, nheads_k, d) (reference :764-840)."""
    seq = (cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k)
    return _call("kv", seq, dropout_p, softmax_scale, causal, window_size, return_attn_probs, deterministic, q, kv)


def flash_attn_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p=0.0,
                           softmax_scale=None, causal=False, window_size=(-1, -1), return_attn_probs=False,
                           deterministic=False):
    """q: (total_q, nheads, d); k, v: (total_k, nheads_k, d) (reference :843-919)."""
    seq = (cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k)
    return _call("none", seq, dropout_p, softmax_scale, causal, window_size, return_attn_probs, deterministic, q, k, v)


def flash_attn_with_kvcache(q, k_cache, v_cache, k=None, v=None, rotary_cos=None, rotary_sin=None,
                            cache_seqlens: Optional[Union[int, torch.Tensor]] = None,
                            cache_batch_idx: Optional[torch.Tensor] = None, softmax_scale=None, causal=False,
                            window_size: Tuple[int, int] = (-1, -1), rotary_interleaved=True, num_splits=0,
                            block_table: Optional[torch.Tensor] = None, return_softmax_lse=False):
    """Decode-time attention against a KV cache (reference :922-1042), no backward.

    If k/v are given they are written into k_cache/v_cache IN PLACE at rows cache_seqlens[b]... of
    slot cache_batch_idx[b] (after rotary with rotary_cos/rotary_sin at those positions) and then
    attended to, all in one call.  q is rotated at cache_seqlens[b] + i when causal or windowed,
    at cache_seqlens[b] otherwise.  rotary_interleaved=False is the GPT-NeoX pairing (i, i + dim/2).
    num_splits: 0 = choose, 1 = never split the keys, up to 128.

    Two arguments beyond this version of the reference:
    block_table: (batch, pages_per_sequence) int32 for a paged cache.  k_cache / v_cache are then pools
        (num_pages, page_block_size, nheads_k, headdim), page_block_size a multiple of 64, and key j of
        sequence b is row j % page_block_size of page block_table[b, j // page_block_size]; new tokens are
        appended through the table.  Not combined with cache_batch_idx.
    return_softmax_lse: also return the log-sum-exp of every row, (batch, nheads, seqlen_q) fp32.

    Returns out (batch, seqlen_q, nheads, headdim), or (out, softmax_lse).
    """
    assert k_cache.stride(-1) == 1, "k_cache must have contiguous last dimension"
    assert v_cache.stride(-1) == 1, "v_cache must have contiguous last dimension"
    q, k, v = _unit_stride(q), _unit_stride(k), _unit_stride(v)
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    if isinstance(cache_seqlens, int):
        rows = q.shape[0] if block_table is not None else k_cache.shape[0]
        cache_seqlens = torch.full((rows,), cache_seqlens, dtype=torch.int32, device=k_cache.device)
    if cache_batch_idx is not None and not cache_batch_idx.is_contiguous():
        cache_batch_idx = cache_batch_idx.contiguous()
    if block_table is not None and block_table.stride(-1) != 1:
        block_table = block_table.contiguous()
    out, lse = _ext.fwd_kvcache(q, k_cache, v_cache, k, v, cache_seqlens, rotary_cos, rotary_sin, cache_batch_idx, None,
                                softmax_scale, causal, window_size[0], window_size[1], rotary_interleaved, num_splits,
                                block_table=block_table)
    return (out, lse) if return_softmax_lse else out
