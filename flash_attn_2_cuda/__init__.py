"""Drop-in replacement for the `flash_attn_2_cuda` extension module of FlashAttention v2.3.3.

The reference's `flash_attn/flash_attn_interface.py` does `import flash_attn_2_cuda as flash_attn_cuda`
(flash_attn/flash_attn_interface.py:8) and calls five functions positionally
(flash_attn_interface.py:47, 79, 121, 165, 1024).  This module provides those five functions with the
argument order, return lists, checks and error type (RuntimeError) of csrc/flash_attn/flash_api.cpp,
on top of libfa_b200.so (hand-written sm_100a kernels, C ABI in include/fa_b200.h).  What the
reference does with ATen in C++ — padding the head dim to a multiple of 8, allocating outputs and
workspaces, RNG bookkeeping, the seqlen_q==1 grouped-query reshape — is done here with torch.

There is no fallback path: every function ends in a call into the CUDA library.
"""
import ctypes
import os

import torch
import torch.nn.functional as F

from flash_attention_b200 import _lib
from flash_attention_b200._lib import FaBwdArgs, FaFwdArgs, FaKvcacheArgs, check, lib, ptr, tensor3

__all__ = ["fwd", "varlen_fwd", "bwd", "varlen_bwd", "fwd_kvcache"]


def _require(cond, msg):
    # TORCH_CHECK raises c10::Error, which python sees as RuntimeError
    if not cond:
        raise RuntimeError(msg)


def _round_up(x, m):
    return (x + m - 1) // m * m


def _dtype_code(t):
    _require(t.dtype in (torch.float16, torch.bfloat16), "FlashAttention only support fp16 and bf16 data type")
    return _lib.FA_DTYPE_BF16 if t.dtype == torch.bfloat16 else _lib.FA_DTYPE_FP16


def _check_device(*ts):
    for t in ts:
        _require(t.is_cuda, "Input tensor must be on CUDA device")


def _check_last_contig(*ts):
    for t in ts:
        _require(t.stride(-1) == 1, "Input tensor must have contiguous last dimension")


def _check_shape(t, *shape):
    _require(tuple(t.shape) == tuple(shape), "tensor must have shape (%s), got %s" % (", ".join(map(str, shape)), tuple(t.shape)))


def _stream(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _pad8(t):
    d = t.shape[-1]
    return t if d % 8 == 0 else F.pad(t, (0, 8 - d % 8))


def _aligned(t):
    """The kernels read 16-byte vectors: a view whose base or strides break that is copied."""
    if t is None:
        return t
    ok = t.data_ptr() % 16 == 0 and all(s % 8 == 0 for s in t.stride()[:-1])
    return t if ok else t.contiguous()


def _sm_count(dev):
    return torch.cuda.get_device_properties(dev).multi_processor_count


def _windows(is_causal, wl, wr, seqlen_k):
    # flash_api.cpp:297 (causal means right window 0) and set_params_fprop (flash_api.cpp:113-114):
    # a window that is open on one side only gets seqlen_k on the open side.  That is NOT the same
    # as unbounded when seqlen_q > seqlen_k, and the reference's behaviour is kept as it is.
    wl, wr = int(wl), int(wr)
    if is_causal:
        wr = 0
    if wl < 0 and wr >= 0:
        wl = int(seqlen_k)
    if wl >= 0 and wr < 0:
        wr = int(seqlen_k)
    return wl, wr


def _philox(gen, p_dropout, batch, heads, device):
    """(seed, offset, rng_state) and advances the generator by batch*heads*32 (flash_api.cpp:391-406)."""
    rng_state = torch.empty(2, dtype=torch.int64, device=device)
    if p_dropout <= 0.0:
        return 0, 0, rng_state
    g = gen if gen is not None else torch.cuda.default_generators[device.index if device.index is not None else torch.cuda.current_device()]
    seed = int(g.initial_seed())
    offset = int(g.get_offset())
    inc = batch * heads * 32
    g.set_offset(offset + _round_up(inc, 4))
    rng_state.copy_(torch.tensor([seed & 0x7FFFFFFFFFFFFFFF, offset], dtype=torch.int64), non_blocking=True)
    return seed & 0x7FFFFFFFFFFFFFFF, offset, rng_state


# -------------------------------------------------------------------------------------------
def fwd(q, k, v, out_, p_dropout, softmax_scale, is_causal, window_size_left, window_size_right, return_softmax, gen_):
    """mha_fwd (csrc/flash_attn/flash_api.cpp:248-424).

    q: (batch, seqlen_q, heads, d); k, v: (batch, seqlen_k, heads_k, d).
    Returns [out, q_padded, k_padded, v_padded, out_padded, softmax_lse, p, rng_state].
    """
    dt = _dtype_code(q)
    _require(k.dtype == q.dtype, "query and key must have the same dtype")
    _require(v.dtype == q.dtype, "query and value must have the same dtype")
    _check_device(q, k, v)
    _check_last_contig(q, k, v)
    batch, seqlen_q, heads, d_og = q.shape
    seqlen_k, heads_k = k.shape[1], k.shape[2]
    _require(batch > 0, "batch size must be postive")
    _require(d_og <= 256, "FlashAttention forward only supports head dimension at most 256")
    _require(heads % heads_k == 0, "Number of heads in key/value must divide number of heads in query")
    if seqlen_q == 1:
        is_causal = False
    wl, wr = _windows(is_causal, window_size_left, window_size_right, seqlen_k)

    swapped = seqlen_q == 1 and heads > heads_k and wl < 0 and wr < 0 and p_dropout == 0.0 and d_og % 8 == 0
    if swapped:
        g = heads // heads_k
        q = q.reshape(batch, heads_k, g, d_og).transpose(1, 2)
        seqlen_q, heads = g, heads_k
    _check_shape(q, batch, seqlen_q, heads, d_og)
    _check_shape(k, batch, seqlen_k, heads_k, d_og)
    _check_shape(v, batch, seqlen_k, heads_k, d_og)

    q_p, k_p, v_p = _aligned(_pad8(q)), _aligned(_pad8(k)), _aligned(_pad8(v))
    d = q_p.shape[-1]
    if out_ is not None:
        out = out_
        _require(out.dtype == q.dtype, "Output must have the same dtype as inputs")
        _check_device(out)
        _check_last_contig(out)
        _check_shape(out, batch, seqlen_q, heads, d_og)
        if d_og % 8 != 0 or _aligned(out) is not out:
            out = torch.empty_like(q_p)
    else:
        out = torch.empty((batch, seqlen_q, heads, d), dtype=q.dtype, device=q.device)

    with torch.cuda.device(q.device):
        lse = torch.empty((batch, heads, seqlen_q), dtype=torch.float32, device=q.device)
        p = None
        if return_softmax:
            _require(p_dropout > 0.0, "return_softmax is only supported when p_dropout > 0.0")
            p = torch.empty((batch, heads, _round_up(seqlen_q, 128), _round_up(seqlen_k, 128)), dtype=q.dtype, device=q.device)
        seed, offset, rng_state = _philox(gen_, p_dropout, batch, heads, q.device)
        if seqlen_k > 0:
            a = FaFwdArgs()
            a.q, a.k, a.v, a.out = tensor3(q_p), tensor3(k_p), tensor3(v_p), tensor3(out)
            a.softmax_lse, a.lse_seqlen = ptr(lse), seqlen_q
            a.batch, a.seqlen_q, a.seqlen_k, a.heads, a.heads_k, a.head_dim = batch, seqlen_q, seqlen_k, heads, heads_k, d
            a.dtype, a.softmax_scale = dt, float(softmax_scale)
            a.window_left, a.window_right = wl, wr
            a.p_dropout, a.rng_seed, a.rng_offset = float(p_dropout), seed, offset
            if p is not None:
                a.s_dmask, a.sdmask_rows, a.sdmask_cols = ptr(p), p.shape[2], p.shape[3]
            a.num_splits = 1
            keep = None
            if p_dropout == 0.0:  # flash_api.cpp:373-389
                ns = lib().fa_fwd_num_splits(batch, heads, seqlen_q, seqlen_k, d, _sm_count(q.device))
                if os.environ.get("FA_B200_FWD_SPLITS"):  # test knob: pin the split count (1 = never split)
                    ns = max(1, min(128, int(os.environ["FA_B200_FWD_SPLITS"])))
                if ns > 1:
                    lse_acc = torch.empty((ns, batch, heads, seqlen_q), dtype=torch.float32, device=q.device)
                    out_acc = torch.empty((ns, batch, heads, seqlen_q, d), dtype=torch.float32, device=q.device)
                    a.num_splits, a.lse_accum, a.out_accum = ns, ptr(lse_acc), ptr(out_acc)
                    keep = (lse_acc, out_acc)
            check(lib().fa_fwd(ctypes.byref(a), _stream(q)), "flash_attn_2_cuda.fwd")
            del keep
        else:
            # no keys: flash_api.cpp:409-414
            out.zero_()
            lse.fill_(float("inf"))

    out_padded = out
    if d_og % 8 != 0:
        out = out[..., :d_og]
        if out_ is not None:
            out_.copy_(out)
    elif out_ is not None and out is not out_:
        out_.copy_(out)
        out = out_
    if swapped:
        g = seqlen_q
        out_padded = out_padded.transpose(1, 2).reshape(batch, 1, heads_k * g, d_og)
        out = out.transpose(1, 2).reshape(batch, 1, heads_k * g, d_og)
        q_p = q_p.transpose(1, 2).reshape(batch, 1, heads_k * g, d_og)
        lse = lse.reshape(batch, heads_k * g, 1)
    return [out, q_p, k_p, v_p, out_padded, lse, p, rng_state]


def varlen_fwd(q, k, v, out_, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, p_dropout, softmax_scale,
               zero_tensors, is_causal, window_size_left, window_size_right, return_softmax, gen_):
    """mha_varlen_fwd (csrc/flash_attn/flash_api.cpp:426-585).

    q: (total_q, heads, d); k, v: (total_k, heads_k, d); cu_seqlens_*: (batch + 1) int32.
    """
    dt = _dtype_code(q)
    _require(k.dtype == q.dtype, "query and key must have the same dtype")
    _require(v.dtype == q.dtype, "query and value must have the same dtype")
    _require(cu_seqlens_q.dtype == torch.int32, "cu_seqlens_q must have dtype int32")
    _require(cu_seqlens_k.dtype == torch.int32, "cu_seqlens_k must have dtype int32")
    _check_device(q, k, v, cu_seqlens_q, cu_seqlens_k)
    _check_last_contig(q, k, v)
    _require(cu_seqlens_q.is_contiguous(), "cu_seqlens_q must be contiguous")
    _require(cu_seqlens_k.is_contiguous(), "cu_seqlens_k must be contiguous")
    total_q, heads, d_og = q.shape
    total_k, heads_k = k.shape[0], k.shape[1]
    batch = cu_seqlens_q.numel() - 1
    _require(batch > 0, "batch size must be positive")
    _require(d_og <= 256, "FlashAttention forward only supports head dimension at most 256")
    _require(heads % heads_k == 0, "Number of heads in key/value must divide number of heads in query")
    _check_shape(q, total_q, heads, d_og)
    _check_shape(k, total_k, heads_k, d_og)
    _check_shape(v, total_k, heads_k, d_og)
    _check_shape(cu_seqlens_q, batch + 1)
    _check_shape(cu_seqlens_k, batch + 1)
    wl, wr = _windows(is_causal, window_size_left, window_size_right, max_seqlen_k)

    q_p, k_p, v_p = _aligned(_pad8(q)), _aligned(_pad8(k)), _aligned(_pad8(v))
    d = q_p.shape[-1]
    if out_ is not None:
        out = out_
        _require(out.dtype == q.dtype, "Output must have the same dtype as inputs")
        _check_device(out)
        _check_last_contig(out)
        _check_shape(out, total_q, heads, d_og)
        if d_og % 8 != 0 or _aligned(out) is not out:
            out = torch.empty_like(q_p)
    else:
        out = torch.empty((total_q, heads, d), dtype=q.dtype, device=q.device)

    with torch.cuda.device(q.device):
        lse = torch.empty((batch, heads, max_seqlen_q), dtype=torch.float32, device=q.device)
        p = None
        if return_softmax:
            _require(p_dropout > 0.0, "return_softmax is only supported when p_dropout > 0.0")
            p = torch.empty((batch, heads, _round_up(max_seqlen_q, 128), _round_up(max_seqlen_k, 128)), dtype=q.dtype, device=q.device)
        if zero_tensors:
            out.zero_()
            lse.fill_(float("-inf"))
            if p is not None:
                p.zero_()
        seed, offset, rng_state = _philox(gen_, p_dropout, batch, heads, q.device)
        a = FaFwdArgs()
        a.q, a.k, a.v, a.out = tensor3(q_p, True), tensor3(k_p, True), tensor3(v_p, True), tensor3(out, True)
        a.softmax_lse, a.lse_seqlen = ptr(lse), max_seqlen_q
        a.batch, a.seqlen_q, a.seqlen_k, a.heads, a.heads_k, a.head_dim = batch, max_seqlen_q, max_seqlen_k, heads, heads_k, d
        a.dtype, a.softmax_scale = dt, float(softmax_scale)
        a.window_left, a.window_right = wl, wr
        a.cu_seqlens_q, a.cu_seqlens_k, a.total_q, a.total_k = ptr(cu_seqlens_q), ptr(cu_seqlens_k), total_q, total_k
        a.p_dropout, a.rng_seed, a.rng_offset = float(p_dropout), seed, offset
        if p is not None:
            a.s_dmask, a.sdmask_rows, a.sdmask_cols = ptr(p), p.shape[2], p.shape[3]
        a.num_splits = 1
        if max_seqlen_q > 0:
            check(lib().fa_fwd(ctypes.byref(a), _stream(q)), "flash_attn_2_cuda.varlen_fwd")

    out_padded = out
    if d_og % 8 != 0:
        out = out[..., :d_og]
        if out_ is not None:
            out_.copy_(out)
    elif out_ is not None and out is not out_:
        out_.copy_(out)
        out = out_
    return [out, q_p, k_p, v_p, out_padded, lse, p, rng_state]


# -------------------------------------------------------------------------------------------
def _grad_out(given, shape, like, name):
    if given is None:
        return torch.empty(shape, dtype=like.dtype, device=like.device), None
    _require(given.dtype == like.dtype, "%s must have the same dtype as q" % name)
    _check_device(given)
    _check_last_contig(given)
    _check_shape(given, *shape)
    if _aligned(given) is not given:
        return torch.empty(shape, dtype=like.dtype, device=like.device), given
    return given, None


def _bwd_common(varlen, dout, q, k, v, out, softmax_lse, dq_, dk_, dv_, cu_q, cu_k, max_q, max_k, p_dropout,
                softmax_scale, is_causal, wl_in, wr_in, rng_state, what, deterministic=False):
    dt = _dtype_code(q)
    _require(k.dtype == q.dtype, "query and key must have the same dtype")
    _require(v.dtype == q.dtype, "query and value must have the same dtype")
    _require(out.dtype == q.dtype, "query and out must have the same dtype")
    _require(dout.dtype == q.dtype, "query and dout must have the same dtype")
    _check_device(q, k, v, out, dout, softmax_lse)
    _check_last_contig(q, k, v)
    _require(out.stride(-1) == 1, "out tensor must have contiguous last dimension")
    _require(dout.stride(-1) == 1, "dout tensor must have contiguous last dimension")
    d_og = dout.shape[-1]
    d = q.shape[-1]
    if varlen:
        _require(cu_q.dtype == torch.int32 and cu_k.dtype == torch.int32, "cu_seqlens must have dtype int32")
        _check_device(cu_q, cu_k)
        _require(cu_q.is_contiguous() and cu_k.is_contiguous(), "cu_seqlens must be contiguous")
        total_q, heads, _ = q.shape
        total_k, heads_k = k.shape[0], k.shape[1]
        batch = cu_q.numel() - 1
        seqlen_q, seqlen_k = int(max_q), int(max_k)
        q_shape, k_shape = (total_q, heads, d), (total_k, heads_k, d)
        _check_shape(dout, total_q, heads, d_og)
        _check_shape(cu_q, batch + 1)
        _check_shape(cu_k, batch + 1)
    else:
        batch, seqlen_q, heads, _ = q.shape
        seqlen_k, heads_k = k.shape[1], k.shape[2]
        total_q = total_k = 0
        q_shape, k_shape = (batch, seqlen_q, heads, d), (batch, seqlen_k, heads_k, d)
        _check_shape(dout, batch, seqlen_q, heads, d_og)
    _require(batch > 0, "batch size must be positive")
    _require(d % 8 == 0, "head_size should be a multiple of 8")
    _require(d <= 256, "FlashAttention backward only supports head dimension at most 256")
    _require(heads % heads_k == 0, "Number of heads in key/value must divide number of heads in query")
    _check_shape(q, *q_shape)
    _check_shape(k, *k_shape)
    _check_shape(v, *k_shape)
    _check_shape(out, *q_shape)
    wl, wr = _windows(is_causal, wl_in, wr_in, seqlen_k)

    dout_p = _aligned(_pad8(dout))
    q, k, v, out = _aligned(q), _aligned(k), _aligned(v), _aligned(out)
    dq, dq_user = _grad_out(dq_, q_shape, q, "dq")
    dk, dk_user = _grad_out(dk_, k_shape, q, "dk")
    dv, dv_user = _grad_out(dv_, k_shape, q, "dv")

    with torch.cuda.device(q.device):
        d_seqlen = _round_up(seqlen_q, 128)
        softmax_d = torch.empty((batch, heads, d_seqlen), dtype=torch.float32, device=q.device)
        seed = offset = 0
        if p_dropout > 0.0:
            _require(rng_state is not None, "rng_state from the forward pass is required when p_dropout > 0")
            seed, offset = [int(x) for x in rng_state.tolist()]
        if seqlen_q > 0 and seqlen_k > 0 and (not varlen or (total_q > 0 and total_k > 0)):
            nbytes = lib().fa_bwd_workspace_bytes(batch, seqlen_q, heads, d, total_q, 1 if varlen else 0)
            dq_accum = torch.empty(nbytes // 4, dtype=torch.float32, device=q.device)
            a = FaBwdArgs()
            a.q, a.k, a.v, a.out, a.dout = (tensor3(x, varlen) for x in (q, k, v, out, dout_p))
            a.dq, a.dk, a.dv = tensor3(dq, varlen), tensor3(dk, varlen), tensor3(dv, varlen)
            a.softmax_lse, a.lse_seqlen = ptr(softmax_lse), softmax_lse.shape[-1]
            a.softmax_d, a.d_seqlen, a.dq_accum = ptr(softmax_d), d_seqlen, ptr(dq_accum)
            a.batch, a.seqlen_q, a.seqlen_k, a.heads, a.heads_k, a.head_dim = batch, seqlen_q, seqlen_k, heads, heads_k, d
            a.dtype, a.softmax_scale = dt, float(softmax_scale)
            a.window_left, a.window_right = wl, wr
            if varlen:
                a.cu_seqlens_q, a.cu_seqlens_k, a.total_q, a.total_k = ptr(cu_q), ptr(cu_k), total_q, total_k
            a.p_dropout, a.rng_seed, a.rng_offset = float(p_dropout), seed, offset
            a.deterministic = 1 if deterministic else 0
            check(lib().fa_bwd(ctypes.byref(a), _stream(q)), what)
            del dq_accum
        else:
            # flash_api.cpp:797-804: nothing to attend to
            dk.zero_()
            dv.zero_()
            dq.zero_()
            softmax_d.zero_()
    for buf, user in ((dq, dq_user), (dk, dk_user), (dv, dv_user)):
        if user is not None:
            user.copy_(buf)
    dq = dq_user if dq_user is not None else dq
    dk = dk_user if dk_user is not None else dk
    dv = dv_user if dv_user is not None else dv
    if d_og % 8 != 0:
        dq, dk, dv = dq[..., :d_og], dk[..., :d_og], dv[..., :d_og]
    return [dq, dk, dv, softmax_d]


def bwd(dout, q, k, v, out, softmax_lse, dq_, dk_, dv_, p_dropout, softmax_scale, is_causal, window_size_left,
        window_size_right, gen_, rng_state, *, deterministic=False):
    """mha_bwd (csrc/flash_attn/flash_api.cpp:609-811). Returns [dq, dk, dv, softmax_d].
    deterministic (keyword only, not in this version of the reference): dq bit-reproducible from run to run
    also when the call takes the any-shape kernel (the tensor-core kernels always are)."""
    return _bwd_common(False, dout, q, k, v, out, softmax_lse, dq_, dk_, dv_, None, None, 0, 0, p_dropout,
                       softmax_scale, is_causal, window_size_left, window_size_right, rng_state, "flash_attn_2_cuda.bwd",
                       deterministic)


def varlen_bwd(dout, q, k, v, out, softmax_lse, dq_, dk_, dv_, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
               p_dropout, softmax_scale, zero_tensors, is_causal, window_size_left, window_size_right, gen_, rng_state,
               *, deterministic=False):
    """mha_varlen_bwd (csrc/flash_attn/flash_api.cpp:813-1036). Returns [dq, dk, dv, softmax_d]."""
    if zero_tensors:
        for t in (dq_, dk_, dv_):
            if t is not None:
                t.zero_()
    return _bwd_common(True, dout, q, k, v, out, softmax_lse, dq_, dk_, dv_, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                       max_seqlen_k, p_dropout, softmax_scale, is_causal, window_size_left, window_size_right,
                       rng_state, "flash_attn_2_cuda.varlen_bwd", deterministic)


# -------------------------------------------------------------------------------------------
def fwd_kvcache(q, kcache, vcache, k_, v_, seqlens_k_, rotary_cos_, rotary_sin_, cache_batch_idx_, out_,
                softmax_scale, is_causal, window_size_left, window_size_right, is_rotary_interleaved, num_splits,
                *, block_table=None):
    """mha_fwd_kvcache (csrc/flash_attn/flash_api.cpp:1038-1279). Returns [out, softmax_lse].

    kcache / vcache are updated in place at rows [seqlens_k[b], seqlens_k[b] + seqlen_new) of batch
    slot cache_batch_idx[b] when k_ / v_ are given.

    block_table (keyword only; not in this version of the reference, whose 16 positional arguments are kept):
    (batch, pages_per_sequence) int32.  kcache / vcache are then pools (num_pages, page_block_size, heads_k, d);
    key j of sequence b is row j % page_block_size of page block_table[b, j // page_block_size].
    """
    dt = _dtype_code(q)
    _require(kcache.dtype == q.dtype, "query and key must have the same dtype")
    _require(vcache.dtype == q.dtype, "query and value must have the same dtype")
    _check_device(q, kcache, vcache)
    _check_last_contig(q, kcache, vcache)
    batch, seqlen_q, heads, d_og = q.shape
    batch_c, seqlen_k, heads_k = kcache.shape[0], kcache.shape[1], kcache.shape[2]
    page_block_size = 0
    if block_table is not None:
        _check_device(block_table)
        _require(block_table.dtype == torch.int32, "block_table must have dtype torch.int32")
        _require(block_table.dim() == 2 and block_table.shape[0] == batch and block_table.stride(-1) == 1,
                 "block_table must have shape (batch, pages per sequence) with contiguous last dimension")
        _require(cache_batch_idx_ is None, "Paged KVcache does not support cache_batch_idx")
        page_block_size = seqlen_k  # kcache is (num_pages, page_block_size, heads_k, d)
        _require(page_block_size % 64 == 0, "Paged KV cache block size must be divisible by 64")
        seqlen_k = block_table.shape[1] * page_block_size  # capacity of one sequence
    _require(batch > 0, "batch size must be postive")
    _require(d_og <= 256, "FlashAttention forward only supports head dimension at most 256")
    _require(heads % heads_k == 0, "Number of heads in key/value must divide number of heads in query")
    if seqlen_q == 1:
        is_causal = False
    wl, wr = _windows(is_causal, window_size_left, window_size_right, seqlen_k)

    swapped = seqlen_q == 1 and heads > heads_k and wl < 0 and wr < 0 and d_og % 8 == 0
    if swapped:
        g = heads // heads_k
        q = q.reshape(batch, heads_k, g, d_og).transpose(1, 2)
        seqlen_q, heads = g, heads_k
    _check_shape(q, batch, seqlen_q, heads, d_og)
    _check_shape(kcache, batch_c, page_block_size or seqlen_k, heads_k, d_og)
    _check_shape(vcache, batch_c, page_block_size or seqlen_k, heads_k, d_og)

    padded = d_og % 8 != 0
    q_p = _aligned(_pad8(q))
    kc, vc = (_pad8(kcache), _pad8(vcache)) if padded else (kcache, vcache)
    _require(_aligned(kc) is kc and _aligned(vc) is vc, "k_cache / v_cache must be 16-byte aligned with strides that are multiples of 8")
    d = q_p.shape[-1]
    if out_ is not None:
        out = out_
        _require(out.dtype == q.dtype, "Output must have the same dtype as inputs")
        _check_device(out)
        _check_last_contig(out)
        _check_shape(out, batch, seqlen_q, heads, d_og)
        if padded or _aligned(out) is not out:
            out = torch.empty_like(q_p)
    else:
        out = torch.empty((batch, seqlen_q, heads, d), dtype=q.dtype, device=q.device)

    a = FaKvcacheArgs()
    seqlen_new = 0
    k_p = v_p = None
    if k_ is not None:
        _require(v_ is not None, "If key is supplied, value must also be passed in")
        _require(seqlens_k_ is not None, "If key is supplied, seqlens_k must also be passed in")
        _require(seqlen_q <= seqlen_k or swapped, "If key is supplied, it must have seqlen <= the seqlen of the KV cache")
        _require(k_.dtype == q.dtype, "Key must have the same dtype as query")
        _require(v_.dtype == q.dtype, "Value must have the same dtype as query")
        _check_device(k_, v_)
        _check_last_contig(k_, v_)
        seqlen_new = k_.shape[1]
        _check_shape(k_, batch, seqlen_new, heads_k, d_og)
        _check_shape(v_, batch, seqlen_new, heads_k, d_og)
        k_p, v_p = _aligned(_pad8(k_)), _aligned(_pad8(v_))
        a.knew, a.vnew = tensor3(k_p), tensor3(v_p)
    if seqlens_k_ is not None:
        _require(seqlens_k_.dtype == torch.int32, "seqlens_k must have dtype int32")
        _check_device(seqlens_k_)
        _require(seqlens_k_.is_contiguous(), "seqlens_k must be contiguous")
        _check_shape(seqlens_k_, batch)
    if rotary_cos_ is not None:
        _require(k_ is not None, "If rotary cos/sin are provided, new key / value to be appended to KV cache must also be provided")
        _require(rotary_sin_ is not None, "rotary_sin must be given with rotary_cos")
        _check_device(rotary_cos_, rotary_sin_)
        rotary_dim = rotary_cos_.shape[1] * 2
        _require(rotary_dim <= d_og, "rotary_dim must be <= headdim")
        _require(rotary_dim % 16 == 0, "Only rotary dimensions divisible by 16 are currently supported")
        seqlen_ro = rotary_cos_.shape[0]
        _require(seqlen_ro >= seqlen_k, "cos/sin seqlen must be at least the seqlen of KV cache")
        _check_shape(rotary_cos_, seqlen_ro, rotary_dim // 2)
        _check_shape(rotary_sin_, seqlen_ro, rotary_dim // 2)
        _require(rotary_cos_.is_contiguous() and rotary_sin_.is_contiguous(), "rotary cos/sin must be contiguous")
        _require(rotary_cos_.dtype == q.dtype, "rotary_cos must have the same dtype as query")
        _require(rotary_sin_.dtype == q.dtype, "rotary_cos must have the same dtype as query")
        a.rotary_cos, a.rotary_sin = ptr(rotary_cos_), ptr(rotary_sin_)
        a.rotary_dim, a.seqlen_ro, a.rotary_interleaved = rotary_dim, seqlen_ro, 1 if is_rotary_interleaved else 0
    if cache_batch_idx_ is not None:
        _check_device(cache_batch_idx_)
        _require(cache_batch_idx_.dtype == torch.int32, "cache_batch_idx must have dtype int32")
        _require(cache_batch_idx_.is_contiguous(), "cache_batch_idx must be contiguous")
        _check_shape(cache_batch_idx_, batch)
    elif block_table is None:
        _require(batch_c >= batch, "the KV cache must hold at least `batch` sequences when cache_batch_idx is not given")
    _require(num_splits <= 128, "num_splits > 128 not supported")

    with torch.cuda.device(q.device):
        lse = torch.empty((batch, heads, seqlen_q), dtype=torch.float32, device=q.device)
        a.q, a.kcache, a.vcache, a.out = tensor3(q_p), tensor3(kc), tensor3(vc), tensor3(out)
        a.softmax_lse = ptr(lse)
        a.batch, a.batch_cache, a.seqlen_q, a.seqlen_cache, a.seqlen_new = batch, batch_c, seqlen_q, seqlen_k, seqlen_new
        a.heads, a.heads_k, a.head_dim = heads, heads_k, d
        a.dtype, a.softmax_scale = dt, float(softmax_scale)
        a.window_left, a.window_right = wl, wr
        a.cache_seqlens, a.cache_batch_idx = ptr(seqlens_k_), ptr(cache_batch_idx_)
        a.q_rows_share_position = 1 if swapped else 0
        a.num_splits = int(num_splits)
        if block_table is not None:
            a.block_table, a.block_table_stride, a.page_block_size = ptr(block_table), block_table.stride(0), page_block_size
        lse_b, out_b = ctypes.c_int64(0), ctypes.c_int64(0)
        ns = lib().fa_kvcache_plan(ctypes.byref(a), _sm_count(q.device), ctypes.byref(lse_b), ctypes.byref(out_b))
        if ns < 0:
            raise RuntimeError("flash_attn_2_cuda.fwd_kvcache: " + _lib.last_error())
        keep = []
        if ns > 1:
            lse_acc = torch.empty(lse_b.value // 4, dtype=torch.float32, device=q.device)
            out_acc = torch.empty(out_b.value // 4, dtype=torch.float32, device=q.device)
            a.lse_accum, a.out_accum = ptr(lse_acc), ptr(out_acc)
            keep += [lse_acc, out_acc]
        if rotary_cos_ is not None:
            q_rot = torch.empty((batch, seqlen_q, heads, d), dtype=q.dtype, device=q.device)
            a.q_rotated = ptr(q_rot)
            keep.append(q_rot)
        check(lib().fa_fwd_kvcache(ctypes.byref(a), _stream(q)), "flash_attn_2_cuda.fwd_kvcache")
        del keep

    if padded:
        out = out[..., :d_og]
        if out_ is not None:
            out_.copy_(out)
        if k_ is not None:
            # as in flash_api.cpp:1266-1272: copy the padded caches back
            kcache.copy_(kc[..., :d_og])
            vcache.copy_(vc[..., :d_og])
    elif out_ is not None and out is not out_:
        out_.copy_(out)
        out = out_
    if swapped:
        g = seqlen_q
        out = out.transpose(1, 2).reshape(batch, 1, heads_k * g, d_og)
        lse = lse.reshape(batch, heads_k * g, 1)
    return [out, lse]
