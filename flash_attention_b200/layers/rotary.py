"""Rotary position embedding in front of attention.

Public surface (names, arguments, in-place behaviour and gradients) of the reference's
flash_attn/layers/rotary.py: apply_rotary_emb (:96-124), apply_rotary_emb_qkv_ (:207-231),
apply_rotary_emb_kv_ (:271-292), RotaryEmbedding (:295-480), plus the attributes that
flash_attn/modules/mha.py:451-455 reads from the module (scale, _update_cos_sin_cache, _cos_cached,
_sin_cached).  Underneath it is built differently: `apply_rotary` binds the `fa_rotary` entry point of the
C ABI (in place of the Triton kernel of flash_attn/ops/triton/rotary.py), ONE autograd node serves every
entry point -- each of them only says which 4-D views of its tensor turn with which table pair -- and the
module keeps its tables in a small cache object of its own.

A rotation is orthogonal, so its backward is the rotation by the negative angle (`conjugate`) of the
incoming gradient: nothing but the tables and the offsets is kept for it.
"""
import ctypes
from typing import Optional, Union

import torch


def apply_rotary(x, cos, sin, seqlen_offsets: Union[int, torch.Tensor] = 0, cu_seqlens=None, max_seqlen=None,
                 interleaved=False, inplace=False, conjugate=False):
    """Same contract as apply_rotary of flash_attn/ops/triton/rotary.py:143-240.
    x: (batch, seqlen, nheads, headdim), or (total_seqlen, nheads, headdim) with cu_seqlens.
    cos, sin: (seqlen_ro, rotary_dim / 2).  Returns the rotated tensor (x itself if inplace)."""
    from flash_attention_b200 import _lib
    from flash_attention_b200._lib import FaRotaryArgs, FaTensor, check, lib

    if not x.is_cuda:
        raise RuntimeError("apply_rotary: x must be a CUDA tensor (there is no CPU path)")
    is_varlen = cu_seqlens is not None
    if not is_varlen:
        batch, seqlen, nheads, headdim = x.shape
        total = 0
    else:
        assert max_seqlen is not None, "If cu_seqlens is passed in, then max_seqlen must be passed"
        total, nheads, headdim = x.shape
        batch = cu_seqlens.shape[0] - 1
        seqlen = max_seqlen
    seqlen_ro, rotary_half = cos.shape
    rotary_dim = rotary_half * 2
    assert sin.shape == cos.shape
    assert rotary_dim <= headdim, "rotary_dim must be <= headdim"
    assert headdim <= 256, "Only support headdim <= 256"
    assert seqlen_ro >= seqlen, "seqlen_ro must be >= seqlen"
    assert cos.dtype == sin.dtype, f"cos and sin must have the same dtype, got {cos.dtype} and {sin.dtype}"
    assert x.dtype == cos.dtype, f"Input and cos/sin must have the same dtype, got {x.dtype} and {cos.dtype}"
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("apply_rotary only supports fp16 and bf16")
    cos, sin = cos.contiguous(), sin.contiguous()
    offs_t = None
    if isinstance(seqlen_offsets, torch.Tensor):
        assert seqlen_offsets.shape == (batch,)
        assert seqlen_offsets.dtype in [torch.int32, torch.int64]
        offs_t = seqlen_offsets.to(torch.int32).contiguous()
        offs_i = 0
    else:
        offs_i = int(seqlen_offsets)
        assert offs_i + seqlen <= seqlen_ro
    if x.stride(-1) != 1:
        if inplace:
            raise RuntimeError("apply_rotary: in-place rotation needs a unit stride in the last dimension")
        x = x.contiguous()
    out = x if inplace else torch.empty_like(x)
    if out.stride(-1) != 1:
        out = torch.empty(x.shape, dtype=x.dtype, device=x.device)

    def t3(t):
        if is_varlen:
            return FaTensor(t.data_ptr(), 0, t.stride(0), t.stride(1))
        return FaTensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))

    a = FaRotaryArgs()
    a.x, a.out = t3(x), t3(out)
    a.cos, a.sin = cos.data_ptr(), sin.data_ptr()
    a.seqlen_offsets = None if offs_t is None else offs_t.data_ptr()
    cu = None
    if is_varlen:
        cu = cu_seqlens.to(torch.int32).contiguous()
        a.cu_seqlens = cu.data_ptr()
    a.batch, a.seqlen, a.heads, a.head_dim, a.total = batch, seqlen, nheads, headdim, total
    a.rotary_dim, a.seqlen_ro, a.seqlen_offset = rotary_dim, seqlen_ro, offs_i
    a.dtype = _lib.FA_DTYPE_BF16 if x.dtype == torch.bfloat16 else _lib.FA_DTYPE_FP16
    a.interleaved, a.conjugate = int(bool(interleaved)), int(bool(conjugate))
    stream = ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)
    with torch.cuda.device(x.device):
        check(lib().fa_rotary(ctypes.byref(a), stream), "apply_rotary")
    return out


# ------------------------------------------------------------------------------------------------
# One autograd node for all entry points
#
# A "turn list" names what to rotate: pairs (view of the tensor, index of the table pair).  The three public
# shapes differ only in that list:
#   x    (batch, seqlen, heads, d)     -> the tensor itself with tables 0
#   qkv  (batch, seqlen, 3, heads, d)  -> q and k; as ONE view over 2 * heads heads when both use tables 0
#   kv   (batch, seqlen, 2, heads, d)  -> k
def _turns_x(t, two_tables):
    return [(t, 0)]


def _turns_qkv(t, two_tables):
    batch, seqlen, three, heads, d = t.shape
    if three != 3:
        raise ValueError("qkv must have shape (batch, seqlen, 3, nheads, headdim)")
    if not two_tables and t.is_contiguous():
        return [(t[:, :, :2].reshape(batch, seqlen, 2 * heads, d), 0)]  # q and k heads are neighbours in memory
    return [(t[:, :, 0], 0), (t[:, :, 1], 1 if two_tables else 0)]


def _turns_kv(t, two_tables):
    if t.shape[2] != 2:
        raise ValueError("kv must have shape (batch, seqlen, 2, nheads, headdim)")
    return [(t[:, :, 0], 0)]


class _Turn(torch.autograd.Function):
    """forward(t, turns, opts, offsets, cos, sin, cos_k, sin_k) -> rotated t.

    opts = (interleaved, inplace, cu_seqlens, max_seqlen).  Out of place only for the plain-x entry (the packed
    entries are in place by contract)."""

    @staticmethod
    def _run(t, turns, opts, offsets, tables, conjugate, inplace):
        interleaved, _, cu_seqlens, max_seqlen = opts
        two = tables[1][0] is not None
        result = t
        for view, which in turns(t, two):
            cos, sin = tables[which]
            r = apply_rotary(view, cos, sin, seqlen_offsets=offsets, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen,
                             interleaved=interleaved, inplace=inplace, conjugate=conjugate)
            if not inplace:
                result = r  # only the single-view entry gets here
        return result

    @staticmethod
    def forward(ctx, t, turns, opts, offsets, cos, sin, cos_k, sin_k):
        inplace = opts[1]
        out = _Turn._run(t, turns, opts, offsets, ((cos, sin), (cos_k, sin_k)), False, inplace)
        ctx.turns, ctx.opts = turns, opts
        ctx.int_offsets = None if torch.is_tensor(offsets) else offsets
        ctx.save_for_backward(cos, sin, cos_k, sin_k, offsets if torch.is_tensor(offsets) else None)
        # an in-place call hands back its own argument (leaves that require grad included), as the reference does
        return out

    @staticmethod
    def backward(ctx, grad):
        cos, sin, cos_k, sin_k, offsets = ctx.saved_tensors
        if offsets is None:
            offsets = ctx.int_offsets
        inplace = ctx.opts[1]
        if inplace and grad.stride(-1) != 1:
            grad = grad.contiguous()
        # an in-place forward lets the gradient be turned in place too: it belongs to this node alone
        dx = _Turn._run(grad, ctx.turns, ctx.opts, offsets, ((cos, sin), (cos_k, sin_k)), True, inplace)
        return (dx,) + (None,) * 7


def apply_rotary_emb(x, cos, sin, interleaved=False, inplace=False, seqlen_offsets: Union[int, torch.Tensor] = 0,
                     cu_seqlens: Optional[torch.Tensor] = None, max_seqlen: Optional[int] = None):
    """Rotates the first rotary_dim of every row of x.

    x: (batch, seqlen, nheads, headdim), or (total_seqlen, nheads, headdim) together with cu_seqlens and
    max_seqlen.  cos, sin: (seqlen_rotary, rotary_dim / 2).  interleaved: pairs are (even, odd) dimensions
    (GPT-J) instead of (first half, second half) (GPT-NeoX).  seqlen_offsets: an int, or one int per batch
    entry: position of each sequence's first row (decoding with a KV cache)."""
    opts = (bool(interleaved), bool(inplace), cu_seqlens, max_seqlen)
    return _Turn.apply(x, _turns_x, opts, seqlen_offsets, cos, sin, None, None)


apply_rotary_emb_func = apply_rotary_emb  # the reference keeps this older name too


def apply_rotary_emb_qkv_(qkv, cos, sin, cos_k=None, sin_k=None, interleaved=False,
                          seqlen_offsets: Union[int, torch.Tensor] = 0):
    """In place on q and k of qkv (batch, seqlen, 3, nheads, headdim); returns qkv.  cos_k, sin_k: separate
    tables for the keys (XPos); the queries' tables serve both when they are None."""
    if (cos_k is None) != (sin_k is None):
        raise ValueError("cos_k and sin_k come together")
    opts = (bool(interleaved), True, None, None)
    return _Turn.apply(qkv, _turns_qkv, opts, seqlen_offsets, cos, sin, cos_k, sin_k)


def apply_rotary_emb_kv_(kv, cos, sin, interleaved=False, seqlen_offsets: Union[int, torch.Tensor] = 0):
    """In place on k of kv (batch, seqlen, 2, nheads, headdim); returns kv."""
    opts = (bool(interleaved), True, None, None)
    return _Turn.apply(kv, _turns_kv, opts, seqlen_offsets, cos, sin, None, None)


# ------------------------------------------------------------------------------------------------
# The module: angle tables made on demand
class _AngleTables:
    """cos / sin of position x frequency for positions [0, rows), in the activations' dtype, for one device.

    With XPos (`xpos` = (per-pair base, scale_base)) queries and keys get reciprocal magnitudes
    zeta ** (+-(position - rows // 2) / scale_base), so that their product depends on the distance alone."""

    def __init__(self):
        self.rows, self.q, self.k = 0, (None, None), (None, None)

    def stale(self, rows, device, dtype, training):
        c = self.q[0]
        return (c is None or rows > self.rows or c.device != device or c.dtype != dtype
                # tables made under torch.inference_mode() cannot enter an autograd graph later
                or (training and c.is_inference()))

    def build(self, rows, freq, xpos, device, dtype):
        pos = torch.arange(rows, device=device, dtype=freq.dtype)
        angle = pos[:, None] * freq[None, :]
        c, s = angle.cos(), angle.sin()
        self.rows = rows
        if xpos is None:
            self.q, self.k = (c.to(dtype), s.to(dtype)), (None, None)
            return
        zeta, scale_base = xpos
        exponent = (torch.arange(rows, device=zeta.device, dtype=zeta.dtype) - rows // 2) / scale_base
        mag = (zeta.to(exponent.device)[None, :] ** exponent[:, None]).to(device)
        self.q = ((c * mag).to(dtype), (s * mag).to(dtype))
        self.k = ((c / mag).to(dtype), (s / mag).to(dtype))


class RotaryEmbedding(torch.nn.Module):
    """Rotary embedding of q and k in front of attention (RoFormer), optionally with XPos magnitudes.

    RotaryEmbedding(dim, base=10000.0, interleaved=False, scale_base=None, pos_idx_in_fp32=True, device=None);
    forward(qkv, kv=None, seqlen_offset=0, max_seqlen=None) turns, in place, q and k of a packed
    (batch, seqlen, 3, nheads, headdim) tensor, or q = `qkv` (batch, seqlen, nheads, headdim) and k inside
    `kv` (batch, seqlen, 2, nheads_k, headdim), and returns what it was given.  Frequencies are
    base ** (-2i / dim); with pos_idx_in_fp32 positions and frequencies stay fp32 whatever dtype the module was
    cast to (bf16 cannot tell position 257 from 256).  The tables grow with the longest sequence seen."""

    def __init__(self, dim: int, base=10000.0, interleaved=False, scale_base=None, pos_idx_in_fp32=True, device=None):
        super().__init__()
        self.dim, self.base, self.interleaved = dim, float(base), interleaved
        self.scale_base, self.pos_idx_in_fp32 = scale_base, pos_idx_in_fp32
        self.register_buffer("inv_freq", self._frequencies(device), persistent=False)
        zeta = None
        if scale_base is not None:
            pair = torch.arange(0, dim, 2, device=device, dtype=torch.float32)
            zeta = (pair + 0.4 * dim) / (1.4 * dim)  # XPos: per-pair base in (0.29, 1)
        self.register_buffer("scale", zeta, persistent=False)
        self._tables = _AngleTables()

    def _frequencies(self, device=None):
        pair = torch.arange(0, self.dim, 2, device=device, dtype=torch.float32)
        return torch.reciprocal(self.base ** (pair / self.dim))  # rounded like the published tables: 1 / base^(2i/dim)

    # what flash_attn/modules/mha.py reads when it hands the tables to the KV-cache kernel
    _cos_cached = property(lambda self: self._tables.q[0])
    _sin_cached = property(lambda self: self._tables.q[1])
    _cos_k_cached = property(lambda self: self._tables.k[0])
    _sin_k_cached = property(lambda self: self._tables.k[1])
    _seq_len_cached = property(lambda self: self._tables.rows)

    def _update_cos_sin_cache(self, seqlen, device=None, dtype=None):
        if not self._tables.stale(seqlen, device, dtype, self.training):
            return
        freq = self.inv_freq
        if self.pos_idx_in_fp32 and freq.dtype != torch.float32:
            freq = self._frequencies(device)  # the buffer was cast with the module; take the exact values again
        xpos = None if self.scale is None else (self.scale, self.scale_base)
        self._tables.build(seqlen, freq.to(device), xpos, device, dtype)

    def forward(self, qkv: torch.Tensor, kv: Optional[torch.Tensor] = None, seqlen_offset: Union[int, torch.Tensor] = 0,
                max_seqlen: Optional[int] = None):
        """seqlen_offset: int, or one int per batch entry (then pass max_seqlen, the longest position + 1 that
        can occur, so the tables can be sized without reading the tensor back)."""
        if max_seqlen is not None:
            self._update_cos_sin_cache(max_seqlen, device=qkv.device, dtype=qkv.dtype)
        elif isinstance(seqlen_offset, int):
            self._update_cos_sin_cache(qkv.shape[1] + seqlen_offset, device=qkv.device, dtype=qkv.dtype)
        (cq, sq), (ck, sk) = self._tables.q, self._tables.k
        how = dict(interleaved=self.interleaved, seqlen_offsets=seqlen_offset)
        if kv is None:
            return apply_rotary_emb_qkv_(qkv, cq, sq, ck, sk, **how)
        q = apply_rotary_emb(qkv, cq, sq, inplace=True, **how)
        if ck is None:
            ck, sk = cq, sq
        return q, apply_rotary_emb_kv_(kv, ck, sk, **how)
