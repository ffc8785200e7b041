"""Rotary position embedding in front of attention: the public functions of the reference's
flash_attn/layers/rotary.py (apply_rotary_emb :96-124, apply_rotary_emb_qkv_ :207-231,
apply_rotary_emb_kv_ :271-292, RotaryEmbedding :295-480) with the same arguments and autograd
behaviour, on top of the `fa_rotary` entry point of the C ABI instead of the Triton kernel
(flash_attn/ops/triton/rotary.py).  The backward of a rotation is the rotation by the negative
angle (`conjugate`), so no activations are saved besides the tables.
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


class ApplyRotaryEmb(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, interleaved=False, inplace=False, seqlen_offsets: Union[int, torch.Tensor] = 0,
                cu_seqlens: Optional[torch.Tensor] = None, max_seqlen: Optional[int] = None):
        out = apply_rotary(x, cos, sin, seqlen_offsets=seqlen_offsets, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen,
                           interleaved=interleaved, inplace=inplace)
        if isinstance(seqlen_offsets, int):
            ctx.save_for_backward(cos, sin, cu_seqlens)
            ctx.seqlen_offsets = seqlen_offsets
        else:
            ctx.save_for_backward(cos, sin, cu_seqlens, seqlen_offsets)
            ctx.seqlen_offsets = None
        ctx.interleaved, ctx.inplace, ctx.max_seqlen = interleaved, inplace, max_seqlen
        return out if not inplace else x

    @staticmethod
    def backward(ctx, do):
        seqlen_offsets = ctx.seqlen_offsets
        if seqlen_offsets is None:
            cos, sin, cu_seqlens, seqlen_offsets = ctx.saved_tensors
        else:
            cos, sin, cu_seqlens = ctx.saved_tensors
        dx = apply_rotary(do, cos, sin, seqlen_offsets=seqlen_offsets, cu_seqlens=cu_seqlens, max_seqlen=ctx.max_seqlen,
                          interleaved=ctx.interleaved, inplace=ctx.inplace and do.stride(-1) == 1, conjugate=True)
        return dx, None, None, None, None, None, None, None


def apply_rotary_emb(x, cos, sin, interleaved=False, inplace=False, seqlen_offsets: Union[int, torch.Tensor] = 0,
                     cu_seqlens: Optional[torch.Tensor] = None, max_seqlen: Optional[int] = None):
    """x: (batch_size, seqlen, nheads, headdim), or (total_seqlen, nheads, headdim) with cu_seqlens.
    cos, sin: (seqlen_rotary, rotary_dim / 2).  interleaved: rotate pairs of even and odd dimensions
    (GPT-J style) instead of first and second half (GPT-NeoX style).  seqlen_offsets: int or (batch_size,):
    shift of every sequence, as used with a KV cache.  Rotates the first rotary_dim of every row."""
    return ApplyRotaryEmb.apply(x, cos, sin, interleaved, inplace, seqlen_offsets, cu_seqlens, max_seqlen)


apply_rotary_emb_func = apply_rotary_emb  # name kept by the reference for backward compatibility


def _rotate_qk_(qkv, cos, sin, cos_k, sin_k, interleaved, seqlen_offsets, conjugate):
    """In-place rotation of q and k inside a (batch, seqlen, 3, nheads, headdim) tensor."""
    batch, seqlen, three, nheads, headdim = qkv.shape
    if cos_k is None and sin_k is None and qkv.is_contiguous():
        # q and k heads are adjacent in memory: one call over 2 * nheads heads
        qk = qkv[:, :, :2].reshape(batch, seqlen, -1, headdim)
        apply_rotary(qk, cos, sin, seqlen_offsets=seqlen_offsets, interleaved=interleaved, inplace=True, conjugate=conjugate)
    else:
        cos_k = cos if cos_k is None else cos_k
        sin_k = sin if sin_k is None else sin_k
        apply_rotary(qkv[:, :, 0], cos, sin, seqlen_offsets, interleaved=interleaved, inplace=True, conjugate=conjugate)
        apply_rotary(qkv[:, :, 1], cos_k, sin_k, seqlen_offsets, interleaved=interleaved, inplace=True, conjugate=conjugate)


class ApplyRotaryEmbQKV_(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cos, sin, cos_k=None, sin_k=None, interleaved=False, seqlen_offsets: Union[int, torch.Tensor] = 0):
        assert qkv.shape[2] == 3
        _rotate_qk_(qkv, cos, sin, cos_k, sin_k, interleaved, seqlen_offsets, False)
        if isinstance(seqlen_offsets, int):
            ctx.save_for_backward(cos, sin, cos_k, sin_k)
            ctx.seqlen_offsets = seqlen_offsets
        else:
            ctx.save_for_backward(cos, sin, cos_k, sin_k, seqlen_offsets)
            ctx.seqlen_offsets = None
        ctx.interleaved = interleaved
        return qkv

    @staticmethod
    def backward(ctx, dqkv):
        seqlen_offsets = ctx.seqlen_offsets
        if seqlen_offsets is None:
            cos, sin, cos_k, sin_k, seqlen_offsets = ctx.saved_tensors
        else:
            cos, sin, cos_k, sin_k = ctx.saved_tensors
        if dqkv.stride(-1) != 1:
            dqkv = dqkv.contiguous()
        _rotate_qk_(dqkv, cos, sin, cos_k, sin_k, ctx.interleaved, seqlen_offsets, True)
        return dqkv, None, None, None, None, None, None


def apply_rotary_emb_qkv_(qkv, cos, sin, cos_k=None, sin_k=None, interleaved=False,
                          seqlen_offsets: Union[int, torch.Tensor] = 0):
    """qkv: (batch_size, seqlen, 3, nheads, headdim); cos, sin (and optionally cos_k, sin_k for the
    keys): (seqlen, rotary_dim / 2).  Rotates the first rotary_dim of Q and K *in place*."""
    return ApplyRotaryEmbQKV_.apply(qkv, cos, sin, cos_k, sin_k, interleaved, seqlen_offsets)


class ApplyRotaryEmbKV_(torch.autograd.Function):
    @staticmethod
    def forward(ctx, kv, cos, sin, interleaved=False, seqlen_offsets: Union[int, torch.Tensor] = 0):
        assert kv.shape[2] == 2
        apply_rotary(kv[:, :, 0], cos, sin, seqlen_offsets=seqlen_offsets, interleaved=interleaved, inplace=True)
        if isinstance(seqlen_offsets, int):
            ctx.save_for_backward(cos, sin)
            ctx.seqlen_offsets = seqlen_offsets
        else:
            ctx.save_for_backward(cos, sin, seqlen_offsets)
            ctx.seqlen_offsets = None
        ctx.interleaved = interleaved
        return kv

    @staticmethod
    def backward(ctx, dkv):
        seqlen_offsets = ctx.seqlen_offsets
        if seqlen_offsets is None:
            cos, sin, seqlen_offsets = ctx.saved_tensors
        else:
            cos, sin = ctx.saved_tensors
        if dkv.stride(-1) != 1:
            dkv = dkv.contiguous()
        apply_rotary(dkv[:, :, 0], cos, sin, seqlen_offsets=seqlen_offsets, interleaved=ctx.interleaved, inplace=True,
                     conjugate=True)
        return dkv, None, None, None, None


def apply_rotary_emb_kv_(kv, cos, sin, interleaved=False, seqlen_offsets: Union[int, torch.Tensor] = 0):
    """kv: (batch_size, seqlen, 2, nheads, headdim).  Rotates the first rotary_dim of K *in place*."""
    return ApplyRotaryEmbKV_.apply(kv, cos, sin, interleaved, seqlen_offsets)


class RotaryEmbedding(torch.nn.Module):
    """Rotary position embedding with cached cos / sin tables and optional XPos scaling
    (flash_attn/layers/rotary.py:295-480): forward(qkv, kv=None, seqlen_offset=0, max_seqlen=None)
    rotates q and k in place, either inside a packed qkv (kv is None) or q in `qkv` and k in `kv`."""

    def __init__(self, dim: int, base=10000.0, interleaved=False, scale_base=None, pos_idx_in_fp32=True, device=None):
        super().__init__()
        self.dim = dim
        self.base = float(base)
        self.pos_idx_in_fp32 = pos_idx_in_fp32
        self.register_buffer("inv_freq", self._compute_inv_freq(device), persistent=False)
        self.interleaved = interleaved
        self.scale_base = scale_base
        scale = ((torch.arange(0, dim, 2, device=device, dtype=torch.float32) + 0.4 * dim) / (1.4 * dim)
                 if scale_base is not None else None)
        self.register_buffer("scale", scale, persistent=False)
        self._seq_len_cached = 0
        self._cos_cached = self._sin_cached = self._cos_k_cached = self._sin_k_cached = None

    def _compute_inv_freq(self, device=None):
        return 1.0 / (self.base ** (torch.arange(0, self.dim, 2, device=device, dtype=torch.float32) / self.dim))

    def _update_cos_sin_cache(self, seqlen, device=None, dtype=None):
        # rebuilt when the sequence grows, the device or dtype changes, or the cache was made under inference mode
        if (seqlen > self._seq_len_cached or self._cos_cached is None or self._cos_cached.device != device
                or self._cos_cached.dtype != dtype or (self.training and self._cos_cached.is_inference())):
            self._seq_len_cached = seqlen
            if self.pos_idx_in_fp32:
                # positions and frequencies in fp32: bf16 positions would collide past 256
                t = torch.arange(seqlen, device=device, dtype=torch.float32)
                inv_freq = self.inv_freq if self.inv_freq.dtype == torch.float32 else self._compute_inv_freq(device=device)
            else:
                t = torch.arange(seqlen, device=device, dtype=self.inv_freq.dtype)
                inv_freq = self.inv_freq
            freqs = torch.outer(t, inv_freq)
            if self.scale is None:
                self._cos_cached = torch.cos(freqs).to(dtype)
                self._sin_cached = torch.sin(freqs).to(dtype)
            else:
                power = (torch.arange(seqlen, dtype=self.scale.dtype, device=self.scale.device) - seqlen // 2) / self.scale_base
                scale = self.scale.to(device=power.device) ** power.unsqueeze(-1)
                self._cos_cached = (torch.cos(freqs) * scale).to(dtype)
                self._sin_cached = (torch.sin(freqs) * scale).to(dtype)
                self._cos_k_cached = (torch.cos(freqs) / scale).to(dtype)
                self._sin_k_cached = (torch.sin(freqs) / scale).to(dtype)

    def forward(self, qkv: torch.Tensor, kv: Optional[torch.Tensor] = None, seqlen_offset: Union[int, torch.Tensor] = 0,
                max_seqlen: Optional[int] = None):
        seqlen = qkv.shape[1]
        if max_seqlen is not None:
            self._update_cos_sin_cache(max_seqlen, device=qkv.device, dtype=qkv.dtype)
        elif isinstance(seqlen_offset, int):
            self._update_cos_sin_cache(seqlen + seqlen_offset, device=qkv.device, dtype=qkv.dtype)
        if kv is None:
            if self.scale is None:
                return apply_rotary_emb_qkv_(qkv, self._cos_cached, self._sin_cached, interleaved=self.interleaved,
                                             seqlen_offsets=seqlen_offset)
            return apply_rotary_emb_qkv_(qkv, self._cos_cached, self._sin_cached, self._cos_k_cached, self._sin_k_cached,
                                         interleaved=self.interleaved, seqlen_offsets=seqlen_offset)
        q = apply_rotary_emb_func(qkv, self._cos_cached, self._sin_cached, interleaved=self.interleaved, inplace=True,
                                  seqlen_offsets=seqlen_offset)
        if self.scale is None:
            kv = apply_rotary_emb_kv_(kv, self._cos_cached, self._sin_cached, interleaved=self.interleaved,
                                      seqlen_offsets=seqlen_offset)
        else:
            kv = apply_rotary_emb_kv_(kv, self._cos_k_cached, self._sin_k_cached, interleaved=self.interleaved,
                                      seqlen_offsets=seqlen_offset)
        return q, kv
