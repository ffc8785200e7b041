"""Shared helpers of the GPU parity tests: the tolerance rule and oracle drivers."""
import torch

from oracle import attention_oracle as O


def assert_within(x, truth, lowp, mult=2.0, atol=1e-3, what=""):
    """|x - truth| <= mult * |lowp - truth| + atol  (max norm).

    `truth` is the oracle in fp32, `lowp` the same oracle computed in the 16-bit input type: the
    acceptance rule of the reference's tests (tests/test_flash_attn.py:650-657) with the absolute
    slack of 1e-3 that this build's contract adds.
    """
    err = (x.float() - truth.float()).abs().max().item()
    yard = (lowp.float() - truth.float()).abs().max().item()
    assert err == err, "%s: NaN in result" % what
    assert err <= mult * yard + atol, "%s: err %.3e > %g * %.3e + %g" % (what, err, mult, yard, atol)
    return err, yard


def oracle_fwd_bwd(q, k, v, dout, **kw):
    """(out, dq, dk, dv, lse) from the fp32 oracle and (out, dq, dk, dv) from the low-precision one."""
    res = []
    for upcast in (True, False):
        qf, kf, vf = (x.detach().clone().requires_grad_(True) for x in (q, k, v))
        out, _ = O.attention_oracle(qf, kf, vf, upcast=upcast, reorder_ops=not upcast, **kw)
        if dout is not None:
            dq, dk, dv = torch.autograd.grad(out, (qf, kf, vf), dout)
        else:
            dq = dk = dv = None
        res.append((out.detach(), dq, dk, dv))
    return res[0], res[1]


def make_qkv(B, Sq, Sk, H, Hk, D, dtype, seed=0, device="cuda"):
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn(B, Sq, H, D, generator=g).to(dtype).to(device)
    k = torch.randn(B, Sk, Hk, D, generator=g).to(dtype).to(device)
    v = torch.randn(B, Sk, Hk, D, generator=g).to(dtype).to(device)
    do = torch.randn(B, Sq, H, D, generator=g).to(dtype).to(device)
    return q, k, v, do


def kvcache_truth(q, k_cache, v_cache, k_new, v_new, cos, sin, cache_seqlens, rotary_interleaved=False, causal=True):
    """(out fp32 truth, out 16-bit yardstick, expected K cache, expected V cache) of a decode step with append +
    rotary.  The kernel rotates in fp32 and rounds once, as the reference's rotary op does in its own KV-cache test
    (tests/test_flash_attn.py:1758-1797): the rotation is therefore done here in fp32 and rounded to the storage
    type before the attention oracle runs."""
    B, Sq, H, D = q.shape
    dt = q.dtype
    cosf, sinf = cos.float(), sin.float()
    if causal:
        q_r = O.rotary_oracle(q.float(), cosf, sinf, cache_seqlens, rotary_interleaved).to(dt)
    else:
        q_r = O.rotary_oracle(q.float().reshape(B, 1, Sq * H, D), cosf, sinf, cache_seqlens, rotary_interleaved).reshape(B, Sq, H, D).to(dt)
    k_r = O.rotary_oracle(k_new.float(), cosf, sinf, cache_seqlens, rotary_interleaved).to(dt)
    kw = dict(cache_seqlens=cache_seqlens, causal=causal)
    out_t, kc_t, vc_t = O.kvcache_oracle(q_r, k_cache, v_cache, k_r, v_new, None, None, **kw)
    out_l, _, _ = O.kvcache_oracle(q_r, k_cache, v_cache, k_r, v_new, None, None, upcast=False, reorder_ops=True, **kw)
    return out_t, out_l, kc_t, vc_t
