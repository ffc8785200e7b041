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
