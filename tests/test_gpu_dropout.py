"""Dropout: API kept, validated statistically through the returned sign-encoded probabilities
(the role of S_dmask in tests/test_flash_attn.py:592-657), and forward/backward consistency."""
import pytest
import torch

from gpu_util import assert_within, make_qkv
from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    import flash_attention_b200 as fa


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("d,h,hk", [(64, 4, 4), (128, 6, 2), (40, 4, 1)])
@pytest.mark.parametrize("sq,sk", [(128, 128), (203, 317), (512, 512)])
def test_dropout_mask_fraction_and_parity(sq, sk, d, h, hk, causal, dtype):
    p_drop = 0.17
    q, k, v, do = make_qkv(3, sq, sk, h, hk, d, dtype, seed=sq + d)
    q, k, v = (x.requires_grad_(True) for x in (q, k, v))
    torch.manual_seed(42)
    out, lse, s_dmask = fa.flash_attn_func(q, k, v, dropout_p=p_drop, causal=causal, return_attn_probs=True)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), do)
    probs = s_dmask[:, :, :sq, :sk]
    # returned matrix = softmax probabilities, sign bit marks dropped entries
    _, attn_t = O.attention_oracle(q.detach(), k.detach(), v.detach(), causal=causal)
    assert (probs.abs().float() - attn_t.float()).abs().max().item() <= 2e-2
    visible = attn_t.float() > 1e-6
    dropped = (probs < 0) & visible
    frac = dropped.sum().item() / max(1, visible.sum().item())
    # keep iff byte <= floor(p_keep*255): drop probability = 1 - (floor(p_keep*255)+1)/256
    expect = 1.0 - (int((1 - p_drop) * 255) + 1) / 256.0
    assert abs(frac - expect) < 0.01, (frac, expect)
    keep_mask = ~(probs < 0)
    # outputs and gradients equal the oracle's with THIS mask
    res = []
    for upcast in (True, False):
        qf, kf, vf = (x.detach().clone().requires_grad_(True) for x in (q, k, v))
        o, _ = O.attention_oracle(qf, kf, vf, None, None, p_drop, keep_mask, causal=causal, upcast=upcast,
                                  reorder_ops=not upcast)
        res.append((o.detach(),) + torch.autograd.grad(o, (qf, kf, vf), do))
    (o_t, dq_t, dk_t, dv_t), (o_l, dq_l, dk_l, dv_l) = res
    assert_within(out.detach(), o_t, o_l, what="out")
    assert_within(dq, dq_t, dq_l, what="dq")
    assert_within(dk, dk_t, dk_l, what="dk")
    assert_within(dv, dv_t, dv_l, what="dv")


def test_dropout_seed_controls_the_mask():
    q, k, v, _ = make_qkv(1, 128, 128, 2, 2, 64, torch.float16, seed=1)
    torch.manual_seed(7)
    a = fa.flash_attn_func(q, k, v, dropout_p=0.3, return_attn_probs=True)[2]
    torch.manual_seed(7)
    b = fa.flash_attn_func(q, k, v, dropout_p=0.3, return_attn_probs=True)[2]
    c = fa.flash_attn_func(q, k, v, dropout_p=0.3, return_attn_probs=True)[2]
    assert torch.equal(a < 0, b < 0)
    assert not torch.equal(a < 0, c < 0)
