"""The CPU oracle against the golden vectors produced by the reference's own functions
(tests/golden/make_golden.py -> tests/golden/reference_cases.pt)."""
import os

import pytest
import torch

from golden.make_golden import make_inputs
from oracle import attention_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_cases.pt")
CASES = torch.load(GOLDEN, weights_only=False)["cases"]


def _inputs(case):
    if "q" in case:
        return case["q"], case["k"], case["v"], case["dout"]
    _, q, k, v, do = make_inputs(*case["recipe"])
    return q, k, v, do


@pytest.mark.parametrize("case", [c for c in CASES if c["kind"] == "attention"], ids=lambda c: c["name"])
def test_attention_oracle_matches_reference(case):
    q, k, v, do = _inputs(case)
    ss = case["subsample"]
    qf, kf, vf = (x.clone().requires_grad_(True) for x in (q, k, v))
    out, attn = O.attention_oracle(qf, kf, vf, case["query_padding_mask"], case["key_padding_mask"], case["dropout_p"],
                                   case["dropout_mask"], causal=case["causal"], window_size=case["window_size"])
    dq, dk, dv = torch.autograd.grad(out, (qf, kf, vf), do)
    # same fp32 math, different op order: allow a few ulps of the 16-bit output type
    tol = dict(atol=2e-3, rtol=2e-2)
    assert torch.allclose(out.detach()[:, ::ss].float(), case["out"].float(), **tol)
    assert torch.allclose(attn.detach()[:, :, ::ss, ::ss].float(), case["attn"].float(), **tol)
    for mine, ref in ((dq, case["dq"]), (dk, case["dk"]), (dv, case["dv"])):
        scale = ref.float().abs().max().item() + 1e-6
        assert (mine[:, ::ss].float() - ref.float()).abs().max().item() <= 1e-2 * scale
    lowp, _ = O.attention_oracle(q, k, v, case["query_padding_mask"], case["key_padding_mask"], case["dropout_p"],
                                 case["dropout_mask"], causal=case["causal"], window_size=case["window_size"],
                                 upcast=False, reorder_ops=True)
    # the low-precision yardstick must have the same error scale as the reference's
    e_mine = (lowp[:, ::ss].float() - case["out"].float()).abs().max().item()
    e_ref = (case["out_lowp"].float() - case["out"].float()).abs().max().item()
    assert e_mine <= 2 * e_ref + 2e-3


@pytest.mark.parametrize("case", [c for c in CASES if c["kind"] == "rotary"], ids=lambda c: c["name"])
def test_rotary_oracle_matches_reference(case):
    out = O.rotary_oracle(case["x"].float(), case["cos"].float(), case["sin"].float(), case["offsets"], case["interleaved"])
    assert torch.allclose(out.to(case["x"].dtype).float(), case["out"].float(), atol=1e-2, rtol=1e-2)
    lowp = O.rotary_oracle(case["x"], case["cos"], case["sin"], case["offsets"], case["interleaved"])
    assert torch.allclose(lowp.float(), case["out_lowp"].float(), atol=2e-2, rtol=2e-2)


def test_lse_oracle_is_consistent_with_attention():
    # softmax = exp(scale*s - lse): rebuild the reference's attention matrix from the oracle LSE
    case = next(c for c in CASES if c["name"] == "padded_causal")
    q, k, v, _ = _inputs(case)
    lse = O.lse_oracle(q, k, case["key_padding_mask"], case["query_padding_mask"], causal=True)
    B, Sq, H, D = q.shape
    kk = k.float().repeat_interleave(H // k.shape[2], dim=2)
    s = torch.einsum("bthd,bshd->bhts", q.float(), kk) / D ** 0.5
    probs = torch.exp(s - lse.unsqueeze(-1))
    ref = case["attn"].float()
    vis = ref > 0
    assert torch.allclose(probs[vis], ref[vis], atol=4e-3, rtol=2e-2)


def test_causal_alignment_examples():
    # the two examples in the docstring of flash_attn_func (flash_attn/flash_attn_interface.py:668-678)
    m = O.visibility_mask(2, 5, (-1, 0)).int().tolist()
    assert m == [[1, 1, 1, 1, 0], [1, 1, 1, 1, 1]]
    m = O.visibility_mask(5, 2, (-1, 0)).int().tolist()
    assert m == [[0, 0], [0, 0], [0, 0], [1, 0], [1, 1]]


def test_merge_oracle_equals_unsplit():
    g = torch.Generator().manual_seed(5)
    q = torch.randn(1, 7, 2, 16, generator=g)
    k = torch.randn(1, 40, 2, 16, generator=g)
    v = torch.randn(1, 40, 2, 16, generator=g)
    full, _ = O.attention_oracle(q, k, v)
    parts, lses = [], []
    for lo, hi in ((0, 16), (16, 17), (17, 40)):
        o, _ = O.attention_oracle(q, k[:, lo:hi], v[:, lo:hi])
        parts.append(o.permute(0, 2, 1, 3).reshape(-1, 16))
        lses.append(O.lse_oracle(q, k[:, lo:hi]).reshape(-1))
    out, lse = O.merge_oracle(torch.stack(parts), torch.stack(lses))
    assert torch.allclose(out, full.permute(0, 2, 1, 3).reshape(-1, 16), atol=1e-5)
    assert torch.allclose(lse, O.lse_oracle(q, k).reshape(-1), atol=1e-5)
    # all-empty parts
    out, lse = O.merge_oracle(torch.zeros(2, 3, 4), torch.full((2, 3), float("-inf")))
    assert torch.all(out == 0) and torch.all(torch.isinf(lse) & (lse > 0))


def test_kvcache_oracle_appends_and_rotates():
    g = torch.Generator().manual_seed(9)
    B, Sk, H, Hk, D = 2, 24, 4, 2, 16
    q = torch.randn(B, 1, H, D, generator=g)
    kc, vc = torch.randn(3, Sk, Hk, D, generator=g), torch.randn(3, Sk, Hk, D, generator=g)
    kn, vn = torch.randn(B, 1, Hk, D, generator=g), torch.randn(B, 1, Hk, D, generator=g)
    ang = torch.rand(Sk, D // 2, generator=g) * 6.28
    cos, sin = torch.cos(ang), torch.sin(ang)
    lens = torch.tensor([5, 17], dtype=torch.int32)
    idx = torch.tensor([2, 0], dtype=torch.int32)
    out, kc2, vc2 = O.kvcache_oracle(q, kc, vc, kn, vn, cos, sin, lens, idx, rotary_interleaved=False)
    for b in range(B):
        L = int(lens[b])
        assert torch.equal(vc2[b, L], vn[b, 0])
        assert torch.equal(kc2[b, :L], kc[int(idx[b]), :L])
        kr = O.rotary_oracle(kn[b:b + 1], cos, sin, L, False)
        assert torch.allclose(kc2[b, L], kr[0, 0])
        # attention over exactly L + 1 keys
        qr = O.rotary_oracle(q[b:b + 1], cos, sin, L, False)
        ref, _ = O.attention_oracle(qr, kc2[b:b + 1, :L + 1], vc2[b:b + 1, :L + 1])
        assert torch.allclose(out[b], ref[0], atol=1e-5)
