"""Parity at the full sizes of the benchmark configurations.

The kernels run the whole problem; the fp32 oracle (and its 16-bit yardstick) runs on the GPU on
slices that attention treats independently — one (batch, head) pair, one KV-head group, one packed
sequence, one cache line — because the score matrix of the whole problem does not fit anywhere.
Rule as everywhere: |x - truth| <= 2 |yardstick - truth| + 1e-3, LSE within 1e-3
(3x for the KV-cache step, as tests/test_flash_attn.py:1860 does).
"""
import math

import pytest
import torch

from gpu_util import assert_within, kvcache_truth
from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    import flash_attention_b200 as fa
    from flash_attention_b200 import _lib


def _oracle_head(q, k, v, do, causal, window):
    """fp32 truth and 16-bit yardstick of one (1, S, 1, D) problem: (out, dq, dk, dv) twice, gradients in fp32."""
    res = []
    for upcast in (True, False):
        qf, kf, vf = ((x.float() if upcast else x).detach().clone().requires_grad_(True) for x in (q, k, v))
        out, _ = O.attention_oracle(qf, kf, vf, causal=causal, window_size=window, upcast=upcast, reorder_ops=not upcast)
        dq, dk, dv = torch.autograd.grad(out, (qf, kf, vf), do.float() if upcast else do)
        res.append((out.detach().float(), dq.float(), dk.float(), dv.float()))
        del out, qf, kf, vf
    return res


def _check_lse(lse, q, k, causal, window):
    lse_t = O.lse_oracle(q, k, causal=causal, window_size=window)
    fin = torch.isfinite(lse_t)
    assert torch.equal(torch.isfinite(lse), fin), "LSE: +inf pattern differs"
    assert (lse[fin] - lse_t[fin]).abs().max().item() <= 1e-3


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("H,D", [(16, 128), (32, 64), (8, 256)])
def test_training_shape_qkvpacked(H, D, causal):
    # packed qkv (16, 2048, 3, H, D) bf16 and dout (16, 2048, H, D), N(0,1), through flash_attn_qkvpacked_func
    B, S = 16, 2048
    g = torch.Generator(device="cuda").manual_seed(1)
    qkv = torch.randn(B, S, 3, H, D, device="cuda", dtype=torch.bfloat16, generator=g).requires_grad_(True)
    do = torch.randn(B, S, H, D, device="cuda", dtype=torch.bfloat16, generator=g)
    out, lse, _ = fa.flash_attn_qkvpacked_func(qkv, causal=causal, return_attn_probs=True)
    assert _lib.last_path() == "fwd_tc"
    (dqkv,) = torch.autograd.grad(out, qkv, do)
    assert _lib.last_path() == ("bwd_wide_tc" if D > 128 else "bwd_tc+bwd_dq_tc")
    for b, h in ((0, 0), (7, H // 2 + 1), (15, H - 1)):
        q, k, v = (qkv.detach()[b:b + 1, :, i, h:h + 1] for i in range(3))
        (o_t, dq_t, dk_t, dv_t), (o_l, dq_l, dk_l, dv_l) = _oracle_head(q, k, v, do[b:b + 1, :, h:h + 1], causal, (-1, -1))
        tag = " b%d h%d" % (b, h)
        assert_within(out.detach()[b:b + 1, :, h:h + 1], o_t, o_l, what="out" + tag)
        assert_within(dqkv[b:b + 1, :, 0, h:h + 1], dq_t, dq_l, what="dq" + tag)
        assert_within(dqkv[b:b + 1, :, 1, h:h + 1], dk_t, dk_l, what="dk" + tag)
        assert_within(dqkv[b:b + 1, :, 2, h:h + 1], dv_t, dv_l, what="dv" + tag)
        _check_lse(lse[b:b + 1, h:h + 1], q, k, causal, (-1, -1))


@pytest.mark.parametrize("causal,window", [(True, (-1, -1)), (False, (4096, 0))])
def test_long_context_gqa(causal, window):
    # batch 1, 32768 tokens, 32 query heads over 8 KV heads, head dim 128, bf16; causal and sliding window
    S, H, Hk, D = 32768, 32, 8, 128
    grp = H // Hk
    g = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn(1, S, H, D, device="cuda", dtype=torch.bfloat16, generator=g).requires_grad_(True)
    k = torch.randn(1, S, Hk, D, device="cuda", dtype=torch.bfloat16, generator=g).requires_grad_(True)
    v = torch.randn(1, S, Hk, D, device="cuda", dtype=torch.bfloat16, generator=g).requires_grad_(True)
    do = torch.randn(1, S, H, D, device="cuda", dtype=torch.bfloat16, generator=g)
    out, lse, _ = fa.flash_attn_func(q, k, v, causal=causal, window_size=window, return_attn_probs=True)
    assert _lib.last_path() == "fwd_tc"
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), do)
    assert _lib.last_path() == "bwd_tc+bwd_dq_tc"
    for hk in (0, Hk - 1):  # two KV-head groups: dk / dv of a group sum over its four query heads
        dk_t = dv_t = dk_l = dv_l = 0
        for h in range(hk * grp, (hk + 1) * grp):
            qh, kh, vh, doh = q.detach()[:, :, h:h + 1], k.detach()[:, :, hk:hk + 1], v.detach()[:, :, hk:hk + 1], do[:, :, h:h + 1]
            (o_t, dq_t, dk1_t, dv1_t), (o_l, dq_l, dk1_l, dv1_l) = _oracle_head(qh, kh, vh, doh, causal, window)
            assert_within(out.detach()[:, :, h:h + 1], o_t, o_l, what="out h%d" % h)
            assert_within(dq[:, :, h:h + 1], dq_t, dq_l, what="dq h%d" % h)
            _check_lse(lse[:, h:h + 1], qh, kh, causal, window)
            dk_t, dv_t, dk_l, dv_l = dk_t + dk1_t, dv_t + dv1_t, dk_l + dk1_l, dv_l + dv1_l
            del o_t, o_l, dq_t, dq_l, dk1_t, dv1_t, dk1_l, dv1_l
            torch.cuda.empty_cache()
        assert_within(dk[:, :, hk:hk + 1], dk_t, dk_l, what="dk group %d" % hk)
        assert_within(dv[:, :, hk:hk + 1], dv_t, dv_l, what="dv group %d" % hk)


def test_packed_varlen_fp16():
    # lengths ~ U[128, 4096] until 65536 tokens (the last one clipped), 16 heads, head dim 128, fp16, causal
    H, D = 16, 128
    gl = torch.Generator().manual_seed(3)
    lens, total = [], 0
    while total < 65536:
        n = int(torch.randint(128, 4097, (1,), generator=gl))
        n = min(n, 65536 - total)
        lens.append(n)
        total += n
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(3)
    q, k, v = (torch.randn(total, H, D, device="cuda", dtype=torch.float16, generator=g).requires_grad_(True) for _ in range(3))
    do = torch.randn(total, H, D, device="cuda", dtype=torch.float16, generator=g)
    out, lse, _ = fa.flash_attn_varlen_func(q, k, v, cu, cu, max(lens), max(lens), causal=True, return_attn_probs=True)
    assert _lib.last_path() == "fwd_tc"
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), do)
    assert _lib.last_path() == "bwd_tc+bwd_dq_tc"
    picks = sorted({0, len(lens) - 1, lens.index(min(lens)), lens.index(max(lens)), len(lens) // 2})
    for i in picks:
        s = slice(int(cu[i]), int(cu[i + 1]))
        for h in (0, 9, H - 1):
            qi, ki, vi, doi = (x.detach()[s, h:h + 1][None] for x in (q, k, v, do))
            (o_t, dq_t, dk_t, dv_t), (o_l, dq_l, dk_l, dv_l) = _oracle_head(qi, ki, vi, doi, True, (-1, -1))
            tag = " seq %d (len %d) h%d" % (i, lens[i], h)
            assert_within(out.detach()[s, h:h + 1][None], o_t, o_l, what="out" + tag)
            assert_within(dq[s, h:h + 1][None], dq_t, dq_l, what="dq" + tag)
            assert_within(dk[s, h:h + 1][None], dk_t, dk_l, what="dk" + tag)
            assert_within(dv[s, h:h + 1][None], dv_t, dv_l, what="dv" + tag)
            _check_lse(lse[i:i + 1, h:h + 1, :lens[i]], qi, ki, True, (-1, -1))


def test_decode_step_batch64_capacity32768():
    # 64 sequences, 32 query heads over 8 KV heads, head dim 128, bf16 cache of capacity 32768, lengths
    # uniform in [1024, 32767], one new token appended in-kernel with non-interleaved rotary
    B, cap, H, Hk, D = 64, 32768, 32, 8, 128
    g = torch.Generator(device="cuda").manual_seed(4)
    kc = torch.randn(B, cap, Hk, D, device="cuda", dtype=torch.bfloat16, generator=g)
    vc = torch.randn(B, cap, Hk, D, device="cuda", dtype=torch.bfloat16, generator=g)
    lens = torch.randint(1024, 32768, (B,), device="cuda", generator=g).to(torch.int32)
    q = torch.randn(B, 1, H, D, device="cuda", dtype=torch.bfloat16, generator=g)
    kn = torch.randn(B, 1, Hk, D, device="cuda", dtype=torch.bfloat16, generator=g)
    vn = torch.randn(B, 1, Hk, D, device="cuda", dtype=torch.bfloat16, generator=g)
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    fr = torch.outer(torch.arange(cap, device="cuda").float(), inv)
    cos, sin = torch.cos(fr).bfloat16(), torch.sin(fr).bfloat16()
    picks = sorted({0, B - 1, int(lens.argmin()), int(lens.argmax()), 31})
    before = {b: (kc[b].clone(), vc[b].clone()) for b in picks}
    k_sum, v_sum = kc.float().sum(dim=(2, 3)), vc.float().sum(dim=(2, 3))  # per (sequence, position) checksums
    out = fa.flash_attn_with_kvcache(q, kc, vc, kn, vn, cos, sin, lens, causal=True, rotary_interleaved=False)
    assert _lib.last_path() == "decode+combine"
    # only position lens[b] of every sequence may have changed
    pos = torch.arange(cap, device="cuda").view(1, cap) == lens.view(B, 1).long()
    assert torch.equal(kc.float().sum(dim=(2, 3))[~pos], k_sum[~pos])
    assert torch.equal(vc.float().sum(dim=(2, 3))[~pos], v_sum[~pos])
    for b in picks:
        kb, vb = before[b]
        sl = slice(b, b + 1)
        o_t, o_l, kc_t, vc_t = kvcache_truth(q[sl], kb[None], vb[None], kn[sl], vn[sl], cos, sin, lens[sl])
        assert_within(out[sl], o_t, o_l, mult=3, what="out seq %d (len %d)" % (b, int(lens[b])))
        assert torch.equal(vc[sl], vc_t), "V cache line %d" % b
        assert torch.allclose(kc[sl].float(), kc_t.float(), atol=1e-3, rtol=1e-3), "K cache line %d" % b
