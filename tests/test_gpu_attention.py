"""GPU parity tests of forward and backward attention against the CPU/GPU-agnostic oracle.

Everything goes through the public API -> flash_attn_2_cuda shim -> C ABI of libfa_b200.so.
The lattice follows the reference's tests/test_flash_attn.py (head dims :536, sequence pairs
:799-813, MHA/MQA/GQA :787, local windows :832, varlen :1043, causal alignment :1323).
"""
import math
import os

import pytest
import torch

from gpu_util import assert_within, make_qkv, oracle_fwd_bwd
from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    import flash_attention_b200 as fa
    from flash_attention_b200 import _lib


class one_pass_forward:
    """Pins the forward to a single pass over the keys (no split-KV), so that a small problem, which the
    split heuristic would hand to the split path, runs on the kernel that large problems take."""

    def __enter__(self):
        self.old = os.environ.get("FA_B200_FWD_SPLITS")
        os.environ["FA_B200_FWD_SPLITS"] = "1"

    def __exit__(self, *a):
        if self.old is None:
            del os.environ["FA_B200_FWD_SPLITS"]
        else:
            os.environ["FA_B200_FWD_SPLITS"] = self.old


def _run(q, k, v, do, fwd_path=None, bwd_path=None, **kw):
    q, k, v = (x.detach().clone().requires_grad_(True) for x in (q, k, v))
    out, lse, _ = fa.flash_attn_func(q, k, v, return_attn_probs=True, **kw)
    if fwd_path is not None:
        assert _lib.last_path() == fwd_path, "forward took %r, the case is meant for %r" % (_lib.last_path(), fwd_path)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), do)
    if bwd_path is not None:
        assert _lib.last_path() == bwd_path, "backward took %r, the case is meant for %r" % (_lib.last_path(), bwd_path)
    return out.detach(), lse, dq, dk, dv


def _check(q, k, v, do, causal=False, window=(-1, -1), grads=True, fwd_path=None, bwd_path=None):
    out, lse, dq, dk, dv = _run(q, k, v, do, causal=causal, window_size=window, fwd_path=fwd_path, bwd_path=bwd_path)
    # The kernels treat a one-sided window as unbounded on the other side (set_params_fprop,
    # csrc/flash_attn/flash_api.cpp:113-114); attention_ref takes the -1 literally, so the oracle
    # is given seqlen_k for the open side.
    sk = k.shape[1]
    if window[0] >= 0 and window[1] < 0 and not causal:
        window = (window[0], sk)
    elif window[0] < 0 and (window[1] >= 0 or causal):
        window = (sk, 0 if causal else window[1])
    (o_t, dq_t, dk_t, dv_t), (o_l, dq_l, dk_l, dv_l) = oracle_fwd_bwd(q, k, v, do, causal=causal, window_size=window)
    assert_within(out, o_t, o_l, what="out")
    lse_t = O.lse_oracle(q, k, causal=causal, window_size=window)
    fin = torch.isfinite(lse_t)
    assert torch.equal(torch.isfinite(lse), fin), "LSE: +inf pattern differs"
    assert (lse[fin] - lse_t[fin]).abs().max().item() <= 1e-3 if fin.any() else True
    if grads:
        assert_within(dq, dq_t, dq_l, what="dq")
        assert_within(dk, dk_t, dk_l, what="dk")
        assert_within(dv, dv_t, dv_l, what="dv")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("d", [32, 40, 59, 64, 80, 96, 111, 128, 160, 192, 224, 256])
@pytest.mark.parametrize("sq,sk", [(113, 203), (128, 217), (1, 147), (512, 256), (384, 384)])
def test_mha_head_dims(sq, sk, d, causal, dtype):
    q, k, v, do = make_qkv(2, sq, sk, 4, 4, d, dtype, seed=d + sq)
    _check(q, k, v, do, causal=causal)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("d", [32, 40, 59, 64, 80, 96, 111, 128, 160, 192, 224, 256])
@pytest.mark.parametrize("sq,sk", [(113, 203), (128, 217), (1, 147), (512, 256), (384, 384)])
def test_mha_head_dims_on_the_tensor_core_kernels(sq, sk, d, causal, dtype):
    # the lattice above at the same small sizes, but pinned to the kernels that large problems run on:
    # single-pass tcgen05 forward, tcgen05 backward (two kernels up to head dim 128, three passes above)
    q, k, v, do = make_qkv(2, sq, sk, 4, 4, d, dtype, seed=d + sq)
    with one_pass_forward():
        _check(q, k, v, do, causal=causal, fwd_path="fwd_tc", bwd_path="bwd_wide_tc" if d > 128 else "bwd_tc+bwd_dq_tc")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("local", [False, True])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("hk", [1, 3, 9])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("sq,sk", [(108, 256), (256, 512), (1023, 1024), (1024, 1023), (2048, 2048), (339, 97)])
def test_gqa_and_windows(sq, sk, d, hk, causal, local, dtype):
    g = torch.Generator().manual_seed(sq * 7 + sk)
    window = tuple(torch.randint(0, sk, (2,), generator=g).tolist()) if local else (-1, -1)
    q, k, v, do = make_qkv(2, sq, sk, 9, hk, d, dtype, seed=sq + hk)
    _check(q, k, v, do, causal=causal, window=window)


@pytest.mark.parametrize("window", [(-1, -1), (64, 0), (200, 17), (0, 0), (-1, 5), (33, -1)])
@pytest.mark.parametrize("sq,sk", [(300, 300), (257, 640), (640, 257)])
def test_window_edges(sq, sk, window):
    q, k, v, do = make_qkv(1, sq, sk, 2, 2, 128, torch.bfloat16, seed=3)
    _check(q, k, v, do, window=window)
    with one_pass_forward():
        _check(q, k, v, do, window=window, fwd_path="fwd_tc", bwd_path="bwd_tc+bwd_dq_tc")


def test_qkvpacked_and_kvpacked_match_unpacked():
    B, S, H, D = 2, 300, 4, 64
    g = torch.Generator().manual_seed(1)
    qkv = torch.randn(B, S, 3, H, D, generator=g).bfloat16().cuda().requires_grad_(True)
    do = torch.randn(B, S, H, D, generator=g).bfloat16().cuda()
    out = fa.flash_attn_qkvpacked_func(qkv, causal=True)
    (dqkv,) = torch.autograd.grad(out, qkv, do)
    q, k, v = (qkv.detach()[:, :, i].contiguous() for i in range(3))
    out2, _, dq, dk, dv = _run(q, k, v, do, causal=True)
    assert torch.equal(out, out2)
    assert torch.equal(dqkv[:, :, 1], dk) and torch.equal(dqkv[:, :, 2], dv)
    assert torch.allclose(dqkv[:, :, 0].float(), dq.float(), atol=2e-2, rtol=2e-2)  # dq is atomically accumulated
    kv = torch.stack((k, v), dim=2).requires_grad_(True)
    out3 = fa.flash_attn_kvpacked_func(q, kv, causal=True)
    assert torch.equal(out3, out2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal,window", [(False, (-1, -1)), (True, (-1, -1)), (False, (50, 10))])
@pytest.mark.parametrize("d,h,hk", [(128, 4, 4), (64, 6, 2), (96, 4, 1), (192, 4, 2), (256, 2, 2)])
def test_varlen(d, h, hk, causal, window, dtype):
    g = torch.Generator().manual_seed(d + h)
    lens_q = torch.randint(1, 400, (5,), generator=g).tolist()
    lens_k = [max(1, l + int(torch.randint(-20, 60, (1,), generator=g))) for l in lens_q]
    cu_q = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32).cuda()
    cu_k = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32).cuda()
    tq, tk = sum(lens_q), sum(lens_k)
    q = torch.randn(tq, h, d, generator=g).to(dtype).cuda().requires_grad_(True)
    k = torch.randn(tk, hk, d, generator=g).to(dtype).cuda().requires_grad_(True)
    v = torch.randn(tk, hk, d, generator=g).to(dtype).cuda().requires_grad_(True)
    do = torch.randn(tq, h, d, generator=g).to(dtype).cuda()
    out, lse, _ = fa.flash_attn_varlen_func(q, k, v, cu_q, cu_k, max(lens_q), max(lens_k), causal=causal,
                                            window_size=window, return_attn_probs=True)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), do)
    for i in range(len(lens_q)):
        sq, sk = slice(int(cu_q[i]), int(cu_q[i + 1])), slice(int(cu_k[i]), int(cu_k[i + 1]))
        qi, ki, vi, doi = q.detach()[sq][None], k.detach()[sk][None], v.detach()[sk][None], do[sq][None]
        (o_t, dq_t, dk_t, dv_t), (o_l, dq_l, dk_l, dv_l) = oracle_fwd_bwd(qi, ki, vi, doi, causal=causal, window_size=window)
        assert_within(out.detach()[sq][None], o_t, o_l, what="out[%d]" % i)
        assert_within(dq[sq][None], dq_t, dq_l, what="dq[%d]" % i)
        assert_within(dk[sk][None], dk_t, dk_l, what="dk[%d]" % i)
        assert_within(dv[sk][None], dv_t, dv_l, what="dv[%d]" % i)
        lse_t = O.lse_oracle(qi, ki, causal=causal, window_size=window)[0]
        mine = lse[i, :, : lens_q[i]]
        fin = torch.isfinite(lse_t)
        assert torch.equal(torch.isfinite(mine), fin)
        if fin.any():
            assert (mine[fin] - lse_t[fin]).abs().max().item() <= 1e-3


def test_varlen_single_key_sequences_have_no_nan():
    # the regression of tests/test_flash_attn.py:2048-2073: cu_seqlens_k = [0, 1, 2, 3]
    g = torch.Generator().manual_seed(0)
    nheads, d = 5, 64
    cu_q = torch.tensor([0, 76, 110, 256], dtype=torch.int32).cuda()
    cu_k = torch.tensor([0, 1, 2, 3], dtype=torch.int32).cuda()
    q = (torch.randn(256, nheads, d, generator=g) * 5).half().cuda().requires_grad_(True)
    k = (torch.randn(3, nheads, d, generator=g) * 3).half().cuda().requires_grad_(True)
    v = (torch.randn(3, nheads, d, generator=g) * 3).half().cuda().requires_grad_(True)
    out = fa.flash_attn_varlen_func(q, k, v, cu_q, cu_k, 146, 1, causal=True)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), torch.randn_like(out))
    for t in (out, dq, dk, dv):
        assert not t.isnan().any()


def test_non_contiguous_dout():
    # tests/test_flash_attn.py:1996-2045: dout with a transposed layout
    q, k, v, _ = make_qkv(2, 200, 200, 4, 4, 64, torch.float16, seed=2)
    do = torch.randn(2, 4, 200, 64, generator=torch.Generator().manual_seed(4)).half().cuda().transpose(1, 2)
    assert not do.is_contiguous()
    _check(q, k, v, do, causal=True)


def test_deterministic_out_lse_dk_dv():
    # tests/test_flash_attn.py:1892-1930: out, lse, dk, dv bit-identical across reruns
    q, k, v, do = make_qkv(2, 500, 500, 4, 2, 128, torch.bfloat16, seed=8)
    ref = _run(q, k, v, do, causal=True)
    for _ in range(20):
        cur = _run(q, k, v, do, causal=True)
        assert torch.equal(cur[0], ref[0]) and torch.equal(cur[1], ref[1])
        assert torch.equal(cur[3], ref[3]) and torch.equal(cur[4], ref[4])
        assert (cur[2].float() - ref[2].float()).abs().max().item() <= 2e-2
    # on the tensor-core kernels nothing is accumulated atomically: dq is bit-identical too
    with one_pass_forward():
        ref = _run(q, k, v, do, causal=True, fwd_path="fwd_tc", bwd_path="bwd_tc+bwd_dq_tc")
        for _ in range(20):
            cur = _run(q, k, v, do, causal=True)
            assert all(torch.equal(x, y) for x, y in zip(cur, ref))


def test_backward_large_values_do_not_overflow():
    # tests/test_flash_attn.py:1940-1993
    g = torch.Generator().manual_seed(0)
    q = (torch.randn(2, 256, 5, 128, generator=g) * 5).half().cuda()
    k, v = ((torch.randn(2, 256, 5, 128, generator=g) * 3).half().cuda() for _ in range(2))
    do = torch.randn(2, 256, 5, 128, generator=g).half().cuda()
    out, lse, dq, dk, dv = _run(q, k, v, do, causal=True)
    (o_t, dq_t, dk_t, dv_t), (o_l, dq_l, dk_l, dv_l) = oracle_fwd_bwd(q, k, v, do, causal=True)
    assert_within(out, o_t, o_l, mult=2, what="out")
    assert_within(dq, dq_t, dq_l, mult=5, what="dq")
    assert_within(dk, dk_t, dk_l, mult=5, what="dk")
    assert_within(dv, dv_t, dv_l, mult=5, what="dv")


def test_tensor_core_and_any_shape_paths_agree():
    q, k, v, do = make_qkv(2, 700, 900, 8, 2, 128, torch.bfloat16, seed=12)
    a = _run(q, k, v, do, causal=True)
    os.environ["FA_B200_FORCE_GENERIC"] = "1"
    try:
        b_ = _run(q, k, v, do, causal=True)
    finally:
        del os.environ["FA_B200_FORCE_GENERIC"]
    assert (a[0].float() - b_[0].float()).abs().max().item() <= 8e-3
    assert (a[1] - b_[1]).abs().max().item() <= 1e-3
    for x, y in zip(a[2:], b_[2:]):
        assert (x.float() - y.float()).abs().max().item() <= 6e-2


def test_split_kv_forward_matches():
    # few query blocks, many keys -> the forward splits the keys and merges by LSE (flash_api.cpp:373-389)
    q, k, v, do = make_qkv(1, 64, 8192, 2, 2, 128, torch.float16, seed=5)
    _check(q, k, v, do, causal=False, grads=False)
    _check(q, k, v, do, causal=True, grads=False)


def test_golden_fixtures_on_gpu():
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_cases.pt")
    from golden.make_golden import make_inputs

    cases = torch.load(path, weights_only=False)["cases"]
    n = 0
    for c in cases:
        if c["kind"] != "attention" or c["dropout_p"] > 0 or c["query_padding_mask"] is not None or c["key_padding_mask"] is not None:
            continue
        if c["window_size"][0] >= 0 and c["window_size"][1] < 0:
            # attention_ref reads a right window of -1 literally, the kernels (reference and this one)
            # replace it by seqlen_k (flash_api.cpp:114): the fixture pins the oracle, not the kernel
            continue
        if "q" in c:
            q, k, v, do = c["q"], c["k"], c["v"], c["dout"]
        else:
            _, q, k, v, do = make_inputs(*c["recipe"])
        ss = c["subsample"]
        out, lse, dq, dk, dv = _run(q.cuda(), k.cuda(), v.cuda(), do.cuda(), causal=c["causal"], window_size=c["window_size"])
        assert_within(out[:, ::ss].cpu(), c["out"], c["out_lowp"], what=c["name"] + " out")
        for mine, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
            ref = c[key].float()
            assert (mine[:, ::ss].cpu().float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-3, c["name"] + key
        n += 1
    assert n >= 7


def test_error_behaviour():
    q, k, v, _ = make_qkv(1, 16, 16, 4, 3, 64, torch.float16)
    with pytest.raises(RuntimeError):
        fa.flash_attn_func(q, k, v)  # 4 heads are not a multiple of 3
    with pytest.raises(RuntimeError):
        fa.flash_attn_func(q.float(), k.float(), v.float())
    q, k, v, _ = make_qkv(1, 16, 16, 2, 2, 264, torch.float16)
    with pytest.raises(RuntimeError):
        fa.flash_attn_func(q, k, v)
