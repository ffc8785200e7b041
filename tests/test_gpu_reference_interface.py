"""The UNMODIFIED python interface of FlashAttention v2.3.3 (flash_attn/flash_attn_interface.py: the
four _flash_attn_* wrappers at :44-190, six autograd Functions at :193-548, seven public functions at
:551-1042) running on this repository's `flash_attn_2_cuda` module, forward and backward, on the GPU.

The file is loaded as it is from an installed copy of the reference: the tree named by the
environment variable FLASH_ATTN_REFERENCE_TREE, else the python-only install under baseline/_ref of
this repository (pip install --target, no CUDA build); without either the module is skipped.
"""
import importlib.util
import os

import pytest
import torch

from gpu_util import assert_within, kvcache_truth, oracle_fwd_bwd
from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _interface_file():
    for r in (os.environ.get("FLASH_ATTN_REFERENCE_TREE"), os.path.join(ROOT, "baseline", "_ref")):
        if r and os.path.exists(os.path.join(r, "flash_attn", "flash_attn_interface.py")):
            return os.path.join(r, "flash_attn", "flash_attn_interface.py")
    return None


@pytest.fixture(scope="module")
def ref():
    path = _interface_file()
    if path is None:
        pytest.skip("no copy of the reference's flash_attn package on this machine")
    import flash_attn_2_cuda as ext

    assert os.path.dirname(os.path.abspath(ext.__file__)).startswith(ROOT), "an unrelated flash_attn_2_cuda shadows the shim"
    spec = importlib.util.spec_from_file_location("flash_attn_interface_v233", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.flash_attn_cuda is ext
    return mod


def _inputs(B, Sq, Sk, H, Hk, D, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g).to(dtype).cuda()  # noqa: E731
    return mk(B, Sq, H, D), mk(B, Sk, Hk, D), mk(B, Sk, Hk, D), mk(B, Sq, H, D)


def _compare(out, grads, q, k, v, do, **kw):
    (o_t, dq_t, dk_t, dv_t), (o_l, dq_l, dk_l, dv_l) = oracle_fwd_bwd(q, k, v, do, **kw)
    assert_within(out, o_t, o_l, what="out")
    for name, mine, t, l in (("dq", grads[0], dq_t, dq_l), ("dk", grads[1], dk_t, dk_l), ("dv", grads[2], dv_t, dv_l)):
        assert_within(mine, t, l, what=name)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("D,H,Hk", [(128, 16, 16), (64, 8, 2), (96, 6, 6), (256, 4, 1)])
def test_flash_attn_func_and_packed_variants(ref, D, H, Hk, causal):
    B, Sq, Sk = 4, 640, 640
    q, k, v, do = _inputs(B, Sq, Sk, H, Hk, D, torch.bfloat16, seed=D + H)
    # flash_attn_func
    qg, kg, vg = (x.clone().requires_grad_(True) for x in (q, k, v))
    out, lse, _ = ref.flash_attn_func(qg, kg, vg, causal=causal, return_attn_probs=True)
    grads = torch.autograd.grad(out, (qg, kg, vg), do)
    _compare(out.detach(), grads, q, k, v, do, causal=causal)
    lse_t = O.lse_oracle(q, k, causal=causal)
    assert (lse - lse_t).abs().max().item() <= 1e-3
    # flash_attn_kvpacked_func: same numbers from the packed (B, S, 2, Hk, D) tensor
    kv = torch.stack((k, v), dim=2).requires_grad_(True)
    qg = q.clone().requires_grad_(True)
    out2 = ref.flash_attn_kvpacked_func(qg, kv, causal=causal)
    dq2, dkv2 = torch.autograd.grad(out2, (qg, kv), do)
    assert torch.equal(out2, out)
    assert torch.equal(dq2, grads[0]) and torch.equal(dkv2[:, :, 0], grads[1]) and torch.equal(dkv2[:, :, 1], grads[2])
    # flash_attn_qkvpacked_func (needs H == Hk)
    if H == Hk:
        qkv = torch.stack((q, k, v), dim=2).requires_grad_(True)
        out3 = ref.flash_attn_qkvpacked_func(qkv, causal=causal)
        (dqkv,) = torch.autograd.grad(out3, qkv, do)
        assert torch.equal(out3, out)
        assert all(torch.equal(dqkv[:, :, i], grads[i]) for i in range(3))


@pytest.mark.parametrize("window", [(-1, -1), (100, 0), (30, 70)])
def test_flash_attn_func_windows_and_odd_head_dim(ref, window):
    q, k, v, do = _inputs(2, 333, 517, 6, 3, 72, torch.float16, seed=7)
    qg, kg, vg = (x.clone().requires_grad_(True) for x in (q, k, v))
    out = ref.flash_attn_func(qg, kg, vg, window_size=window)
    grads = torch.autograd.grad(out, (qg, kg, vg), do)
    _compare(out.detach(), grads, q, k, v, do, window_size=window)


@pytest.mark.parametrize("causal", [False, True])
def test_varlen_functions(ref, causal):
    H, Hk, D = 8, 2, 128
    lens = [77, 1, 300, 129, 512]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32).cuda()
    tot = sum(lens)
    g = torch.Generator().manual_seed(11)
    mk = lambda *s: torch.randn(*s, generator=g).half().cuda()  # noqa: E731
    q, k, v, do = mk(tot, H, D), mk(tot, Hk, D), mk(tot, Hk, D), mk(tot, H, D)
    qg, kg, vg = (x.clone().requires_grad_(True) for x in (q, k, v))
    out = ref.flash_attn_varlen_func(qg, kg, vg, cu, cu, max(lens), max(lens), causal=causal)
    dq, dk, dv = torch.autograd.grad(out, (qg, kg, vg), do)
    for i, n in enumerate(lens):
        s = slice(int(cu[i]), int(cu[i + 1]))
        _compare(out.detach()[s][None], (dq[s][None], dk[s][None], dv[s][None]), q[s][None], k[s][None], v[s][None], do[s][None],
                 causal=causal)
    kv = torch.stack((k, v), dim=1).requires_grad_(True)
    qg = q.clone().requires_grad_(True)
    out2 = ref.flash_attn_varlen_kvpacked_func(qg, kv, cu, cu, max(lens), max(lens), causal=causal)
    dq2, dkv2 = torch.autograd.grad(out2, (qg, kv), do)
    assert torch.equal(out2, out) and torch.equal(dq2, dq) and torch.equal(dkv2[:, 0], dk) and torch.equal(dkv2[:, 1], dv)
    # qkv-packed needs equal head counts
    k4, v4 = k.repeat_interleave(H // Hk, dim=1), v.repeat_interleave(H // Hk, dim=1)
    qkv = torch.stack((q, k4, v4), dim=1).requires_grad_(True)
    out3 = ref.flash_attn_varlen_qkvpacked_func(qkv, cu, max(lens), causal=causal)
    (dqkv,) = torch.autograd.grad(out3, qkv, do)
    for i, n in enumerate(lens):
        s = slice(int(cu[i]), int(cu[i + 1]))
        _compare(out3.detach()[s][None], (dqkv[s, 0][None], dqkv[s, 1][None], dqkv[s, 2][None]), q[s][None], k4[s][None],
                 v4[s][None], do[s][None], causal=causal)


def test_dropout_returns_usable_mask(ref):
    # return_attn_probs with dropout: the sign-encoded probabilities give the mask that reproduces the output
    q, k, v, do = _inputs(2, 256, 256, 4, 4, 64, torch.float16, seed=3)
    out, lse, p = ref.flash_attn_func(q, k, v, dropout_p=0.2, causal=True, return_attn_probs=True)
    keep = p[:, :, :256, :256] >= 0
    frac = 1.0 - keep.float().mean().item() / 1.0
    o_t, _ = O.attention_oracle(q, k, v, dropout_p=0.2, dropout_mask=keep, causal=True)
    o_l, _ = O.attention_oracle(q, k, v, dropout_p=0.2, dropout_mask=keep, causal=True, upcast=False, reorder_ops=True)
    assert_within(out, o_t, o_l, what="out with dropout")
    assert 0.05 < frac < 0.35


def test_flash_attn_with_kvcache(ref):
    B, cap, H, Hk, D = 5, 4096, 16, 4, 128
    g = torch.Generator().manual_seed(5)
    mk = lambda *s: torch.randn(*s, generator=g).bfloat16().cuda()  # noqa: E731
    kc, vc, q, kn, vn = mk(B, cap, Hk, D), mk(B, cap, Hk, D), mk(B, 1, H, D), mk(B, 1, Hk, D), mk(B, 1, Hk, D)
    lens = torch.tensor([0, 1, 700, 4000, 4095], dtype=torch.int32).cuda()
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2).float() / D))
    fr = torch.outer(torch.arange(cap).float(), inv)
    cos, sin = torch.cos(fr).bfloat16().cuda(), torch.sin(fr).bfloat16().cuda()
    kc0, vc0 = kc.clone(), vc.clone()
    out = ref.flash_attn_with_kvcache(q, kc, vc, kn, vn, rotary_cos=cos, rotary_sin=sin, cache_seqlens=lens, causal=True,
                                      rotary_interleaved=False)
    o_t, o_l, kc_t, vc_t = kvcache_truth(q, kc0, vc0, kn, vn, cos, sin, lens)
    assert_within(out, o_t, o_l, mult=3, what="kvcache out")
    assert torch.equal(vc, vc_t)
    assert torch.allclose(kc.float(), kc_t.float(), atol=1e-3, rtol=1e-3)
