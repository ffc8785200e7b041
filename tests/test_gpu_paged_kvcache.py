"""Paged KV cache (block_table), return_softmax_lse and the deterministic switch: the arguments that later
versions of the upstream interface added to flash_attn_with_kvcache / the attention functions.

A paged call must equal the same call on the contiguous cache that the table describes: the contiguous
cache is cut into pages, the pages are scattered over a larger pool in random order, and the oracle runs on
the contiguous form.  Output against the oracle (fp32 truth, 16-bit yardstick), appended K within 1e-3, V
bit-equal, pages that no sequence owns untouched."""
import math

import pytest
import torch

from gpu_util import assert_within, kvcache_truth
from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    import flash_attention_b200 as fa
    from flash_attention_b200 import _lib


def _to_pages(cache, page, n_extra, gen):
    """cache (B, cap, Hk, D) -> (pool (B * cap/page + n_extra, page, Hk, D), table (B, cap/page) int32)."""
    B, cap, Hk, D = cache.shape
    per = cap // page
    n = B * per + n_extra
    perm = torch.randperm(n, generator=gen)[: B * per]
    pool = torch.randn(n, page, Hk, D, generator=gen).to(cache.dtype).to(cache.device)
    pool[perm.to(cache.device)] = cache.reshape(B * per, page, Hk, D)
    return pool, perm.reshape(B, per).to(torch.int32).to(cache.device)


def _from_pages(pool, table):
    B, per = table.shape
    return pool[table.long().reshape(-1)].reshape(B, per * pool.shape[1], pool.shape[2], pool.shape[3])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("num_splits", [0, 1, 3])
@pytest.mark.parametrize("page", [64, 256])
@pytest.mark.parametrize("d,H,Hk", [(128, 8, 2), (64, 4, 4)])
def test_paged_decode_step_with_append_and_rotary(d, H, Hk, page, num_splits, dtype):
    g = torch.Generator().manual_seed(d + page + num_splits)
    B, cap = 5, 2048
    q = torch.randn(B, 1, H, d, generator=g).to(dtype).cuda()
    kc = torch.randn(B, cap, Hk, d, generator=g).to(dtype).cuda()
    vc = torch.randn(B, cap, Hk, d, generator=g).to(dtype).cuda()
    k_new = torch.randn(B, 1, Hk, d, generator=g).to(dtype).cuda()
    v_new = torch.randn(B, 1, Hk, d, generator=g).to(dtype).cuda()
    lens = torch.tensor([0, page - 1, page, 1000, cap - 1], dtype=torch.int32).cuda()  # page edges, empty, almost full
    ang = torch.rand(cap, d // 2, generator=g) * 2 * math.pi
    cos, sin = ang.cos().to(dtype).cuda(), ang.sin().to(dtype).cuda()
    gp = torch.Generator().manual_seed(7)
    k_pool, table = _to_pages(kc, page, 9, gp)
    gp = torch.Generator().manual_seed(7)
    v_pool, table_v = _to_pages(vc, page, 9, gp)
    assert torch.equal(table, table_v)
    k_pool0, v_pool0 = k_pool.clone(), v_pool.clone()
    out, lse = fa.flash_attn_with_kvcache(q, k_pool, v_pool, k_new, v_new, cos, sin, lens, causal=True,
                                          rotary_interleaved=False, num_splits=num_splits, block_table=table,
                                          return_softmax_lse=True)
    assert _lib.last_path().startswith("decode")
    out_t, out_l, kc_t, vc_t = kvcache_truth(q, kc, vc, k_new, v_new, cos, sin, lens)
    assert_within(out, out_t, out_l, mult=3, atol=1e-3, what="out")
    assert torch.allclose(_from_pages(k_pool, table).float(), kc_t.float(), rtol=1e-3, atol=1e-3)
    assert torch.equal(_from_pages(v_pool, table), vc_t)
    owned = torch.zeros(k_pool.shape[0], dtype=torch.bool, device="cuda")
    owned[table.long().reshape(-1)] = True
    assert torch.equal(k_pool[~owned], k_pool0[~owned]) and torch.equal(v_pool[~owned], v_pool0[~owned])
    # the returned log-sum-exp is that of the scaled scores over the visible keys
    q_r = O.rotary_oracle(q.float().reshape(B, 1, H, d), cos.float(), sin.float(), lens, False).to(dtype).float()
    for b in range(B):
        L = int(lens[b]) + 1
        kk = kc_t[b, :L].float().repeat_interleave(H // Hk, dim=1)  # (L, H, d)
        s = torch.einsum("hd,lhd->hl", q_r[b, 0], kk) * d ** -0.5
        assert torch.allclose(lse[b, :, 0], torch.logsumexp(s, dim=-1), atol=2e-3, rtol=1e-3), b
    # and the contiguous call gives the same numbers bit for bit (same kernel, same tiles)
    kc2, vc2 = kc.clone(), vc.clone()
    out2 = fa.flash_attn_with_kvcache(q, kc2, vc2, k_new, v_new, cos, sin, lens, causal=True, rotary_interleaved=False,
                                      num_splits=num_splits)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("seqlen_q,d,causal,window", [(5, 96, True, (-1, -1)), (16, 128, False, (300, 40)), (3, 40, True, (-1, -1))])
def test_paged_cache_on_the_any_shape_path_with_tokens_straddling_a_page(seqlen_q, d, causal, window):
    g = torch.Generator().manual_seed(seqlen_q + d)
    B, H, Hk, page, cap = 3, 6, 3, 128, 1024
    dtype = torch.bfloat16
    q = torch.randn(B, seqlen_q, H, d, generator=g).to(dtype).cuda()
    kc = torch.randn(B, cap, Hk, d, generator=g).to(dtype).cuda()
    vc = torch.randn(B, cap, Hk, d, generator=g).to(dtype).cuda()
    k_new = torch.randn(B, seqlen_q, Hk, d, generator=g).to(dtype).cuda()
    v_new = torch.randn(B, seqlen_q, Hk, d, generator=g).to(dtype).cuda()
    lens = torch.tensor([page - 2, 0, cap - seqlen_q], dtype=torch.int32).cuda()  # the first one crosses into the next page
    gp = torch.Generator().manual_seed(11)
    k_pool, table = _to_pages(kc, page, 4, gp)
    gp = torch.Generator().manual_seed(11)
    v_pool, _ = _to_pages(vc, page, 4, gp)
    out = fa.flash_attn_with_kvcache(q, k_pool, v_pool, k_new, v_new, cache_seqlens=lens, causal=causal,
                                     window_size=window, block_table=table)
    assert _lib.last_path().startswith("kvcache_prep+fwd_generic")
    kw = dict(cache_seqlens=lens, causal=causal, window_size=window)
    out_t, kc_t, vc_t = O.kvcache_oracle(q, kc, vc, k_new, v_new, None, None, **kw)
    out_l, _, _ = O.kvcache_oracle(q, kc, vc, k_new, v_new, None, None, upcast=False, reorder_ops=True, **kw)
    assert_within(out, out_t, out_l, mult=3, atol=1e-3, what="out")
    assert torch.equal(_from_pages(k_pool, table), kc_t) and torch.equal(_from_pages(v_pool, table), vc_t)


def test_paged_cache_argument_errors():
    q = torch.zeros(2, 1, 4, 64, dtype=torch.float16, device="cuda")
    pool = torch.zeros(8, 64, 4, 64, dtype=torch.float16, device="cuda")
    table = torch.zeros(2, 4, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="cache_batch_idx"):
        fa.flash_attn_with_kvcache(q, pool, pool, cache_seqlens=3, block_table=table,
                                   cache_batch_idx=torch.zeros(2, dtype=torch.int32, device="cuda"))
    with pytest.raises(RuntimeError, match="divisible by 64"):
        fa.flash_attn_with_kvcache(q, pool[:, :32], pool[:, :32], cache_seqlens=3, block_table=table)
    with pytest.raises(RuntimeError, match="int32"):
        fa.flash_attn_with_kvcache(q, pool, pool, cache_seqlens=3, block_table=table.long())


def test_deterministic_switch_makes_dq_reproducible_on_the_any_shape_backward():
    """With dropout the backward runs on the any-shape kernel, whose dq is summed with fp32 atomics; with
    deterministic=True it is launched per key block and dq is bit-identical from run to run, and equal to
    the unordered result up to the order of fp32 additions."""
    g = torch.Generator().manual_seed(5)
    B, S, H, D = 2, 700, 4, 64
    q, k, v, do = (torch.randn(B, S, H, D, generator=g).half().cuda() for _ in range(4))

    def run(det):
        torch.manual_seed(123)  # same dropout mask every time
        qq, kk, vv = (x.clone().requires_grad_() for x in (q, k, v))
        out = fa.flash_attn_func(qq, kk, vv, dropout_p=0.2, causal=True, deterministic=det)
        grads = torch.autograd.grad(out, (qq, kk, vv), do)
        assert _lib.last_path() == "bwd_generic"
        return (out.detach(),) + grads

    ref = run(True)
    for _ in range(10):
        cur = run(True)
        assert all(torch.equal(a, b) for a, b in zip(cur, ref))
    loose = run(False)
    assert torch.equal(loose[0], ref[0]) and torch.equal(loose[2], ref[2]) and torch.equal(loose[3], ref[3])
    assert (loose[1].float() - ref[1].float()).abs().max().item() <= 2e-2
