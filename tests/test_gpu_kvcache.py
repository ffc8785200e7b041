"""flash_attn_with_kvcache against the oracle: in-place append, rotary, cache_batch_idx, split-KV.
Lattice after tests/test_flash_attn.py:1662-1860 (K cache within 1e-3, V cache bit-equal)."""
import math

import pytest
import torch

from gpu_util import assert_within
from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    import flash_attention_b200 as fa


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("num_splits", [1, 0])
@pytest.mark.parametrize("mha_type", ["mha", "mqa", "gqa"])
@pytest.mark.parametrize("new_kv", [False, True])
@pytest.mark.parametrize("causal,local", [(False, False), (True, False), (False, True)])
@pytest.mark.parametrize("rotary_interleaved,rotary_fraction", [(False, 0.0), (False, 1.0), (True, 0.5)])
@pytest.mark.parametrize("has_batch_idx", [False, True])
@pytest.mark.parametrize("d", [64, 128, 59])
@pytest.mark.parametrize("seqlen_q,seqlen_k", [(1, 128), (1, 339), (3, 1024), (64, 800), (16, 20000), (1, 128 * 1024)])
def test_kvcache(seqlen_q, seqlen_k, d, has_batch_idx, rotary_interleaved, rotary_fraction, causal, local, new_kv,
                 mha_type, num_splits, dtype):
    if not new_kv and rotary_fraction > 0.0:
        pytest.skip("rotary needs new k/v")
    if seqlen_k > 4096 and (d != 128 or dtype != torch.bfloat16 or mha_type == "mqa"):
        pytest.skip("long caches are run on one dtype/head-dim to bound the suite")
    g = torch.Generator().manual_seed(seqlen_q * 31 + seqlen_k + d)
    dev = "cuda"
    batch = 2
    batch_c = batch if not has_batch_idx else batch * 2
    nheads = 6
    rotary_dim = math.floor(int(rotary_fraction * d) / 16) * 16
    nheads_k = nheads if mha_type == "mha" else (1 if mha_type == "mqa" else 3)
    window = (-1, -1) if not local else tuple(torch.randint(0, seqlen_k, (2,), generator=g).tolist())
    q = torch.randn(batch, seqlen_q, nheads, d, generator=g).to(dtype).to(dev)
    seqlen_new = seqlen_q
    k = v = None
    if new_kv:
        k = torch.randn(batch, seqlen_new, nheads_k, d, generator=g).to(dtype).to(dev)
        v = torch.randn(batch, seqlen_new, nheads_k, d, generator=g).to(dtype).to(dev)
    k_cache = torch.randn(batch_c, seqlen_k, nheads_k, d, generator=g).to(dtype).to(dev)
    v_cache = torch.randn(batch_c, seqlen_k, nheads_k, d, generator=g).to(dtype).to(dev)
    hi = (seqlen_k - seqlen_q + 1) if new_kv else (seqlen_k + 1)
    cache_seqlens = torch.randint(0, hi, (batch,), generator=g).to(torch.int32).to(dev)
    idx = torch.randperm(batch_c, generator=g)[:batch].to(torch.int32).to(dev) if has_batch_idx else None
    cos = sin = None
    if rotary_dim > 0:
        ang = torch.rand(seqlen_k, rotary_dim // 2, generator=g) * 2 * math.pi
        cos, sin = torch.cos(ang).to(dtype).to(dev), torch.sin(ang).to(dtype).to(dev)
    kc0, vc0 = k_cache.clone(), v_cache.clone()
    out = fa.flash_attn_with_kvcache(q, k_cache, v_cache, k, v, cos, sin, cache_seqlens, idx, causal=causal,
                                     window_size=window, rotary_interleaved=rotary_interleaved, num_splits=num_splits)
    # oracle: rotary in fp32 (what the kernel does), then rounded once
    cosf, sinf = (None, None) if cos is None else (cos.float(), sin.float())
    kw = dict(cache_seqlens=cache_seqlens, cache_batch_idx=idx, causal=causal, window_size=window,
              rotary_interleaved=rotary_interleaved)
    qf = q.float() if cos is not None else q
    kf = k.float() if (k is not None and cos is not None) else k
    if cos is not None:
        # rotate in fp32, round to the storage type, then attend
        if causal or local:
            q_r = O.rotary_oracle(qf, cosf, sinf, cache_seqlens, rotary_interleaved).to(dtype)
        else:
            q_r = O.rotary_oracle(qf.reshape(batch, 1, seqlen_q * nheads, d), cosf, sinf, cache_seqlens,
                                  rotary_interleaved).reshape(batch, seqlen_q, nheads, d).to(dtype)
        k_r = O.rotary_oracle(kf, cosf, sinf, cache_seqlens, rotary_interleaved).to(dtype)
    else:
        q_r, k_r = q, k
    kw2 = dict(kw)
    out_t, kc_t, vc_t = O.kvcache_oracle(q_r, kc0, vc0, k_r, v, None, None, **kw2)
    out_l, _, _ = O.kvcache_oracle(q_r, kc0, vc0, k_r, v, None, None, upcast=False, reorder_ops=True, **kw2)
    if new_kv:
        sel_k = k_cache if idx is None else k_cache[idx.long()]
        sel_v = v_cache if idx is None else v_cache[idx.long()]
        assert torch.allclose(sel_k.float(), kc_t.float(), rtol=1e-3, atol=1e-3)
        assert torch.equal(sel_v, vc_t)
    else:
        assert torch.equal(k_cache, kc0) and torch.equal(v_cache, vc0)
    assert_within(out, out_t, out_l, mult=3, atol=1e-3, what="out")


def test_kvcache_int_cache_seqlens_and_no_seqlens():
    g = torch.Generator().manual_seed(3)
    q = torch.randn(2, 1, 8, 128, generator=g).half().cuda()
    kc = torch.randn(2, 512, 2, 128, generator=g).half().cuda()
    vc = torch.randn(2, 512, 2, 128, generator=g).half().cuda()
    out = fa.flash_attn_with_kvcache(q, kc, vc, cache_seqlens=300)
    ref, _ = O.attention_oracle(q, kc[:, :300], vc[:, :300])
    low, _ = O.attention_oracle(q, kc[:, :300], vc[:, :300], upcast=False, reorder_ops=True)
    assert_within(out, ref, low, mult=3)
    out = fa.flash_attn_with_kvcache(q, kc, vc)
    ref, _ = O.attention_oracle(q, kc, vc)
    low, _ = O.attention_oracle(q, kc, vc, upcast=False, reorder_ops=True)
    assert_within(out, ref, low, mult=3)
