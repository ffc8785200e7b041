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


def test_decode_loop_in_a_cuda_graph():
    """The decode step (append one token with rotary + attend) captured once in a CUDA graph and
    replayed for several tokens, as the generation loop of the reference does
    (flash_attn/utils/generation.py:662-700): every replay must give what eager calls give, and the
    cache must end up identical.  The lengths live on the device and advance between replays."""
    import flash_attention_b200 as fa

    g = torch.Generator().manual_seed(11)
    B, cap, H, Hk, D, steps = 4, 512, 8, 2, 128, 6
    dev = "cuda"
    kc0 = torch.randn(B, cap, Hk, D, generator=g).bfloat16().to(dev)
    vc0 = torch.randn(B, cap, Hk, D, generator=g).bfloat16().to(dev)
    lens0 = torch.tensor([17, 130, 255, 300], dtype=torch.int32, device=dev)
    qs = torch.randn(steps, B, 1, H, D, generator=g).bfloat16().to(dev)
    kn = torch.randn(steps, B, 1, Hk, D, generator=g).bfloat16().to(dev)
    vn = torch.randn(steps, B, 1, Hk, D, generator=g).bfloat16().to(dev)
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2, device=dev).float() / D))
    fr = torch.outer(torch.arange(cap, device=dev).float(), inv)
    cos, sin = torch.cos(fr).bfloat16(), torch.sin(fr).bfloat16()

    def eager():
        kc, vc, lens = kc0.clone(), vc0.clone(), lens0.clone()
        outs = []
        for t in range(steps):
            outs.append(fa.flash_attn_with_kvcache(qs[t], kc, vc, kn[t], vn[t], cos, sin, lens, causal=True,
                                                   rotary_interleaved=False).clone())
            lens += 1
        return outs, kc, vc

    want, kc_want, vc_want = eager()
    kc, vc, lens = kc0.clone(), vc0.clone(), lens0.clone()
    q_in, k_in, v_in = qs[0].clone(), kn[0].clone(), vn[0].clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # warm-up on the capture stream, then restore the state it changed
        fa.flash_attn_with_kvcache(q_in, kc, vc, k_in, v_in, cos, sin, lens, causal=True, rotary_interleaved=False)
    torch.cuda.current_stream().wait_stream(side)
    kc.copy_(kc0)
    vc.copy_(vc0)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out_g = fa.flash_attn_with_kvcache(q_in, kc, vc, k_in, v_in, cos, sin, lens, causal=True, rotary_interleaved=False)
        lens += 1
    kc.copy_(kc0)
    vc.copy_(vc0)
    lens.copy_(lens0)
    for t in range(steps):
        q_in.copy_(qs[t])
        k_in.copy_(kn[t])
        v_in.copy_(vn[t])
        graph.replay()
        assert torch.equal(out_g, want[t]), t
    torch.cuda.synchronize()
    assert torch.equal(kc, kc_want) and torch.equal(vc, vc_want)
    assert torch.equal(lens, lens0 + steps)
