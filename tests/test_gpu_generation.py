"""The decode caller path on the GPU: prefill + token-by-token decoding through the KV cache must give what
one causal pass over the whole sequence gives (the property the reference's generation tests rest on,
tests/models/test_gpt.py greedy-decoding checks), eagerly and through captured CUDA graphs; and the
reference's own unmodified MHA module (flash_attn/modules/mha.py) generates on this repository's kernels."""
import importlib
import math
import os
import sys
import types

import pytest
import torch

from gpu_util import assert_within
from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rotary_tables(rot_dim, rows, dtype):
    inv = 1.0 / (10000.0 ** (torch.arange(0, rot_dim, 2, dtype=torch.float32) / rot_dim))
    ang = torch.outer(torch.arange(rows, dtype=torch.float32), inv)
    return ang.cos().to(dtype).cuda(), ang.sin().to(dtype).cuda()


@pytest.mark.parametrize("rotary_dim,interleaved", [(0, False), (128, False), (64, True), (24, False)])
@pytest.mark.parametrize("tokens_per_step", [1, 2])
def test_prefill_then_decode_equals_one_causal_pass(rotary_dim, interleaved, tokens_per_step):
    from flash_attention_b200 import _lib
    from flash_attention_b200.generation import CachedSelfAttention, DecodeGraphs, InferenceParams

    g = torch.Generator().manual_seed(rotary_dim + tokens_per_step)
    B, H, Hk, D, S0, steps, layers = 3, 8, 2, 128, 70, 6, 2
    S = S0 + steps * tokens_per_step
    dt = torch.bfloat16
    qs = [torch.randn(B, S, H, D, generator=g).to(dt).cuda() for _ in range(layers)]
    kvs = [torch.randn(B, S, 2, Hk, D, generator=g).to(dt).cuda() for _ in range(layers)]
    attn = [CachedSelfAttention(i, D, rotary_dim=rotary_dim, rotary_interleaved=interleaved, device="cuda") for i in range(layers)]

    def generate(graphed):
        params = InferenceParams(max_seqlen=S + 5, max_batch_size=B).allocate(range(layers), Hk, D, dt, "cuda")
        params.lengths_per_sample = torch.zeros(B, dtype=torch.int32, device="cuda")
        outs = [[a(q[:, :S0].clone(), kv[:, :S0].clone(), params)] for a, q, kv in zip(attn, qs, kvs)]
        assert _lib.last_path().startswith("fwd_tc")

        def step(p, *xs):  # xs: q and kv of every layer for this step
            return torch.stack([a(xs[2 * i], xs[2 * i + 1], p) for i, a in enumerate(attn)])

        graphs = DecodeGraphs(step, params) if graphed else None
        for t in range(steps):
            pos = S0 + t * tokens_per_step
            sl = slice(pos, pos + tokens_per_step)
            xs = [x for q, kv in zip(qs, kvs) for x in (q[:, sl].clone(), kv[:, sl].clone())]
            params.seqlen_offset = pos
            if graphed:
                o = graphs.run(*xs, seqlen=pos).clone()
            else:
                params.lengths_per_sample.fill_(pos)
                o = step(params, *xs)
            for i in range(layers):
                outs[i].append(o[i])
        if graphed:
            graphs.release()
        return [torch.cat(o, dim=1) for o in outs], params

    eager, params = generate(False)
    graphed, params_g = generate(True)
    for i in range(layers):
        q, kv = qs[i], kvs[i]
        k, v = kv[:, :, 0], kv[:, :, 1]
        if rotary_dim > 0:
            cos, sin = _rotary_tables(rotary_dim, S + 5, dt)
            q = O.rotary_oracle(q.float(), cos.float(), sin.float(), 0, interleaved).to(dt)
            k = O.rotary_oracle(k.float(), cos.float(), sin.float(), 0, interleaved).to(dt)
        truth, _ = O.attention_oracle(q, k, v, causal=True)
        lowp, _ = O.attention_oracle(q, k, v, causal=True, upcast=False, reorder_ops=True)
        assert_within(eager[i], truth, lowp, mult=3, atol=1e-3, what="layer %d" % i)
        assert torch.equal(eager[i], graphed[i])  # a replayed step is the same launches on the same data
        cache = params.key_value_memory_dict[i]
        assert torch.allclose(cache[:, :S, 0].float(), k.float(), rtol=1e-3, atol=1e-3) and torch.equal(cache[:, :S, 1], v)
        assert torch.equal(cache[:, :S], params_g.key_value_memory_dict[i][:, :S])


def test_decode_step_host_time_is_measurable_and_graph_replay_is_cheaper_or_equal():
    from flash_attention_b200.generation import CachedSelfAttention, DecodeGraphs, InferenceParams, host_time_per_call_us

    B, H, Hk, D, cap = 8, 32, 8, 128, 4096
    dt = torch.bfloat16
    attn = CachedSelfAttention(0, D, rotary_dim=D, device="cuda")
    params = InferenceParams(max_seqlen=cap, max_batch_size=B).allocate([0], Hk, D, dt, "cuda")
    params.key_value_memory_dict[0].normal_()
    params.lengths_per_sample = torch.full((B,), 1000, dtype=torch.int32, device="cuda")
    params.seqlen_offset = 1000
    q = torch.randn(B, 1, H, D, device="cuda", dtype=dt)
    kv = torch.randn(B, 1, 2, Hk, D, device="cuda", dtype=dt)
    graphs = DecodeGraphs(lambda p, q_, kv_: attn(q_, kv_, p), params)
    want = attn(q, kv, params).clone()
    got = graphs.run(q, kv, seqlen=1000)
    assert torch.equal(want, got)
    eager_us = host_time_per_call_us(lambda: attn(q, kv, params), iters=50)
    graph_us = host_time_per_call_us(lambda: graphs.run(q, kv, seqlen=1000), iters=50)
    assert 0 < graph_us and 0 < eager_us
    graphs.release()


@pytest.fixture()
def reference_mha(monkeypatch):
    """flash_attn.modules.mha of an installed copy of the reference, imported unmodified on top of this
    repository's flash_attn_2_cuda and rotary kernel."""
    ref_root = None
    for r in (os.environ.get("FLASH_ATTN_REFERENCE_TREE"), os.path.join(ROOT, "baseline", "_ref")):
        if r and os.path.exists(os.path.join(r, "flash_attn", "modules", "mha.py")):
            ref_root = r
            break
    if ref_root is None:
        pytest.skip("no copy of the reference's flash_attn package on this machine")
    import flash_attn_2_cuda as ext

    assert os.path.dirname(os.path.abspath(ext.__file__)).startswith(ROOT), "an unrelated flash_attn_2_cuda shadows the shim"
    for name in [m for m in sys.modules if m == "flash_attn" or m.startswith("flash_attn.")]:
        monkeypatch.delitem(sys.modules, name)
    monkeypatch.syspath_prepend(ref_root)
    from flash_attention_b200.layers import rotary as mine

    pkg = importlib.import_module("flash_attn")
    assert os.path.abspath(pkg.__file__).startswith(os.path.abspath(ref_root))
    importlib.import_module("flash_attn.ops")
    tri = types.ModuleType("flash_attn.ops.triton")
    tri.__path__ = []
    monkeypatch.setitem(sys.modules, "flash_attn.ops.triton", tri)
    stub = types.ModuleType("flash_attn.ops.triton.rotary")
    stub.apply_rotary = mine.apply_rotary
    monkeypatch.setitem(sys.modules, "flash_attn.ops.triton.rotary", stub)
    mha = importlib.import_module("flash_attn.modules.mha")
    assert mha.flash_attn_with_kvcache is not None and mha.RotaryEmbedding is not None
    assert sys.modules["flash_attn.flash_attn_interface"].flash_attn_cuda is ext
    yield mha
    for name in [m for m in sys.modules if m == "flash_attn" or m.startswith("flash_attn.")]:
        monkeypatch.delitem(sys.modules, name, raising=False)


@pytest.mark.parametrize("heads,heads_kv,rotary", [(8, 8, 64), (8, 2, 64), (8, 8, 0)])
def test_unmodified_reference_mha_generates_on_these_kernels(reference_mha, heads, heads_kv, rotary):
    from flash_attention_b200 import _lib
    from flash_attention_b200.generation import InferenceParams

    torch.manual_seed(0)
    B, S0, steps, D = 2, 33, 5, 64
    S, E = S0 + steps, heads * D
    mha = reference_mha.MHA(E, heads, num_heads_kv=heads_kv, causal=True, layer_idx=0, rotary_emb_dim=rotary,
                            use_flash_attn=True, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(B, S, E, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        full = mha(x)  # training path: rotary + flash_attn_(kv|qkv)packed_func
        assert _lib.last_path().startswith("fwd_tc")
        params = InferenceParams(max_seqlen=S, max_batch_size=B)
        outs = [mha(x[:, :S0], inference_params=params)]
        for t in range(steps):
            params.seqlen_offset = S0 + t
            outs.append(mha(x[:, S0 + t:S0 + t + 1], inference_params=params))
            assert _lib.last_path().startswith("decode")  # the fused step: rotary + append + attention in one launch
    got = torch.cat(outs, dim=1)
    scale = full.float().abs().max().item()
    assert (got.float() - full.float()).abs().max().item() <= 3e-2 * scale + 1e-2
    assert params.key_value_memory_dict[0].shape == (B, S, 2, heads_kv, D)
