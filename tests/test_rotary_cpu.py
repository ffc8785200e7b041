"""Host side of the rotary layer (flash_attention_b200/layers/rotary.py) on the CPU: which views turn with
which tables, what the gradients are, and what the module's tables hold.  The CUDA entry point is
replaced by the oracle's rotation, so only the logic above the C ABI is under test here.

Where a copy of the reference's python package is at hand (FLASH_ATTN_REFERENCE_TREE, else the
python-only install under baseline/_ref), the reference's own unmodified flash_attn/layers/rotary.py is
loaded on the same stand-in and must agree bit for bit: tables, outputs and gradients."""
import importlib.util
import os
import sys
import types

import pytest
import torch

from oracle import attention_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _oracle_apply_rotary(x, cos, sin, seqlen_offsets=0, cu_seqlens=None, max_seqlen=None, interleaved=False,
                         inplace=False, conjugate=False):
    assert cu_seqlens is None
    y = O.rotary_oracle(x.float(), cos.float(), (-sin if conjugate else sin).float(), seqlen_offsets, interleaved).to(x.dtype)
    if inplace:
        x.copy_(y)
        return x
    return y


@pytest.fixture()
def mine(monkeypatch):
    from flash_attention_b200.layers import rotary

    monkeypatch.setattr(rotary, "apply_rotary", _oracle_apply_rotary)
    return rotary


@pytest.fixture()
def theirs(monkeypatch):
    path = None
    for r in (os.environ.get("FLASH_ATTN_REFERENCE_TREE"), os.path.join(ROOT, "baseline", "_ref")):
        if r and os.path.exists(os.path.join(r, "flash_attn", "layers", "rotary.py")):
            path = os.path.join(r, "flash_attn", "layers", "rotary.py")
            break
    if path is None:
        pytest.skip("no copy of the reference's flash_attn package on this machine")
    # the one symbol the file imports from its Triton module
    for name in ("flash_attn", "flash_attn.ops", "flash_attn.ops.triton"):
        if name not in sys.modules:
            monkeypatch.setitem(sys.modules, name, types.ModuleType(name))
    stub = types.ModuleType("flash_attn.ops.triton.rotary")
    stub.apply_rotary = _oracle_apply_rotary
    monkeypatch.setitem(sys.modules, "flash_attn.ops.triton.rotary", stub)
    spec = importlib.util.spec_from_file_location("reference_layers_rotary", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _tables(rows, half, gen):
    angle = torch.rand(rows, half, generator=gen) * 6.28
    return angle.cos(), angle.sin()


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("inplace", [False, True])
def test_x_entry_rotates_and_backward_is_the_inverse_rotation(mine, interleaved, inplace):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(2, 9, 3, 16, generator=g)
    cos, sin = _tables(20, 4, g)
    offs = torch.tensor([3, 7], dtype=torch.int32)
    want = O.rotary_oracle(x, cos, sin, offs, interleaved)
    leaf = x.clone().requires_grad_()
    out = mine.apply_rotary_emb(leaf, cos, sin, interleaved=interleaved, inplace=inplace, seqlen_offsets=offs)
    assert torch.allclose(out, want, atol=1e-6)
    assert (out.data_ptr() == leaf.data_ptr()) == inplace
    do = torch.randn(x.shape, generator=g)
    out.backward(do.clone())
    assert torch.allclose(leaf.grad, O.rotary_oracle(do, cos, -sin, offs, interleaved), atol=1e-6)
    # rotating back gives the input again: the op is orthogonal
    back = mine.apply_rotary_emb(want, cos, -sin, interleaved=interleaved, seqlen_offsets=offs)
    assert torch.allclose(back, x, atol=1e-5)


@pytest.mark.parametrize("two_tables", [False, True])
@pytest.mark.parametrize("contiguous", [True, False])
def test_qkv_entry_turns_q_and_k_only(mine, two_tables, contiguous):
    g = torch.Generator().manual_seed(2)
    B, S, H, D = 2, 11, 3, 8
    base = torch.randn(B, S, 3, H, D + (0 if contiguous else 4), generator=g)
    qkv = base[..., :D]
    cos, sin = _tables(S, 2, g)
    cos_k, sin_k = _tables(S, 2, g) if two_tables else (None, None)
    want_q = O.rotary_oracle(qkv[:, :, 0], cos, sin, 0, False)
    want_k = O.rotary_oracle(qkv[:, :, 1], cos_k if two_tables else cos, sin_k if two_tables else sin, 0, False)
    v = qkv[:, :, 2].clone()
    inp = qkv.clone() if contiguous else qkv
    inp.requires_grad_(contiguous)
    out = mine.apply_rotary_emb_qkv_(inp, cos, sin, cos_k, sin_k)
    assert out.data_ptr() == inp.data_ptr()
    assert torch.allclose(out[:, :, 0], want_q, atol=1e-6) and torch.allclose(out[:, :, 1], want_k, atol=1e-6)
    assert torch.equal(out[:, :, 2], v)
    if contiguous:
        do = torch.randn(B, S, 3, H, D, generator=g)
        out.backward(do.clone())
        assert torch.allclose(inp.grad[:, :, 0], O.rotary_oracle(do[:, :, 0], cos, -sin, 0, False), atol=1e-6)
        assert torch.equal(inp.grad[:, :, 2], do[:, :, 2])


def test_kv_entry_turns_k_only_and_shape_errors_are_loud(mine):
    g = torch.Generator().manual_seed(3)
    kv = torch.randn(2, 5, 2, 2, 8, generator=g)
    cos, sin = _tables(9, 4, g)
    want = O.rotary_oracle(kv[:, :, 0], cos, sin, 4, True)
    v = kv[:, :, 1].clone()
    out = mine.apply_rotary_emb_kv_(kv, cos, sin, interleaved=True, seqlen_offsets=4)
    assert torch.allclose(out[:, :, 0], want, atol=1e-6) and torch.equal(out[:, :, 1], v)
    with pytest.raises(ValueError):
        mine.apply_rotary_emb_kv_(torch.zeros(1, 2, 3, 1, 8), cos, sin)
    with pytest.raises(ValueError):
        mine.apply_rotary_emb_qkv_(torch.zeros(1, 2, 2, 1, 8), cos, sin)
    with pytest.raises(ValueError):
        mine.apply_rotary_emb_qkv_(torch.zeros(1, 2, 3, 1, 8), cos, sin, cos_k=cos)


def test_module_tables_closed_form_growth_and_xpos(mine):
    dim, base = 16, 10000.0
    rot = mine.RotaryEmbedding(dim, base=base)
    assert rot.scale is None and rot._cos_cached is None
    rot._update_cos_sin_cache(10, device=torch.device("cpu"), dtype=torch.float32)
    pos = torch.arange(10, dtype=torch.float32)[:, None]
    freq = base ** (-torch.arange(0, dim, 2, dtype=torch.float32) / dim)
    assert torch.allclose(rot._cos_cached, (pos * freq).cos(), atol=1e-6)
    assert torch.allclose(rot._sin_cached, (pos * freq).sin(), atol=1e-6)
    first = rot._cos_cached
    rot._update_cos_sin_cache(6, device=torch.device("cpu"), dtype=torch.float32)
    assert rot._cos_cached is first  # shorter sequences reuse the tables
    rot._update_cos_sin_cache(12, device=torch.device("cpu"), dtype=torch.float32)
    assert rot._cos_cached.shape[0] == 12 and rot._seq_len_cached == 12
    rot._update_cos_sin_cache(12, device=torch.device("cpu"), dtype=torch.float16)
    assert rot._cos_cached.dtype == torch.float16  # a new dtype rebuilds
    # a module cast to bf16 still makes its tables from fp32 positions and frequencies
    cast = mine.RotaryEmbedding(dim).to(torch.bfloat16)
    cast.inv_freq = cast.inv_freq.to(torch.bfloat16)
    cast._update_cos_sin_cache(300, device=torch.device("cpu"), dtype=torch.float32)
    pos = torch.arange(300, dtype=torch.float32)[:, None]
    assert torch.allclose(cast._cos_cached, (pos * freq).cos(), atol=1e-5)
    # XPos: q and k magnitudes are reciprocal, so q_i . k_j depends on i - j only
    xp = mine.RotaryEmbedding(dim, scale_base=64)
    xp._update_cos_sin_cache(8, device=torch.device("cpu"), dtype=torch.float32)
    mag_q = (xp._cos_cached ** 2 + xp._sin_cached ** 2).sqrt()
    mag_k = (xp._cos_k_cached ** 2 + xp._sin_k_cached ** 2).sqrt()
    assert torch.allclose(mag_q * mag_k, torch.ones_like(mag_q), atol=1e-5)
    assert torch.allclose(mag_q[4], torch.ones(dim // 2), atol=1e-6)  # the middle position is unscaled
    zeta = (torch.arange(0, dim, 2, dtype=torch.float32) + 0.4 * dim) / (1.4 * dim)
    assert torch.allclose(mag_q[5] / mag_q[4], zeta ** (1 / 64), atol=1e-6)


@pytest.mark.parametrize("scale_base", [None, 32.0])
@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("packed", [True, False])
def test_module_agrees_with_the_unmodified_reference_module(mine, theirs, scale_base, interleaved, packed):
    g = torch.Generator().manual_seed(4)
    B, S, H, Hk, D, off = 2, 13, 4, 2, 16, 3
    a = mine.RotaryEmbedding(D, interleaved=interleaved, scale_base=scale_base)
    b = theirs.RotaryEmbedding(D, interleaved=interleaved, scale_base=scale_base)
    assert torch.equal(a.inv_freq, b.inv_freq)
    if packed:
        qkv = torch.randn(B, S, 3, H, D, generator=g)
        xa, xb = qkv.clone().requires_grad_(), qkv.clone().requires_grad_()
        ya, yb = a(xa, seqlen_offset=off), b(xb, seqlen_offset=off)
        assert torch.equal(ya, yb)
        do = torch.randn(qkv.shape, generator=g)
        ya.backward(do.clone())
        yb.backward(do.clone())
        assert torch.equal(xa.grad, xb.grad)
    else:
        q, kv = torch.randn(B, S, H, D, generator=g), torch.randn(B, S, 2, Hk, D, generator=g)
        qa, kva = a(q.clone(), kv.clone(), seqlen_offset=off)
        qb, kvb = b(q.clone(), kv.clone(), seqlen_offset=off)
        assert torch.equal(qa, qb) and torch.equal(kva, kvb)
    for name in ("_cos_cached", "_sin_cached", "_cos_k_cached", "_sin_k_cached"):
        ta, tb = getattr(a, name), getattr(b, name)
        assert (ta is None) == (tb is None) and (ta is None or torch.equal(ta, tb)), name
    # tensor offsets with max_seqlen, as the decode path calls it
    offs = torch.tensor([1, 5], dtype=torch.int32)
    q = torch.randn(B, 1, H, D, generator=g)
    kv = torch.randn(B, 1, 2, Hk, D, generator=g)
    qa, kva = a(q.clone(), kv.clone(), seqlen_offset=offs, max_seqlen=20)
    qb, kvb = b(q.clone(), kv.clone(), seqlen_offset=offs, max_seqlen=20)
    assert torch.equal(qa, qb) and torch.equal(kva, kvb)
