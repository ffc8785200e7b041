"""Parity of the rotary op (flash_attention_b200/layers/rotary.py over fa_rotary) with the oracle's
restatement of apply_rotary_emb_torch, over the lattice of the reference's tests/test_rotary.py:
in place or not, interleaved or halves, full or half rotary fraction, int / tensor / no offsets,
padded and packed (cu_seqlens) input, q+k inside packed qkv / kv, forward and backward.
Tolerance as there: rtol 1e-3, atol = 2 x the rounding of the expected value's dtype."""
import math

import pytest
import torch

from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu


def _tables(seqlen, rotary_dim, dtype, gen):
    angle = torch.rand(seqlen * 2, rotary_dim // 2, generator=gen) * 2 * math.pi
    return torch.cos(angle).to(dtype).cuda(), torch.sin(angle).to(dtype).cuda()


def _offsets(kind, batch, seqlen, gen):
    if kind == 0:
        return 0
    if kind is int:
        return int(torch.randint(0, seqlen + 1, (1,), generator=gen))
    return torch.randint(0, seqlen + 1, (batch,), dtype=torch.int32, generator=gen).cuda()


def _close(mine, want):
    atol = ((want + 0.3 - 0.3) - want).abs().max().item()
    assert torch.allclose(mine, want, rtol=1e-3, atol=2 * atol), (mine.float() - want.float()).abs().max().item()


def _expected(x, cos, sin, offs, interleaved):
    """Oracle in fp32 on the 16-bit inputs, rounded once: the kernel computes in fp32 as well."""
    return O.rotary_oracle(x.float(), cos.float(), sin.float(), offs, interleaved).to(x.dtype)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("offs_kind", [0, int, torch.Tensor])
@pytest.mark.parametrize("rotary_fraction", [1.0, 0.5])
@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("inplace", [False, True])
def test_rotary_emb_func(inplace, interleaved, rotary_fraction, offs_kind, dtype):
    from flash_attention_b200.layers.rotary import apply_rotary_emb

    g = torch.Generator().manual_seed(42)
    B, H, S, D = 32, 4, 217, 128
    rd = int(rotary_fraction * D)
    x = torch.randn(B, S, H, D, generator=g).to(dtype).cuda()
    cos, sin = _tables(S, rd, dtype, g)
    offs = _offsets(offs_kind, B, S, g)
    want = _expected(x, cos, sin, offs, interleaved)
    x_in = x.clone().requires_grad_()
    out = apply_rotary_emb(x_in, cos, sin, seqlen_offsets=offs, interleaved=interleaved, inplace=inplace)
    if inplace:
        assert out.data_ptr() == x_in.data_ptr()
    _close(out.detach(), want)
    do = torch.randn(B, S, H, D, generator=g).to(dtype).cuda()
    # the gradient of a rotation is the rotation of the incoming gradient by the negative angle
    want_dx = _expected(do, cos, -sin, offs, interleaved)
    out.backward(do.clone())
    _close(x_in.grad, want_dx)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("offs_kind", [0, int, torch.Tensor])
@pytest.mark.parametrize("rotary_fraction", [1.0, 0.5])
@pytest.mark.parametrize("interleaved", [False, True])
def test_rotary_emb_qkv(interleaved, rotary_fraction, offs_kind, dtype):
    from flash_attention_b200.layers.rotary import apply_rotary_emb_qkv_

    g = torch.Generator().manual_seed(43)
    B, H, S, D = 32, 4, 512, 128
    rd = int(rotary_fraction * D)
    qkv = torch.randn(B, S, 3, H, D, generator=g).to(dtype).cuda()
    cos, sin = _tables(S, rd, dtype, g)
    offs = _offsets(offs_kind, B, S, g)
    want_q = _expected(qkv[:, :, 0], cos, sin, offs, interleaved)
    want_k = _expected(qkv[:, :, 1], cos, sin, offs, interleaved)
    want_v = qkv[:, :, 2].clone()
    qkv_in = qkv.clone().requires_grad_()
    out = apply_rotary_emb_qkv_(qkv_in, cos, sin, seqlen_offsets=offs, interleaved=interleaved)
    _close(out[:, :, 0].detach(), want_q)
    _close(out[:, :, 1].detach(), want_k)
    assert torch.equal(out[:, :, 2].detach(), want_v)
    do = torch.randn(B, S, 3, H, D, generator=g).to(dtype).cuda()
    want = [_expected(do[:, :, 0], cos, -sin, offs, interleaved), _expected(do[:, :, 1], cos, -sin, offs, interleaved), do[:, :, 2].clone()]
    out.backward(do.clone())
    for i in range(3):
        _close(qkv_in.grad[:, :, i], want[i])


@pytest.mark.parametrize("interleaved", [False, True])
def test_rotary_emb_qkv_separate_key_tables_and_strided_input(interleaved):
    from flash_attention_b200.layers.rotary import apply_rotary_emb_qkv_

    g = torch.Generator().manual_seed(44)
    B, H, S, D, rd = 3, 5, 100, 64, 32
    big = torch.randn(B, S, 3, H, D + 8, generator=g).half().cuda()
    qkv = big[..., :D]  # not contiguous: the two-call path
    cos, sin = _tables(S, rd, torch.float16, g)
    cos_k, sin_k = _tables(S, rd, torch.float16, g)
    want_q = _expected(qkv[:, :, 0], cos, sin, 0, interleaved)
    want_k = _expected(qkv[:, :, 1], cos_k, sin_k, 0, interleaved)
    out = apply_rotary_emb_qkv_(qkv, cos, sin, cos_k, sin_k, interleaved=interleaved)
    _close(out[:, :, 0], want_q)
    _close(out[:, :, 1], want_k)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("offs_kind", [0, int, torch.Tensor])
@pytest.mark.parametrize("rotary_fraction", [1.0, 0.5])
@pytest.mark.parametrize("interleaved", [False, True])
def test_rotary_emb_kv(interleaved, rotary_fraction, offs_kind, dtype):
    from flash_attention_b200.layers.rotary import apply_rotary_emb_kv_

    g = torch.Generator().manual_seed(45)
    B, H, S, D = 32, 4, 781, 64
    rd = int(rotary_fraction * D)
    kv = torch.randn(B, S, 2, H, D, generator=g).to(dtype).cuda()
    cos, sin = _tables(S, rd, dtype, g)
    offs = _offsets(offs_kind, B, S, g)
    want_k = _expected(kv[:, :, 0], cos, sin, offs, interleaved)
    want_v = kv[:, :, 1].clone()
    kv_in = kv.clone().requires_grad_()
    out = apply_rotary_emb_kv_(kv_in, cos, sin, seqlen_offsets=offs, interleaved=interleaved)
    _close(out[:, :, 0].detach(), want_k)
    assert torch.equal(out[:, :, 1].detach(), want_v)
    do = torch.randn(B, S, 2, H, D, generator=g).to(dtype).cuda()
    want_dk = _expected(do[:, :, 0], cos, -sin, offs, interleaved)
    out.backward(do.clone())
    _close(kv_in.grad[:, :, 0], want_dk)
    assert torch.equal(kv_in.grad[:, :, 1], do[:, :, 1])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("offs_kind", [0, torch.Tensor])
@pytest.mark.parametrize("rotary_fraction", [1.0, 0.5])
@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("inplace", [False, True])
def test_rotary_emb_varlen_func(inplace, interleaved, rotary_fraction, offs_kind, dtype):
    from flash_attention_b200.layers.rotary import apply_rotary_emb

    g = torch.Generator().manual_seed(46)
    B, H, S, D = 32, 4, 217, 128
    rd = int(rotary_fraction * D)
    x = torch.randn(B, S, H, D, generator=g).to(dtype).cuda()
    lens = torch.randint(0, S + 1, (B,), generator=g)
    lens[3] = 0  # an empty sequence in the middle
    cu = torch.zeros(B + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(lens, 0)
    packed = torch.cat([x[b, : lens[b]] for b in range(B)], dim=0)
    cos, sin = _tables(S, rd, dtype, g)
    offs = _offsets(offs_kind, B, S, g)
    full = _expected(x, cos, sin, offs, interleaved)
    want = torch.cat([full[b, : lens[b]] for b in range(B)], dim=0)
    x_in = packed.clone().requires_grad_()
    out = apply_rotary_emb(x_in, cos, sin, seqlen_offsets=offs, interleaved=interleaved, inplace=inplace,
                           cu_seqlens=cu.cuda(), max_seqlen=S)
    _close(out.detach(), want)
    do = torch.randn(packed.shape, generator=g).to(dtype).cuda()
    do_pad = torch.zeros_like(x)
    for b in range(B):
        do_pad[b, : lens[b]] = do[cu[b]:cu[b + 1]]
    full_dx = _expected(do_pad, cos, -sin, offs, interleaved)
    want_dx = torch.cat([full_dx[b, : lens[b]] for b in range(B)], dim=0)
    out.backward(do.clone())
    _close(x_in.grad, want_dx)


def test_rotary_odd_shapes_take_the_scalar_path():
    """rotary_dim / 2 not a multiple of 8 and a head dim that is not a multiple of 8."""
    from flash_attention_b200.layers.rotary import apply_rotary_emb

    g = torch.Generator().manual_seed(47)
    for interleaved in (False, True):
        for B, S, H, D, rd in ((2, 33, 3, 36, 20), (1, 7, 1, 12, 12), (2, 50, 2, 96, 40)):
            x = torch.randn(B, S, H, D, generator=g).half().cuda()
            cos, sin = _tables(S, rd, torch.float16, g)
            out = apply_rotary_emb(x, cos, sin, interleaved=interleaved, seqlen_offsets=3)
            _close(out, _expected(x, cos, sin, 3, interleaved))


def test_rotary_embedding_module_matches_function_and_attention_runs_on_it():
    from flash_attention_b200 import flash_attn_qkvpacked_func
    from flash_attention_b200.layers.rotary import RotaryEmbedding

    g = torch.Generator().manual_seed(48)
    B, S, H, D = 2, 300, 4, 64
    qkv = torch.randn(B, S, 3, H, D, generator=g).half().cuda()
    rot = RotaryEmbedding(D, interleaved=False, device="cuda")
    want_q = O.rotary_oracle(qkv[:, :, 0].float(), *[t.float() for t in (torch.cos(torch.outer(torch.arange(S, device="cuda").float(), rot.inv_freq)).half(), torch.sin(torch.outer(torch.arange(S, device="cuda").float(), rot.inv_freq)).half())], 0, False).half()
    out = rot(qkv.clone())
    _close(out[:, :, 0], want_q)
    o = flash_attn_qkvpacked_func(out, causal=True)
    assert torch.isfinite(o).all()
    # XPos: keys use the inverse scale
    rot_x = RotaryEmbedding(D, scale_base=512, device="cuda")
    q, kv = rot_x(qkv[:, :, 0].clone(), qkv[:, :, 1:].clone(), seqlen_offset=5)
    assert q.shape == (B, S, H, D) and kv.shape == (B, S, 2, H, D)
    assert torch.equal(kv[:, :, 1], qkv[:, :, 2])


def test_unmodified_reference_rotary_layer_on_this_kernel(monkeypatch):
    """The reference's own flash_attn/layers/rotary.py, loaded as it is, with the one symbol it imports
    (apply_rotary of its Triton module) supplied by this repository's CUDA binding: module forward and
    backward against the oracle, and bit-equal to this repository's own layer."""
    import importlib.util
    import os
    import sys
    import types

    from flash_attention_b200.layers import rotary as mine

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = None
    for r in (os.environ.get("FLASH_ATTN_REFERENCE_TREE"), os.path.join(root, "baseline", "_ref")):
        if r and os.path.exists(os.path.join(r, "flash_attn", "layers", "rotary.py")):
            path = os.path.join(r, "flash_attn", "layers", "rotary.py")
            break
    if path is None:
        pytest.skip("no copy of the reference's flash_attn package on this machine")
    for name in ("flash_attn", "flash_attn.ops", "flash_attn.ops.triton"):
        if name not in sys.modules:
            monkeypatch.setitem(sys.modules, name, types.ModuleType(name))
    stub = types.ModuleType("flash_attn.ops.triton.rotary")
    stub.apply_rotary = mine.apply_rotary
    monkeypatch.setitem(sys.modules, "flash_attn.ops.triton.rotary", stub)
    spec = importlib.util.spec_from_file_location("reference_layers_rotary", path)
    theirs = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(theirs)

    g = torch.Generator().manual_seed(49)
    B, S, H, D, off = 3, 257, 6, 128, 11
    qkv = torch.randn(B, S, 3, H, D, generator=g).bfloat16().cuda()
    do = torch.randn(B, S, 3, H, D, generator=g).bfloat16().cuda()
    for interleaved in (False, True):
        a = mine.RotaryEmbedding(D, interleaved=interleaved, device="cuda")
        b = theirs.RotaryEmbedding(D, interleaved=interleaved, device="cuda")
        xa, xb = qkv.clone().requires_grad_(), qkv.clone().requires_grad_()
        ya, yb = a(xa, seqlen_offset=off), b(xb, seqlen_offset=off)
        cos, sin = b._cos_cached, b._sin_cached
        _close(yb[:, :, 0].detach(), _expected(qkv[:, :, 0], cos, sin, off, interleaved))
        _close(yb[:, :, 1].detach(), _expected(qkv[:, :, 1], cos, sin, off, interleaved))
        assert torch.equal(ya, yb)
        ya.backward(do.clone())
        yb.backward(do.clone())
        _close(xb.grad[:, :, 1], _expected(do[:, :, 1], cos, -sin, off, interleaved))
        assert torch.equal(xa.grad, xb.grad)
