"""Generates tests/golden/reference_cases.pt from the REFERENCE's own functions.

Run where the FlashAttention v2.3.3 tree is available:

    python tests/golden/make_golden.py /path/to/flash-attention

The reference's test module cannot be imported without a GPU (tests/test_flash_attn.py:23-26 query
the device at import) and flash_attn/layers/rotary.py pulls in triton, so the pure-PyTorch function
definitions are taken out of the files with `ast` and executed as they are:
  construct_local_mask, attention_ref                  tests/test_flash_attn.py:153-259
  rotate_half, apply_rotary_emb_torch                  flash_attn/layers/rotary.py:11-32
  index_cos_sin                                        tests/test_rotary.py:32-42
Inputs come from seeded CPU generators; each case stores the seed recipe's tensors in fp16/bf16 and
the reference's outputs, sub-sampled where large, so the file stays small.
"""
import ast
import math
import os
import sys

import torch


def load_functions(path, names):
    src = open(path).read()
    tree = ast.parse(src)
    picked = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
    assert {n.name for n in picked} == set(names), (path, names)
    mod = ast.Module(body=picked, type_ignores=[])
    from einops import rearrange, repeat

    env = {"torch": torch, "math": math, "rearrange": rearrange, "repeat": repeat}
    exec(compile(mod, path, "exec"), env)
    return {n: env[n] for n in names}


def make_inputs(seed, B, Sq, Sk, H, Hk, D, dtype):
    """The seeded input recipe of every attention case (also used by the tests to rebuild the inputs
    of cases that are stored without them)."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Sq, H, D, generator=g).to(dtype)
    k = torch.randn(B, Sk, Hk, D, generator=g).to(dtype)
    v = torch.randn(B, Sk, Hk, D, generator=g).to(dtype)
    do = torch.randn(B, Sq, H, D, generator=g).to(dtype)
    return g, q, k, v, do


def main(ref_root):
    t = load_functions(os.path.join(ref_root, "tests", "test_flash_attn.py"), ["construct_local_mask", "attention_ref"])
    r = load_functions(os.path.join(ref_root, "flash_attn", "layers", "rotary.py"), ["rotate_half", "apply_rotary_emb_torch"])
    ix = load_functions(os.path.join(ref_root, "tests", "test_rotary.py"), ["index_cos_sin"])
    attention_ref = t["attention_ref"]
    cases = []

    def attn_case(name, seed, B, Sq, Sk, H, Hk, D, dtype, causal=False, window=(-1, -1), qpad=False, kpad=False,
                  dropout_p=0.0, subsample=1):
        g, q, k, v, do = make_inputs(seed, B, Sq, Sk, H, Hk, D, dtype)
        qm = km = dm = None
        if qpad:
            lens = torch.randint(max(1, Sq // 2), Sq + 1, (B,), generator=g)
            qm = torch.arange(Sq).view(1, -1) < lens.view(-1, 1)
        if kpad:
            lens = torch.randint(max(1, Sk // 2), Sk + 1, (B,), generator=g)
            km = torch.arange(Sk).view(1, -1) < lens.view(-1, 1)
        if dropout_p > 0:
            dm = torch.rand(B, H, Sq, Sk, generator=g) > dropout_p
        qf, kf, vf = (x.clone().requires_grad_(True) for x in (q, k, v))
        out, attn = attention_ref(qf, kf, vf, qm, km, dropout_p, dm, causal=causal, window_size=window)
        dq, dk, dv = torch.autograd.grad(out, (qf, kf, vf), do)
        out_pt, _ = attention_ref(q, k, v, qm, km, dropout_p, dm, causal=causal, window_size=window, upcast=False,
                                  reorder_ops=True)
        ss = subsample
        sub = lambda x: x.detach()[:, ::ss].clone()
        case = dict(kind="attention", name=name, recipe=(seed, B, Sq, Sk, H, Hk, D, dtype), query_padding_mask=qm,
                    key_padding_mask=km, dropout_p=dropout_p, dropout_mask=dm, causal=causal, window_size=window,
                    subsample=ss, out=sub(out), attn=attn.detach()[:, :, ::ss, ::ss].clone(),
                    dq=sub(dq), dk=sub(dk), dv=sub(dv), out_lowp=sub(out_pt))
        if ss == 1:  # small cases carry their inputs; large ones are rebuilt from the recipe
            case.update(q=q, k=k, v=v, dout=do)
        cases.append(case)

    bf, hf = torch.bfloat16, torch.float16
    attn_case("mha_noncausal", 1, 2, 33, 47, 4, 4, 32, hf)
    attn_case("mha_causal_sq_lt_sk", 2, 2, 33, 47, 4, 4, 32, bf, causal=True)
    attn_case("mha_causal_sq_gt_sk", 3, 2, 47, 33, 4, 4, 32, bf, causal=True)
    attn_case("gqa_causal", 4, 1, 64, 64, 6, 2, 40, hf, causal=True)
    attn_case("mqa_window", 5, 2, 50, 70, 4, 1, 16, bf, window=(7, 3))
    attn_case("window_left_only", 6, 1, 40, 40, 2, 2, 16, hf, window=(5, -1))
    attn_case("window_right_only", 7, 1, 40, 56, 2, 2, 16, hf, window=(-1, 4))
    attn_case("padded_causal", 8, 3, 48, 48, 4, 2, 32, bf, causal=True, qpad=True, kpad=True)
    attn_case("padded_window", 9, 3, 40, 56, 2, 2, 16, hf, window=(9, 2), qpad=True, kpad=True)
    attn_case("dropout", 10, 2, 32, 48, 2, 2, 32, hf, dropout_p=0.17)
    attn_case("dropout_causal_gqa", 11, 1, 48, 48, 4, 2, 16, bf, causal=True, dropout_p=0.17)
    # the CPU-runnable configuration: batch 2, seqlen 512, 8 heads, head_dim 64, causal, bf16
    attn_case("config_b2_s512_h8_d64_causal", 0, 2, 512, 512, 8, 8, 64, bf, causal=True, subsample=16)

    def rotary_case(name, seed, B, S, H, D, rd, dtype, interleaved, tensor_offsets):
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(B, S, H, D, generator=g).to(dtype)
        seqlen_ro = S + 40
        ang = torch.rand(seqlen_ro, rd // 2, generator=g) * 2 * math.pi
        cos, sin = torch.cos(ang).to(dtype), torch.sin(ang).to(dtype)
        off = torch.randint(0, 40, (B,), generator=g).to(torch.int32) if tensor_offsets else 11
        cos_pt, sin_pt = ix["index_cos_sin"](cos, sin, off, S)
        out = r["apply_rotary_emb_torch"](x.float(), cos_pt.float(), sin_pt.float(), interleaved=interleaved).to(dtype)
        out_lowp = r["apply_rotary_emb_torch"](x, cos_pt, sin_pt, interleaved=interleaved)
        cases.append(dict(kind="rotary", name=name, x=x, cos=cos, sin=sin, offsets=off, interleaved=interleaved,
                          out=out, out_lowp=out_lowp))

    rotary_case("neox_full", 20, 2, 9, 3, 32, 32, bf, False, True)
    rotary_case("neox_half", 21, 2, 9, 3, 64, 32, hf, False, True)
    rotary_case("interleaved_full", 22, 2, 5, 2, 32, 32, hf, True, True)
    rotary_case("interleaved_partial_int_offset", 23, 1, 7, 2, 48, 16, bf, True, False)

    out_path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_cases.pt")
    torch.save(dict(reference="flash-attention v2.3.3", torch=torch.__version__, cases=cases), out_path)
    print("wrote %s (%d cases, %.1f KiB)" % (out_path, len(cases), os.path.getsize(out_path) / 1024))


if __name__ == "__main__":
    if len(sys.argv) < 2 and not os.environ.get("FLASH_ATTN_REFERENCE_TREE"):
        sys.exit("usage: make_golden.py /path/to/flash-attention  (or set FLASH_ATTN_REFERENCE_TREE)")
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["FLASH_ATTN_REFERENCE_TREE"])
