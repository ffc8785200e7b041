"""Ring (context-parallel) attention schedule and LSE merge on CPU ranks over gloo, world size 2
and 4, with the oracle's math standing in for the per-block CUDA kernels."""
import math
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import attention_oracle as O


class OracleBlockOps:
    """Per-block attention with an explicit mask shift, in fp32 torch (test stand-in for the kernels)."""

    @staticmethod
    def _scores(q, k, scale, window, shift):
        B, Sq, H, D = q.shape
        Sk = k.shape[1]
        kk = k.float().repeat_interleave(H // k.shape[2], dim=2)
        s = torch.einsum("bthd,bshd->bhts", q.float(), kk) * scale
        i = torch.arange(Sq).view(-1, 1)
        j = torch.arange(Sk).view(1, -1)
        vis = torch.ones(Sq, Sk, dtype=torch.bool)
        if window[1] >= 0:
            vis &= j <= i + shift + window[1]
        if window[0] >= 0:
            vis &= j >= i + shift - window[0]
        return s.masked_fill(~vis, float("-inf"))

    @staticmethod
    def fwd(q, k, v, scale, window, shift):
        s = OracleBlockOps._scores(q, k, scale, window, shift)
        lse = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - lse.unsqueeze(-1))
        p = torch.where(torch.isnan(p), torch.zeros_like(p), p)
        vv = v.float().repeat_interleave(q.shape[2] // v.shape[2], dim=2)
        out = torch.einsum("bhts,bshd->bthd", p, vv)
        lse = torch.where(torch.isinf(lse), torch.full_like(lse, float("inf")), lse)
        return out.to(q.dtype), lse

    @staticmethod
    def bwd(dout, q, k, v, out, lse, dk_acc, dv_acc, scale, window, shift):
        H, Hk = q.shape[2], k.shape[2]
        s = OracleBlockOps._scores(q, k, scale, window, shift)
        p = torch.exp(s - lse.unsqueeze(-1))  # lse = +inf for empty rows -> p = 0
        p = torch.where(torch.isnan(p), torch.zeros_like(p), p)
        vv = v.float().repeat_interleave(H // Hk, dim=2)
        kk = k.float().repeat_interleave(H // Hk, dim=2)
        do = dout.float()
        dsum = (do * out.float()).sum(-1).permute(0, 2, 1)  # (B, H, Sq)
        dp = torch.einsum("bthd,bshd->bhts", do, vv)
        ds = p * (dp - dsum.unsqueeze(-1))
        dq = torch.einsum("bhts,bshd->bthd", ds, kk) * scale
        dk = torch.einsum("bhts,bthd->bshd", ds, q.float()) * scale
        dv = torch.einsum("bhts,bthd->bshd", p, do)
        B, Sk = k.shape[0], k.shape[1]
        dk_acc += dk.view(B, Sk, Hk, H // Hk, -1).sum(3)
        dv_acc += dv.view(B, Sk, Hk, H // Hk, -1).sum(3)
        return dq.to(q.dtype)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, causal, window, out_q, layout="contiguous"):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flash_attention_b200.ring import ring_flash_attn_func

        g = torch.Generator().manual_seed(0)
        B, S, H, Hk, D = 1, 32 * world, 4, 2, 16
        q = torch.randn(B, S, H, D, generator=g)
        k = torch.randn(B, S, Hk, D, generator=g)
        v = torch.randn(B, S, Hk, D, generator=g)
        do = torch.randn(B, S, H, D, generator=g)
        from flash_attention_b200.ring import zigzag_shard

        if layout == "zigzag":
            shard = lambda x: zigzag_shard(x, rank, world)
        else:
            shard = lambda x: x[:, rank * S // world:(rank + 1) * S // world]
        ql, kl, vl = (shard(x).clone().requires_grad_(True) for x in (q, k, v))
        out = ring_flash_attn_func(ql, kl, vl, causal=causal, window_size=window, block_ops=OracleBlockOps, layout=layout)
        dq, dk, dv = torch.autograd.grad(out, (ql, kl, vl), shard(do))
        qf, kf, vf = (x.clone().requires_grad_(True) for x in (q, k, v))
        ref, _ = O.attention_oracle(qf, kf, vf, causal=causal, window_size=window)
        rdq, rdk, rdv = torch.autograd.grad(ref, (qf, kf, vf), do)
        errs = [(out - shard(ref)).abs().max().item(), (dq - shard(rdq)).abs().max().item(),
                (dk - shard(rdk)).abs().max().item(), (dv - shard(rdv)).abs().max().item()]
        out_q.put((rank, errs))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("causal,window", [(False, (-1, -1)), (True, (-1, -1)), (False, (20, 0)), (False, (9, 5))])
def test_ring_matches_full_attention(world, causal, window):
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, causal, window, out_q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [out_q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, errs in results:
        assert max(errs) < 1e-4, (rank, errs)


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("causal,window", [(True, (-1, -1)), (False, (9, 5))])
def test_zigzag_ring_matches_full_attention(world, causal, window):
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, causal, window, out_q, "zigzag")) for r in range(world)]
    for p in procs:
        p.start()
    results = [out_q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, errs in results:
        assert max(errs) < 1e-4, (rank, errs)


def test_zigzag_shard_roundtrip_and_balance():
    from flash_attention_b200.ring import block_visible, layout_chunks, zigzag_shard, zigzag_unshard

    x = torch.arange(2 * 48 * 3).view(2, 48, 3)
    for world in (2, 4):
        assert torch.equal(zigzag_unshard([zigzag_shard(x, r, world) for r in range(world)]), x)
        # under a causal mask every rank sees the same number of (query chunk, key chunk) pairs per step,
        # except the step with its own keys (two diagonal blocks instead of one full block)
        for step in range(1, world):
            counts = []
            for r in range(world):
                mine, theirs = layout_chunks("zigzag", r, world, 12), layout_chunks("zigzag", (r - step) % world, world, 12)
                counts.append(sum(block_visible(qg, qn, kg, kn, (-1, 0)) for qg, qn in mine for kg, kn in theirs))
            assert counts == [2] * world, counts


def test_merge_partials_matches_oracle():
    from flash_attention_b200.ring import merge_partials

    g = torch.Generator().manual_seed(1)
    B, S, H, D = 2, 5, 3, 8
    oa, ob = torch.randn(B, S, H, D, generator=g), torch.randn(B, S, H, D, generator=g)
    la, lb = torch.randn(B, H, S, generator=g), torch.randn(B, H, S, generator=g)
    la[0, 0, 0] = float("inf")  # empty in part a
    lb[0, 0, 1] = float("-inf")
    la[1, 2, 3] = float("inf")
    lb[1, 2, 3] = float("inf")  # empty in both
    out, lse = merge_partials(oa, la, ob, lb)
    parts = torch.stack((oa.permute(0, 2, 1, 3).reshape(-1, D), ob.permute(0, 2, 1, 3).reshape(-1, D)))
    lses = torch.stack((la.reshape(-1), lb.reshape(-1)))
    lses = torch.where(torch.isinf(lses) & (lses > 0), torch.full_like(lses, float("-inf")), lses)
    ro, rl = O.merge_oracle(parts, lses)
    assert torch.allclose(out.permute(0, 2, 1, 3).reshape(-1, D), ro, atol=1e-6)
    mine = torch.where(torch.isinf(lse) & (lse < 0), torch.full_like(lse, float("inf")), lse).reshape(-1)
    assert torch.allclose(mine, rl, atol=1e-6)
