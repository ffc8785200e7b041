"""Context-parallel ring attention on real GPUs (NCCL): every rank's shard of out, dq, dk, dv must
match the oracle on the gathered sequence.  Needs at least 2 GPUs; skipped otherwise."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, causal, window, out_q, layout="contiguous"):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from flash_attention_b200.ring import ring_flash_attn_func, zigzag_shard
        from oracle import attention_oracle as O

        g = torch.Generator().manual_seed(0)
        B, S, H, Hk, D = 1, 512 * world, 8, 2, 128
        q = torch.randn(B, S, H, D, generator=g).bfloat16()
        k = torch.randn(B, S, Hk, D, generator=g).bfloat16()
        v = torch.randn(B, S, Hk, D, generator=g).bfloat16()
        do = torch.randn(B, S, H, D, generator=g).bfloat16()
        if layout == "zigzag":
            shard = lambda x: zigzag_shard(x, rank, world)
        else:
            shard = lambda x: x[:, rank * S // world:(rank + 1) * S // world]
        dev = torch.device("cuda", rank)
        ql, kl, vl = (shard(x).to(dev).requires_grad_(True) for x in (q, k, v))
        out = ring_flash_attn_func(ql, kl, vl, causal=causal, window_size=window, layout=layout)
        dq, dk, dv = torch.autograd.grad(out, (ql, kl, vl), shard(do).to(dev))
        res = []
        for upcast in (True, False):
            qf, kf, vf = (x.to(dev).requires_grad_(True) for x in (q, k, v))
            ref, _ = O.attention_oracle(qf, kf, vf, causal=causal, window_size=window, upcast=upcast, reorder_ops=not upcast)
            res.append((ref.detach(),) + torch.autograd.grad(ref, (qf, kf, vf), do.to(dev)))
        truth, lowp = res
        errs = []
        for mine, t, l in zip((out.detach(), dq, dk, dv), truth, lowp):
            e = (mine.float() - shard(t).float()).abs().max().item()
            y = (shard(l).float() - shard(t).float()).abs().max().item()
            errs.append((e, y))
        out_q.put((rank, errs))
    finally:
        from flash_attention_b200 import ring

        ring.release_graphs()
        dist.destroy_process_group()


def _run_ring(world, causal, window, layout):
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, causal, window, out_q, layout)) for r in range(world)]
    for p in procs:
        p.start()
    results = [out_q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, errs in results:
        for e, y in errs:
            # partial outputs are rounded to bf16 once per ring step before the merge
            assert e <= 3 * y + 2e-3, (rank, errs)


@pytest.mark.parametrize("causal,window,layout", [(True, (-1, -1), "contiguous"), (False, (-1, -1), "contiguous"),
                                                  (False, (300, 0), "contiguous"), (True, (-1, -1), "zigzag")])
def test_ring_attention_two_gpus(causal, window, layout):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _run_ring(2, causal, window, layout)


@pytest.mark.parametrize("world", [4, 8])
@pytest.mark.parametrize("causal,window,layout", [(True, (-1, -1), "zigzag"), (False, (700, 0), "contiguous")])
def test_ring_attention_more_gpus(world, causal, window, layout):
    # the balanced causal layout, and a window that ends the ring after two steps (most dK / dV slots stay zero)
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    _run_ring(world, causal, window, layout)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fused_merge_matches_torch_merge(dtype):
    """fa_merge_partial (in place, on views) against the torch formulation used on CPU ranks."""
    from flash_attention_b200.ring import CudaBlockOps, merge_partials

    g = torch.Generator().manual_seed(3)
    B, S, H, D = 2, 77, 3, 64
    acc = torch.randn(B, 2 * S, H, D, generator=g).cuda()
    lacc = torch.randn(B, H, 2 * S, generator=g).cuda()
    o = torch.randn(B, S, H, D, generator=g).to(dtype).cuda()
    l = torch.randn(B, H, S, generator=g).cuda()
    lacc[0, 0, S + 1] = float("-inf")  # accumulator still empty
    l[0, 1, 2] = float("inf")          # partial saw no key
    lacc[1, 2, S + 5] = float("-inf")  # both empty
    l[1, 2, 5] = float("inf")
    want_o, want_l = merge_partials(acc[:, S:].clone(), lacc[:, :, S:].clone(), o.float(), l)
    keep_o, keep_l = acc[:, :S].clone(), lacc[:, :, :S].clone()
    CudaBlockOps.merge(acc[:, S:], lacc[:, :, S:], o, l)
    torch.cuda.synchronize()
    assert torch.allclose(acc[:, S:], want_o, atol=1e-5, rtol=1e-5)
    assert torch.equal(torch.isinf(lacc[:, :, S:]), torch.isinf(want_l))
    fin = ~torch.isinf(want_l)
    assert torch.allclose(lacc[:, :, S:][fin], want_l[fin], atol=1e-5)
    assert torch.equal(acc[:, :S], keep_o) and torch.equal(lacc[:, :, :S], keep_l)  # rows outside the view untouched


@pytest.mark.gpu
@pytest.mark.parametrize("d", [64, 128, 192, 256])
def test_block_backward_adds_dk_dv_into_fp32_accumulators(d):
    """fa_bwd with accumulate_dkv (the ring's per-block call) against the plain call, on every tensor-core
    backward kernel: two calls into zeroed accumulators hold twice the plain dk / dv; dq is the plain dq."""
    from flash_attention_b200 import flash_attn_func
    from flash_attention_b200.ring import CudaBlockOps

    g = torch.Generator().manual_seed(11)
    B, Sq, Sk, H, Hk = 2, 200, 333, 4, 2
    q = torch.randn(B, Sq, H, d, generator=g).bfloat16().cuda()
    k, v = (torch.randn(B, Sk, Hk, d, generator=g).bfloat16().cuda() for _ in range(2))
    do = torch.randn(B, Sq, H, d, generator=g).bfloat16().cuda()
    qq, kk, vv = (x.clone().requires_grad_(True) for x in (q, k, v))
    want_dq, want_dk, want_dv = torch.autograd.grad(flash_attn_func(qq, kk, vv, causal=True), (qq, kk, vv), do)
    scale, shift = d ** -0.5, Sk - Sq  # bottom-right aligned causal mask as a shifted window
    out, lse = CudaBlockOps.fwd(q, k, v, scale, (-1, 0), shift)
    dk_acc = torch.zeros(B, Sk, Hk, d, dtype=torch.float32, device="cuda")
    dv_acc = torch.zeros_like(dk_acc)
    # once whole, once as its two halves (dot(dO, O) + dQ, then dK / dV)
    for parts in (0, (1, 2)):
        dq = CudaBlockOps.bwd(do, q, k, v, out, lse, dk_acc, dv_acc, scale, (-1, 0), shift, parts=parts)
    torch.cuda.synchronize()
    assert torch.allclose(dq.float(), want_dq.float(), atol=1e-2, rtol=1e-2)
    # the plain call rounds dk / dv to bf16 once; the accumulators keep fp32
    for acc, want in ((dk_acc, want_dk), (dv_acc, want_dv)):
        err = (acc / 2 - want.float()).abs().max().item()
        assert err <= 2e-2 * max(1.0, want.float().abs().max().item()), err
