"""bench.py --workload ring: ONE long sequence (batch 1, seqlen 32768, 32 query heads, 8 KV heads,
head_dim 128, bf16, causal) sharded by rows over the ranks with context-parallel ring attention.
Strong scaling: the total work is fixed, every rank owns seqlen / N rows (for N > 1 in the zigzag
layout, which gives all ranks the same share of the causal mask).  At N = 1 the ring has a
single step and is plain local attention.  FLOP model as in bench.py (fwd 4*S^2*H*D/2, bwd 2.5x).
"""
import json
import os

import torch


def main(args):
    from flash_attention_b200 import _lib
    from flash_attention_b200.ring import ring_flash_attn_func

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    import torch.distributed as dist

    if not dist.is_initialized():
        if world == 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    S, H, Hk, D = 32768, 32, 8, 128
    S_loc = S // world
    layout = "zigzag" if world > 1 else "contiguous"  # balances the causal mask over the ranks
    g = torch.Generator(device=dev).manual_seed(2 + rank)
    q = torch.randn(1, S_loc, H, D, device=dev, dtype=torch.bfloat16, generator=g).requires_grad_(True)
    k = torch.randn(1, S_loc, Hk, D, device=dev, dtype=torch.bfloat16, generator=g).requires_grad_(True)
    v = torch.randn(1, S_loc, Hk, D, device=dev, dtype=torch.bfloat16, generator=g).requires_grad_(True)
    do = torch.randn(1, S_loc, H, D, device=dev, dtype=torch.bfloat16, generator=g)

    def step():
        out = ring_flash_attn_func(q, k, v, causal=True, layout=layout)
        return torch.autograd.grad(out, (q, k, v), do)

    for _ in range(max(3, args.warmup)):
        step()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    torch.cuda.synchronize()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([ev0.elapsed_time(ev1) / args.steps], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item()
    flops = 3.5 * 4.0 * S * S * H * D / 2.0
    status = _lib.lib().fa_device_status()
    if rank == 0:
        print(json.dumps({
            "metric": "attention fwd+bwd TFLOPS/s (bf16, d128, causal, context-parallel ring)",
            "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOPS/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "ring_gqa_b1_s32768_h32_hk8_d128_causal", "rows_per_gpu": S_loc, "layout": layout,
                       "exchange": "K/V blocks by NCCL send/recv, dK/dV fp32 accumulators travel in the backward",
                       "l2": "inputs larger than L2"},
            "gpu_launches": args.steps * 4 * (2 * world + 1 if world > 1 else 1), "device_status": status,
        }))
    dist.destroy_process_group()
