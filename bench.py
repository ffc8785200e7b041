"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" = one forward + backward of exact attention on the workload's batch.  Default workload:
packed-QKV training shape, batch 16 x seqlen 2048 x 16 heads x head_dim 128, bf16, causal,
dropout 0 (the shape of the reference's own sweep, benchmarks/benchmark_flash_attention.py:74-78).
Metric: fwd+bwd TFLOPS/s with the reference's FLOP model (benchmarks/benchmark_flash_attention.py:27-30):
fwd = 4*B*S^2*H*D (halved when causal), bwd = 2.5x fwd.

N > 1 (torchrun, one rank per GPU): every rank runs the same per-GPU batch (independent
(batch x head) units, no communication); value = total FLOPs of all ranks / max-over-ranks time.
`--workload ring` shards ONE long sequence over the ranks with context-parallel ring attention.

`--impl reference` times the reference's CPU attention (the fp32 oracle restatement of attention_ref)
on the host cores, on a bounded sample of the same workload.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT in sys.path:
    sys.path.remove(ROOT)
sys.path.insert(0, ROOT)

import torch  # noqa: E402

# dram__bytes_read.sum + dram__bytes_write.sum of the two tensor-core backward kernels, per launch pair, from the ncu
# capture summarised in profiles/ (bwd_tc_kernel 781.6 MB + bwd_dq_tc_kernel 660.7 MB; algorithmic bytes: 1479 MB)
# and of the three passes of the wide kernel (516.7 + 658.0 + 657.4 MB; algorithmic: 3 x 671 MB - 134 MB for the pass without V)
NCU_DRAM_BYTES_PER_BACKWARD = {"train_b16_s2048_h16_d128_causal": 1.4423e9, "train_b16_s2048_h8_d256": 1.8321e9}

WORKLOADS = {
    # name: (batch, seqlen, heads, heads_k, head_dim, causal, dtype)
    "train_b16_s2048_h16_d128_causal": (16, 2048, 16, 16, 128, True, torch.bfloat16),
    "train_b16_s2048_h16_d128": (16, 2048, 16, 16, 128, False, torch.bfloat16),
    "train_b16_s2048_h32_d64_causal": (16, 2048, 32, 32, 64, True, torch.bfloat16),
    "gqa_b1_s32768_h32_hk8_d128_causal": (1, 32768, 32, 8, 128, True, torch.bfloat16),
    "train_b16_s2048_h32_d64": (16, 2048, 32, 32, 64, False, torch.bfloat16),
    "train_b16_s2048_h8_d256_causal": (16, 2048, 8, 8, 256, True, torch.bfloat16),
    "train_b16_s2048_h8_d256": (16, 2048, 8, 8, 256, False, torch.bfloat16),
}
DEFAULT = "train_b16_s2048_h16_d128_causal"


def fwd_flops(B, S, H, D, causal):
    return 4.0 * B * S * S * H * D / (2.0 if causal else 1.0)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(source="measured", hbm_gbs=p["hbm_gbs"], tflops_burst=p["bf16_tflops"],
                    tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]))
    return dict(source="fallback", hbm_gbs=6650.0, tflops_burst=1590.0, tflops_sustained=1400.0)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.rows = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def cpu_attention_sample(D, S, causal, heads=1, repeats=1, budget_s=0.0):
    """fp32 oracle forward+backward on the host cores for `heads` (batch x head) units of length S.
    Returns the best time of one pass; keeps passing until `budget_s` seconds of CPU work are spent."""
    from oracle import attention_oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(1, S, heads, D, generator=g).requires_grad_(True) for _ in range(3))
    do = torch.randn(1, S, heads, D, generator=g)
    best, spent, n = None, 0.0, 0
    while n < repeats + 1 or spent < budget_s:  # the first pass warms the allocator
        t0 = time.perf_counter()
        out, _ = O.attention_oracle(q, k, v, causal=causal)
        torch.autograd.grad(out, (q, k, v), do)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
        spent += dt
        n += 1
    return best


def run_reference(args, wl):
    B, S, H, Hk, D, causal, dtype = WORKLOADS[wl]
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    units = 16  # (batch x head) units per step: a bounded sample of the B*H units of the workload
    times = []
    for i in range(args.warmup + args.steps):
        dt = cpu_attention_sample(D, S, causal, heads=units)
        if i >= args.warmup:
            times.append(dt)
    t = sum(times) / len(times)
    fl = 3.5 * fwd_flops(1, S, units, D, causal)
    val = fl / t / 1e12
    sample = "%d of %d (batch x head) units at full seqlen %d per step, fp32 attention_ref restatement, fwd+bwd" % (units, B * H, S)
    print(json.dumps({
        "impl": "reference", "metric": "attention fwd+bwd TFLOPS/s", "value": val, "unit": "TFLOPS/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl, "sample": sample},
        "cpu_baseline": {"value": val, "unit": "TFLOPS/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOPS/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_decode(args):
    """KV-cache decode step: batch 64 (per GPU), 32 query heads, 8 KV heads, head_dim 128, bf16 cache of
    capacity 32768 filled N(0,1), cache_seqlens uniform in [1024, 32767], one new token appended
    in-kernel with NeoX rotary.  Metric: GB/s over the K and V rows actually attended to."""
    import flash_attention_b200 as fa
    from flash_attention_b200 import _lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    B, cap, H, Hk, D = 64, 32768, 32, 8, 128
    g = torch.Generator(device=dev).manual_seed(4 + rank)
    kc = torch.randn(B, cap, Hk, D, device=dev, dtype=torch.bfloat16, generator=g)
    vc = torch.randn(B, cap, Hk, D, device=dev, dtype=torch.bfloat16, generator=g)
    lens = torch.randint(1024, 32768, (B,), device=dev, generator=g).to(torch.int32)
    q = torch.randn(B, 1, H, D, device=dev, dtype=torch.bfloat16, generator=g)
    kn = torch.randn(B, 1, Hk, D, device=dev, dtype=torch.bfloat16, generator=g)
    vn = torch.randn(B, 1, Hk, D, device=dev, dtype=torch.bfloat16, generator=g)
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2, device=dev).float() / D))
    fr = torch.outer(torch.arange(cap, device=dev).float(), inv)
    cos, sin = torch.cos(fr).bfloat16(), torch.sin(fr).bfloat16()
    nbytes = float((lens.long() + 1).sum().item()) * Hk * D * 2 * 2

    def step():
        return fa.flash_attn_with_kvcache(q, kc, vc, kn, vn, cos, sin, lens, causal=True, rotary_interleaved=False)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, args.warmup)):
        step()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with ClockSampler(local) as clk:
        ev0.record()
        for _ in range(args.steps):
            step()  # the 8 GiB cache is far larger than L2: every step streams from HBM
        ev1.record()
        barrier()
    ms = ev0.elapsed_time(ev1) / args.steps
    if dist is not None:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    gbs = world * nbytes / (ms * 1e-3) / 1e9
    # end to end: the per-step host inputs are the new token's q/k/v and the lengths; the cache is device state
    hq, hk_, hv, hl = (x.cpu().pin_memory() for x in (q, kn, vn, lens))
    out_host = torch.empty((B, 1, H, D), dtype=torch.bfloat16).pin_memory()

    def e2e():
        q.copy_(hq, non_blocking=True)
        kn.copy_(hk_, non_blocking=True)
        vn.copy_(hv, non_blocking=True)
        lens.copy_(hl, non_blocking=True)
        out_host.copy_(step(), non_blocking=True)

    e2e()
    barrier()
    ev0.record()
    for _ in range(args.steps):
        e2e()
    ev1.record()
    barrier()
    ms_e2e = ev0.elapsed_time(ev1) / args.steps
    pk = peaks()
    status = _lib.lib().fa_device_status()
    if rank == 0:
        print(json.dumps({
            "metric": "decode KV-cache GB/s (bf16, d128, split-KV)", "value": gbs, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "decode_b64_hq32_hk8_d128_cap32768", "batch_per_gpu": B, "cache_capacity": cap,
                       "cache_seqlens": "uniform [1024, 32767]", "new_tokens": 1, "rotary": "neox, dim 128, base 10000",
                       "l2": "8 GiB cache per GPU, larger than L2", "bytes_model": "sum_b (L_b + 1) * 8 * 128 * 2 B * 2"},
            "roofline": {"bound": "hbm", "kernel": "decode_kernel (+ combine_kernel)", "achieved": gbs / world,
                         "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / world / pk["hbm_gbs"], "traffic": None,
                         "peak_source": pk["source"]},
            "cpu_baseline": None,
            "e2e": {"value": world * nbytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": sum(x.numel() * x.element_size() for x in (hq, hk_, hv, hl)),
                    "d2h_bytes_per_step": out_host.numel() * 2, "ms_per_step": ms_e2e},
            "gpu_launches": args.steps * 2, "clocks": clk.summary(), "device_status": status,
        }))
    if dist is not None:
        dist.destroy_process_group()


def run_rotary(args):
    """Rotary embedding of q and k inside the default workload's packed qkv (16 x 2048 x 3 x 16 x 128 bf16 per GPU),
    in place, forward (the backward is the same kernel with the conjugate flag).  Metric: GB/s over the bytes of
    q and k read and written."""
    from flash_attention_b200 import _lib
    from flash_attention_b200.layers.rotary import apply_rotary_emb_qkv_

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    B, S, H, D = 16, 2048, 16, 128
    g = torch.Generator(device=dev).manual_seed(5 + rank)
    qkv = torch.randn(B, S, 3, H, D, device=dev, dtype=torch.bfloat16, generator=g)
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2, device=dev).float() / D))
    fr = torch.outer(torch.arange(S, device=dev).float(), inv)
    cos, sin = torch.cos(fr).bfloat16(), torch.sin(fr).bfloat16()
    nbytes = 2.0 * 2 * B * S * H * D * 2  # q and k, read + write

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.no_grad():
        for _ in range(max(3, args.warmup)):
            apply_rotary_emb_qkv_(qkv, cos, sin)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        with ClockSampler(local) as clk:
            ev0.record()
            for _ in range(args.steps):
                apply_rotary_emb_qkv_(qkv, cos, sin)  # 268 MB of q, k per call: larger than L2
            ev1.record()
            barrier()
    ms = ev0.elapsed_time(ev1) / args.steps
    if dist is not None:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    gbs = world * nbytes / (ms * 1e-3) / 1e9
    pk = peaks()
    if rank == 0:
        print(json.dumps({
            "metric": "rotary embedding GB/s (bf16, q and k of packed qkv, in place)", "value": gbs, "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "rotary_qkv_b16_s2048_h16_d128", "batch_per_gpu": B, "seqlen": S, "heads": H, "head_dim": D,
                       "rotary_dim": D, "style": "neox", "l2": "268 MB of q and k per call, larger than L2",
                       "bytes_model": "2 (q, k) x 2 (read, write) x B S H D x 2 B"},
            "roofline": {"bound": "hbm", "kernel": "rotary_vec_kernel", "achieved": gbs / world, "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / world / pk["hbm_gbs"], "traffic": None, "peak_source": pk["source"]},
            "cpu_baseline": None, "e2e": None, "gpu_launches": args.steps, "clocks": clk.summary(),
            "device_status": _lib.lib().fa_device_status(),
        }))
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.workload == "ring":
        from flash_attention_b200 import ring_bench

        return ring_bench.main(args)
    if args.workload == "rotary":
        return run_rotary(args)
    if args.workload == "decode":
        return run_decode(args)
    wl = args.workload
    if args.impl == "reference":
        return run_reference(args, wl)

    import flash_attention_b200 as fa
    from flash_attention_b200 import _lib

    B, S, H, Hk, D, causal, dtype = WORKLOADS[wl]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    g = torch.Generator(device=dev).manual_seed(1 + rank)
    packed = H == Hk
    if packed:
        qkv = torch.randn(B, S, 3, H, D, device=dev, dtype=dtype, generator=g).requires_grad_(True)
        inputs = (qkv,)
    else:
        q = torch.randn(B, S, H, D, device=dev, dtype=dtype, generator=g).requires_grad_(True)
        k = torch.randn(B, S, Hk, D, device=dev, dtype=dtype, generator=g).requires_grad_(True)
        v = torch.randn(B, S, Hk, D, device=dev, dtype=dtype, generator=g).requires_grad_(True)
        inputs = (q, k, v)
    dout = torch.randn(B, S, H, D, device=dev, dtype=dtype, generator=g)

    def forward(inp):
        if packed:
            return fa.flash_attn_qkvpacked_func(inp[0], causal=causal)
        return fa.flash_attn_func(inp[0], inp[1], inp[2], causal=causal)

    def step(inp, do):
        out = forward(inp)
        return out, torch.autograd.grad(out, inp, do)

    f_fwd = fwd_flops(B, S, H, D, causal)
    f_step = 3.5 * f_fwd
    for _ in range(max(3, args.warmup)):
        step(inputs, dout)
    # ---- timed region: K steps, device timed, max over ranks
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with ClockSampler(local) as clk:
        ev0.record()
        for _ in range(args.steps):
            step(inputs, dout)
        ev1.record()
        barrier()
    ms = ev0.elapsed_time(ev1)
    if dist is not None:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    ms_step = ms / args.steps
    value = world * f_step / (ms_step * 1e-3) / 1e12

    # ---- forward and backward timed separately (the kernels behind the roofline numbers)
    def timed(fn, n):
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(n):
            fn()
        b_.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b_) / n

    n_sub = max(3, min(args.steps, 20))
    with torch.no_grad():
        ms_fwd = timed(lambda: forward(inputs), n_sub)
    out = forward(inputs)
    ms_bwd = timed(lambda: torch.autograd.grad(out, inputs, dout, retain_graph=True), n_sub)
    pk = peaks()
    tf_fwd = f_fwd / (ms_fwd * 1e-3) / 1e12
    tf_bwd = 2.5 * f_fwd / (ms_bwd * 1e-3) / 1e12
    # the backward pass dominates a step: two tensor-core kernels of similar length (dK/dV per key
    # block, dQ per query block) after one small bandwidth kernel (dot_do_o, a few percent: see
    # profiles/).  FLOPs are the algorithmic 5 GEMMs; the two kernels execute 7 (S and dP twice).
    # Head dims above 128 run one kernel as three passes (dV, dK, dQ), which execute 8 GEMMs (S three times, dP twice).
    wide = D > 128
    bwd_kernels = ("backward (bwd_dot_do_o + bwd_wide_tc_kernel x3 [dV, dK, dQ passes])" if wide else
                   "backward (bwd_dot_do_o + bwd_tc_kernel [dK,dV] + bwd_dq_tc_kernel [dQ])")
    roofline = {"bound": "tensor", "kernel": bwd_kernels,
                "achieved": tf_bwd, "peak": pk["tflops_burst"], "unit": "TFLOP/s",
                "frac": tf_bwd / pk["tflops_burst"], "traffic": NCU_DRAM_BYTES_PER_BACKWARD.get(wl), "peak_source": pk["source"],
                "forward": {"kernel": "fwd_tc_kernel", "achieved": tf_fwd, "frac": tf_fwd / pk["tflops_burst"],
                            "frac_of_sustained": tf_fwd / pk["tflops_sustained"]},
                "frac_of_sustained": tf_bwd / pk["tflops_sustained"]}

    # ---- end to end: host (pinned) -> device copies of the step's inputs, device -> host read of a result.
    # Every step copies its own inputs and reads its own result; as a training loop would, the copy of step
    # i+1 (copy stream, second input buffer) runs while step i computes, so a step costs max(copy, compute).
    host_in = [x.detach().cpu().pin_memory() for x in inputs]
    host_do = dout.cpu().pin_memory()
    dev_in = [[torch.empty_like(x).requires_grad_(True) for x in inputs] for _ in range(2)]
    dev_do = [torch.empty_like(dout) for _ in range(2)]
    h2d = sum(x.numel() * x.element_size() for x in host_in) + host_do.numel() * host_do.element_size()
    res_host = torch.empty(1, dtype=torch.float32).pin_memory()
    copy_stream = torch.cuda.Stream()
    main_stream = torch.cuda.current_stream()
    copied = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]

    def e2e_steps(n):
        for buf in range(2):
            consumed[buf].record(main_stream)
        for i in range(n):
            buf = i & 1
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(consumed[buf])  # the step that last used this buffer has finished
                for d_, h_ in zip(dev_in[buf], host_in):
                    d_.data.copy_(h_, non_blocking=True)
                dev_do[buf].copy_(host_do, non_blocking=True)
                copied[buf].record(copy_stream)
            main_stream.wait_event(copied[buf])
            o, grads = step(tuple(dev_in[buf]), dev_do[buf])
            res_host.copy_(grads[0].flatten()[:1].float(), non_blocking=True)
            consumed[buf].record(main_stream)

    e2e_steps(2)
    barrier()
    n_e2e = max(4, min(args.steps, 10))
    ev0.record()
    e2e_steps(n_e2e)
    ev1.record()
    barrier()
    ms_e2e = ev0.elapsed_time(ev1) / n_e2e
    if dist is not None:
        t = torch.tensor([ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = t.item()
    e2e_val = world * f_step / (ms_e2e * 1e-3) / 1e12
    status = _lib.lib().fa_device_status()

    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            units = 16
            dt = cpu_attention_sample(D, S, causal, heads=units, budget_s=12.0)
            cpu = {"value": 3.5 * fwd_flops(1, S, units, D, causal) / dt / 1e12, "unit": "TFLOPS/s",
                   "cores": os.cpu_count() or 1, "kind": "port",
                   "sample": "%d of %d (batch x head) units at full seqlen %d per pass, fp32 attention_ref restatement, fwd+bwd, best of ~12 s of passes (%.2f s per pass)" % (units, B * H, S, dt)}
        line = {
            "metric": "attention fwd+bwd TFLOPS/s (bf16, d%d%s)" % (D, ", causal" if causal else ""),
            "value": value, "unit": "TFLOPS/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16" if dtype == torch.bfloat16 else "fp16", "data": "synthetic",
            "config": {"workload": wl, "batch_per_gpu": B, "seqlen": S, "heads": H, "heads_k": Hk, "head_dim": D,
                       "causal": causal, "dropout_p": 0.0, "api": "flash_attn_qkvpacked_func" if packed else "flash_attn_func",
                       "l2": "inputs (%.0f MiB per step) larger than L2" % (h2d / 2**20),
                       "flop_model": "fwd 4*B*S^2*H*D%s, bwd 2.5x" % ("/2" if causal else "")},
            "fwd_tflops": tf_fwd, "bwd_tflops": tf_bwd, "ms_fwd": ms_fwd, "ms_bwd": ms_bwd,
            "roofline": roofline, "cpu_baseline": cpu,
            "e2e": {"value": e2e_val, "unit": "TFLOPS/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                    "ms_per_step": ms_e2e, "pipeline": "copy of step i+1 overlaps compute of step i (2 input buffers)"},
            "gpu_launches": args.steps * (5 if wide else 4),
            "clocks": clk.summary(), "device_status": status,
        }
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
