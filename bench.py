"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" = one forward + backward of exact attention on the workload's batch.  Default workload:
packed-QKV training shape, batch 16 x seqlen 2048 x 16 heads x head_dim 128, bf16, causal,
dropout 0 (the shape of the reference's own sweep, benchmarks/benchmark_flash_attention.py:74-78).
Metric: fwd+bwd TFLOPS/s with the reference's FLOP model (benchmarks/benchmark_flash_attention.py:27-30):
fwd = 4*B*S^2*H*D (halved when causal), bwd = 2.5x fwd.

The K-step region is timed several times (CUDA events, barrier + synchronize on both sides, max over
ranks); `ms_per_step` and `value` are the median repeat.  N > 1 (torchrun, one rank per GPU): every
rank runs the same per-GPU batch (independent (batch x head) units, no communication); value =
total FLOPs of all ranks / max-over-ranks time.

The JSON line also carries, under "also", the other headline numbers measured in the same run:
forward only, the KV-cache decode step (GB/s), and the context-parallel ring over the N ranks on
one 32768-token sequence (strong scaling, next to the same sequence on one GPU).

`--impl reference` times the reference's CPU attention (attention_ref of tests/test_flash_attn.py
from a reference tree named by FLASH_ATTN_REFERENCE_TREE when there is one, else its fp32 restatement
in oracle/) on the host cores, on a bounded sample of the same workload.
"""
import argparse
import json
import math
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

METRIC = "attention fwd+bwd TFLOPS/s"

# dram__bytes_read.sum + dram__bytes_write.sum of the backward kernels of one step, from ncu captures of these
# kernels on these workloads (d128: dK/dV kernel + dQ kernel; d256: the three passes of the wide kernel)
NCU_DRAM_BYTES_PER_BACKWARD = {"train_b16_s2048_h16_d128_causal": 1.4427e9, "train_b16_s2048_h8_d256": 1.8399e9}

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
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw")

    def __init__(self, index):
        self.index = index
        self.rows = []
        self.stamps = []
        self.windows = []  # (start, end) wall-clock times of the timed regions
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "20"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])
            self.stamps.append(time.time())

    def mark(self, t0, t1):
        self.windows.append((t0, t1))

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        # a sample counts when it was taken while a timed region ran (nvidia-smi reports ~10 ms after it reads);
        # with no region marked, every sample counts
        inside = [r for r, t in zip(self.rows, self.stamps)
                  if not self.windows or any(a <= t - 0.01 <= b + 0.02 for a, b in self.windows)]
        for r in inside:
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
            try:
                pw.append(float(r[6]))
            except (ValueError, IndexError):
                pass
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm), power_w_max=max(pw) if pw else None)


class Ranks:
    """Rank bookkeeping of one process per GPU (torchrun) or a single process."""

    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, x):
        if self.dist is None:
            return x
        t = torch.tensor([x], device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.item()

    def close(self):
        if self.dist is not None:
            from flash_attention_b200 import ring

            ring.release_graphs()  # graphs that hold NCCL kernels must go before their communicator does
            self.dist.barrier()
            self.dist.destroy_process_group()


def timed_repeats(R, fn, steps, min_repeats=5, target_ms=250.0, max_repeats=40, gap_s=0.0, clk=None):
    """Times `steps` calls of fn as one region, several times.  Each region is bracketed by a barrier +
    synchronize on both sides, timed with CUDA events on the launching stream, and its time is the max
    over ranks.  The number of repeats (the same on all ranks) is chosen from the first region so that
    the regions together last about target_ms.  gap_s > 0 leaves the GPU idle for that long before every
    region, so that each region starts from the idle power state (how a burst peak is measured); gap_s = 0
    runs them back to back (sustained, under the power cap).  clk: a ClockSampler that is told when each
    region ran.  Returns the list of per-step times in ms."""
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def region():
        if gap_s > 0:
            time.sleep(gap_s)
        R.barrier()
        t0 = time.time()
        ev0.record()
        for _ in range(steps):
            fn()
        ev1.record()
        R.barrier()
        if clk is not None:
            clk.mark(t0, time.time())
        return R.max_over_ranks(ev0.elapsed_time(ev1))

    first = region()
    n = int(min(max_repeats, max(min_repeats, math.ceil(target_ms / max(first, 1e-3)))))
    times = [first] + [region() for _ in range(n - 1)]
    return [t / steps for t in times]


# ------------------------------------------------------------------------------------------------ CPU arms
def _reference_attention_ref():
    """attention_ref of the reference's own test file, when a reference tree is at hand (its pure-PyTorch
    function definitions are taken out of the file with `ast`: the module itself needs a GPU to import)."""
    tree = os.environ.get("FLASH_ATTN_REFERENCE_TREE")
    path = os.path.join(tree, "tests", "test_flash_attn.py") if tree else None
    if not path or not os.path.exists(path):
        return None
    import ast

    from einops import rearrange, repeat

    names = ("construct_local_mask", "attention_ref")
    mod = ast.Module(body=[n for n in ast.parse(open(path).read()).body
                           if isinstance(n, ast.FunctionDef) and n.name in names], type_ignores=[])
    env = {"torch": torch, "math": math, "rearrange": rearrange, "repeat": repeat}
    exec(compile(mod, path, "exec"), env)
    return env["attention_ref"]


def cpu_attention_sample(D, S, causal, heads=1, repeats=1, budget_s=0.0):
    """fp32 attention forward+backward on the host cores for `heads` (batch x head) units of length S.
    Returns (best time of one pass, kind); keeps passing until `budget_s` seconds of CPU work are spent."""
    ref = _reference_attention_ref()
    if ref is None:
        from oracle import attention_oracle as O

        fn, kind = (lambda q, k, v: O.attention_oracle(q, k, v, causal=causal)[0]), "port"
    else:
        fn, kind = (lambda q, k, v: ref(q, k, v, causal=causal)[0]), "reference"
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(1, S, heads, D, generator=g).requires_grad_(True) for _ in range(3))
    do = torch.randn(1, S, heads, D, generator=g)
    best, spent, n = None, 0.0, 0
    while n < repeats + 1 or spent < budget_s:  # the first pass warms the allocator
        t0 = time.perf_counter()
        out = fn(q, k, v)
        torch.autograd.grad(out, (q, k, v), do)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
        spent += dt
        n += 1
    return best, kind


def run_reference(args, wl):
    B, S, H, Hk, D, causal, dtype = WORKLOADS[wl]
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    units = 16  # (batch x head) units per step: a bounded sample of the B*H units of the workload
    times, kind = [], "port"
    for i in range(args.warmup + args.steps):
        dt, kind = cpu_attention_sample(D, S, causal, heads=units)
        if i >= args.warmup:
            times.append(dt)
    t = statistics.median(times)
    fl = 3.5 * fwd_flops(1, S, units, D, causal)
    val = fl / t / 1e12
    what = "attention_ref of the reference's tests" if kind == "reference" else "fp32 restatement of attention_ref"
    sample = "%d of %d (batch x head) units at full seqlen %d per step, %s, fwd+bwd" % (units, B * H, S, what)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOPS/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl, "sample": sample},
        "cpu_baseline": {"value": val, "unit": "TFLOPS/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": "TFLOPS/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------------------------------ decode
def measure_other_shapes(R, steps):
    """The other BASELINE shapes in the same run, briefly: fwd+bwd, forward and backward TFLOP/s per GPU for every
    workload of WORKLOADS besides the default one, and for the packed variable-length case (lengths ~ U[128, 4096]
    until 65536 tokens, seed 3, 16 heads, head dim 128, fp16, causal).  Three regions of `steps` steps each, every
    region started from an idle GPU; the median is reported."""
    import flash_attention_b200 as fa

    dev = R.dev
    res = {}

    def timed(fn):
        fn()
        return statistics.median(timed_repeats(R, fn, steps, min_repeats=3, max_repeats=3, gap_s=0.2))

    def fwd_bwd(name, forward, inputs, dout, f_fwd):
        def fwd_only():
            with torch.no_grad():
                forward()

        ms_f = timed(fwd_only)
        out = forward()
        ms_b = timed(lambda: torch.autograd.grad(out, inputs, dout, retain_graph=True))
        del out
        # fwd_bwd: from the forward and the backward timed separately
        res[name] = {"fwd_bwd_tflops": 3.5 * f_fwd / ((ms_f + ms_b) * 1e-3) / 1e12, "fwd_tflops": f_fwd / (ms_f * 1e-3) / 1e12,
                     "bwd_tflops": 2.5 * f_fwd / (ms_b * 1e-3) / 1e12, "ms_fwd": ms_f, "ms_bwd": ms_b}

    for wl, (B, S, H, Hk, D, causal, dtype) in WORKLOADS.items():
        if wl == DEFAULT:
            continue
        g = torch.Generator(device=dev).manual_seed(11 + R.rank)
        q = torch.randn(B, S, H, D, device=dev, dtype=dtype, generator=g).requires_grad_(True)
        k = torch.randn(B, S, Hk, D, device=dev, dtype=dtype, generator=g).requires_grad_(True)
        v = torch.randn(B, S, Hk, D, device=dev, dtype=dtype, generator=g).requires_grad_(True)
        do = torch.randn(B, S, H, D, device=dev, dtype=dtype, generator=g)
        fwd_bwd(wl, lambda: fa.flash_attn_func(q, k, v, causal=causal), (q, k, v), do, fwd_flops(B, S, H, D, causal))
        del q, k, v, do
    H, D = 16, 128
    gl = torch.Generator().manual_seed(3)
    lens, total = [], 0
    while total < 65536:
        n = min(int(torch.randint(128, 4097, (1,), generator=gl)), 65536 - total)
        lens.append(n)
        total += n
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
    g = torch.Generator(device=dev).manual_seed(12 + R.rank)
    q, k, v = (torch.randn(total, H, D, device=dev, dtype=torch.float16, generator=g).requires_grad_(True) for _ in range(3))
    do = torch.randn(total, H, D, device=dev, dtype=torch.float16, generator=g)
    f_fwd = sum(4.0 * n * n * H * D / 2.0 for n in lens)
    fwd_bwd("varlen_fp16_%dseqs_65536tok_h16_d128_causal" % len(lens),
            lambda: fa.flash_attn_varlen_func(q, k, v, cu, cu, max(lens), max(lens), causal=True), (q, k, v), do, f_fwd)
    del q, k, v, do
    torch.cuda.empty_cache()
    return res


def measure_decode(R, steps, warmup, B=64, cap=32768, caller_path=True):
    """KV-cache decode step: batch 64 (per GPU), 32 query heads, 8 KV heads, head_dim 128, bf16 cache of
    capacity 32768 filled N(0,1), cache_seqlens uniform in [capacity / 32, capacity), one new token appended
    in-kernel with NeoX rotary.  GB/s over the K and V rows actually attended to.  (B, cap) = (8, 8192) is
    the same kernel on 0.27 GB of cache, for profiler captures.)"""
    import flash_attention_b200 as fa

    dev = R.dev
    H, Hk, D = 32, 8, 128
    g = torch.Generator(device=dev).manual_seed(4 + R.rank)
    kc = torch.randn(B, cap, Hk, D, device=dev, dtype=torch.bfloat16, generator=g)
    vc = torch.randn(B, cap, Hk, D, device=dev, dtype=torch.bfloat16, generator=g)
    lens = torch.randint(cap // 32, cap, (B,), device=dev, generator=g).to(torch.int32)
    q = torch.randn(B, 1, H, D, device=dev, dtype=torch.bfloat16, generator=g)
    kn = torch.randn(B, 1, Hk, D, device=dev, dtype=torch.bfloat16, generator=g)
    vn = torch.randn(B, 1, Hk, D, device=dev, dtype=torch.bfloat16, generator=g)
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2, device=dev).float() / D))
    fr = torch.outer(torch.arange(cap, device=dev).float(), inv)
    cos, sin = torch.cos(fr).bfloat16(), torch.sin(fr).bfloat16()
    nbytes = float((lens.long() + 1).sum().item()) * Hk * D * 2 * 2

    def step():
        return fa.flash_attn_with_kvcache(q, kc, vc, kn, vn, cos, sin, lens, causal=True, rotary_interleaved=False)

    for _ in range(max(3, warmup)):
        step()
    # the 8 GiB cache is far larger than L2: every step streams from HBM
    with ClockSampler(R.local) as clk:
        per_step = timed_repeats(R, step, steps, target_ms=500.0)
    ms = statistics.median(per_step)
    gbs = R.world * nbytes / (ms * 1e-3) / 1e9
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
    ms_e2e = statistics.median(timed_repeats(R, e2e, steps, min_repeats=3, target_ms=200.0))
    # the caller path: host time to enqueue one step, eagerly and as a replayed CUDA graph of the same step
    caller = None
    if caller_path:
        from flash_attention_b200.generation import DecodeGraphs, InferenceParams, host_time_per_call_us

        params = InferenceParams(max_seqlen=cap, max_batch_size=B, lengths_per_sample=lens.clone())
        graphs = DecodeGraphs(lambda p, q_, kn_, vn_: fa.flash_attn_with_kvcache(
            q_, kc, vc, kn_, vn_, cos, sin, p.lengths_per_sample, causal=True, rotary_interleaved=False), params)
        replay = lambda: graphs.run(q, kn, vn, seqlen=lens)  # noqa: E731
        replay()
        caller = {"host_us_per_step_eager": host_time_per_call_us(step, 100),
                  "host_us_per_step_graph": host_time_per_call_us(replay, 100),
                  "ms_per_step_graph": statistics.median(timed_repeats(R, replay, steps, min_repeats=3, target_ms=200.0))}
        graphs.release()
    pk = peaks()
    res = {
        "value": gbs, "unit": "GB/s", "ms_per_step": ms, "repeats": len(per_step), "caller_path": caller,
        "config": {"workload": "decode_b%d_hq32_hk8_d128_cap%d" % (B, cap), "batch_per_gpu": B, "cache_capacity": cap,
                   "cache_seqlens": "uniform [%d, %d]" % (cap // 32, cap - 1), "new_tokens": 1,
                   "rotary": "neox, dim 128, base 10000",
                   "l2": "%.2f GiB of cache per GPU, larger than L2" % (2.0 * B * cap * Hk * D * 2 / 2 ** 30),
                   "bytes_model": "sum_b (L_b + 1) * 8 * 128 * 2 B * 2"},
        "roofline": {"bound": "hbm", "kernel": "decode_kernel (+ combine_kernel)", "achieved": gbs / R.world,
                     "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / R.world / pk["hbm_gbs"], "traffic": None,
                     "peak_source": pk["source"]},
        "e2e": {"value": R.world * nbytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": sum(x.numel() * x.element_size() for x in (hq, hk_, hv, hl)),
                "d2h_bytes_per_step": out_host.numel() * 2, "ms_per_step": ms_e2e},
        "gpu_launches_per_step": 2, "clocks": clk.summary(),
    }
    del kc, vc
    torch.cuda.empty_cache()
    return res


def run_decode(args):
    from flash_attention_b200 import _lib

    R = Ranks()
    small = args.workload == "decode_b8_cap8192"
    res = measure_decode(R, args.steps, args.warmup, *((8, 8192) if small else (64, 32768)), caller_path=not args.no_also)
    status = _lib.lib().fa_device_status()
    if R.rank == 0:
        print(json.dumps({
            "metric": "decode KV-cache GB/s (bf16, d128, split-KV)", "value": res["value"], "unit": "GB/s", "n_gpus": R.world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": res["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": res["config"],
            "roofline": res["roofline"], "cpu_baseline": None, "e2e": res["e2e"], "caller_path": res["caller_path"],
            "gpu_launches": args.steps * 2, "clocks": res["clocks"], "device_status": status,
        }))
    R.close()


# ------------------------------------------------------------------------------------------------ ring
def measure_ring(R, steps, warmup, single_gpu_too=True):
    """ONE sequence (batch 1, 32768 tokens, 32 query heads over 8 KV heads, head_dim 128, bf16, causal)
    sharded by rows over the ranks with context-parallel ring attention: strong scaling.  Next to it, on
    rank 0 alone, the same sequence on one GPU (plain local attention) as the base of the speed-up."""
    import flash_attention_b200 as fa
    from flash_attention_b200.ring import ring_flash_attn_func

    dev, world = R.dev, R.world
    S, H, Hk, D = 32768, 32, 8, 128
    flops = 3.5 * 4.0 * S * S * H * D / 2.0
    single = None
    if single_gpu_too or world == 1:
        if R.rank == 0:
            g = torch.Generator(device=dev).manual_seed(2)
            q, k, v = (torch.randn(1, S, h, D, device=dev, dtype=torch.bfloat16, generator=g).requires_grad_(True)
                       for h in (H, Hk, Hk))
            do = torch.randn(1, S, H, D, device=dev, dtype=torch.bfloat16, generator=g)

            def one():
                out = fa.flash_attn_func(q, k, v, causal=True)
                torch.autograd.grad(out, (q, k, v), do)

            for _ in range(3):
                one()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ts = []
            for _ in range(5):
                torch.cuda.synchronize()
                e0.record()
                one()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            ms1 = statistics.median(ts)
            single = {"value": flops / (ms1 * 1e-3) / 1e12, "ms_per_step": ms1}
            del q, k, v, do
            torch.cuda.empty_cache()
        R.barrier()
    if world == 1:
        return {"value": single["value"], "unit": "TFLOPS/s", "ms_per_step": single["ms_per_step"], "n_gpus": 1,
                "scaling": "strong", "config": {"workload": "ring_gqa_b1_s32768_h32_hk8_d128_causal", "rows_per_gpu": S,
                                                "note": "one GPU: a ring of one step is plain local attention"}}
    S_loc = S // world
    g = torch.Generator(device=dev).manual_seed(2 + R.rank)
    q = torch.randn(1, S_loc, H, D, device=dev, dtype=torch.bfloat16, generator=g).requires_grad_(True)
    k = torch.randn(1, S_loc, Hk, D, device=dev, dtype=torch.bfloat16, generator=g).requires_grad_(True)
    v = torch.randn(1, S_loc, Hk, D, device=dev, dtype=torch.bfloat16, generator=g).requires_grad_(True)
    do = torch.randn(1, S_loc, H, D, device=dev, dtype=torch.bfloat16, generator=g)

    def step():
        out = ring_flash_attn_func(q, k, v, causal=True, layout="zigzag")
        return torch.autograd.grad(out, (q, k, v), do)

    for _ in range(max(3, warmup)):
        step()
    per_step = timed_repeats(R, step, max(1, min(steps, 10)), target_ms=600.0, max_repeats=20)
    ms = statistics.median(per_step)
    res = {"value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOPS/s", "ms_per_step": ms, "n_gpus": world, "scaling": "strong",
           "repeats": len(per_step),
           "config": {"workload": "ring_gqa_b1_s32768_h32_hk8_d128_causal", "rows_per_gpu": S_loc, "layout": "zigzag",
                      "exchange": "K/V blocks by NCCL send/recv into local buffers; fp32 dK/dV partials stay local, one reduce-scatter at the end of the backward"}}
    if single is not None or R.rank != 0:
        base = torch.tensor([single["value"] if single else 0.0], device=dev, dtype=torch.float64)
        if R.dist is not None:
            R.dist.broadcast(base, src=0)
        res["single_gpu_value"] = base.item()
        res["speedup_over_single_gpu"] = res["value"] / base.item() if base.item() > 0 else None
    if world > 1:
        # the same kernels in the same order with nothing exchanged: what is left of a step is exchange that the
        # kernels did not hide (send/recv of K/V, the reduce-scatter of dK/dV)
        try:
            from flash_attention_b200 import ring

            with ring.kernels_only():
                step()
                ms_k = statistics.median(timed_repeats(R, step, max(1, min(steps, 10)), min_repeats=3, target_ms=200.0))
            res["kernels_only_ms_per_step"] = ms_k
            res["exposed_exchange_share"] = max(0.0, 1.0 - ms_k / ms)
        except Exception as e:  # a diagnostic: must not cost the number above
            res["kernels_only_error"] = repr(e)[:200]
    return res


def ring_parity_small(R):
    """A small ring problem checked against the oracle on the gathered sequence (rank 0 reports)."""
    from flash_attention_b200.ring import ring_flash_attn_func, zigzag_shard
    from oracle import attention_oracle as O

    world, dev = R.world, R.dev
    g = torch.Generator().manual_seed(0)
    S, H, Hk, D = 256 * 2 * world, 8, 2, 128
    q, k, v, do = (torch.randn(1, S, h, D, generator=g).bfloat16() for h in (H, Hk, Hk, H))
    sh = lambda x: zigzag_shard(x, R.rank, world).to(dev)  # noqa: E731
    ql, kl, vl = (sh(x).requires_grad_(True) for x in (q, k, v))
    out = ring_flash_attn_func(ql, kl, vl, causal=True, layout="zigzag")
    grads = torch.autograd.grad(out, (ql, kl, vl), sh(do))
    res = []
    for upcast in (True, False):
        qf, kf, vf = (x.to(dev).requires_grad_(True) for x in (q, k, v))
        ref, _ = O.attention_oracle(qf, kf, vf, causal=True, upcast=upcast, reorder_ops=not upcast)
        res.append((ref.detach(),) + torch.autograd.grad(ref, (qf, kf, vf), do.to(dev)))
    err = yard = 0.0
    for mine, t, l in zip((out.detach(),) + tuple(grads), *res):
        err = max(err, (mine.float() - sh(t.cpu()).float()).abs().max().item())
        yard = max(yard, (sh(l.cpu()).float() - sh(t.cpu()).float()).abs().max().item())
    err, yard = R.max_over_ranks(err), R.max_over_ranks(yard)
    return {"max_err": err, "yardstick": yard, "ok": bool(err <= 2 * yard + 1e-3), "seqlen": S}


def run_ring(args):
    from flash_attention_b200 import _lib

    R = Ranks()
    res = measure_ring(R, args.steps, args.warmup)
    if R.world > 1:
        res["parity"] = ring_parity_small(R)
    status = _lib.lib().fa_device_status()
    if R.rank == 0:
        print(json.dumps({
            "metric": "attention fwd+bwd TFLOPS/s (bf16, d128, causal, context-parallel ring)",
            "value": res["value"], "unit": "TFLOPS/s", "n_gpus": R.world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": res["config"], "ring": res, "device_status": status,
        }))
    R.close()


# ------------------------------------------------------------------------------------------------ rotary
def run_rotary(args):
    """Rotary embedding of q and k inside the default workload's packed qkv (16 x 2048 x 3 x 16 x 128 bf16 per GPU),
    in place, forward (the backward is the same kernel with the conjugate flag).  Metric: GB/s over the bytes of
    q and k read and written."""
    from flash_attention_b200 import _lib
    from flash_attention_b200.layers.rotary import apply_rotary_emb_qkv_

    R = Ranks()
    dev = R.dev
    B, S, H, D = 16, 2048, 16, 128
    g = torch.Generator(device=dev).manual_seed(5 + R.rank)
    qkv = torch.randn(B, S, 3, H, D, device=dev, dtype=torch.bfloat16, generator=g)
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2, device=dev).float() / D))
    fr = torch.outer(torch.arange(S, device=dev).float(), inv)
    cos, sin = torch.cos(fr).bfloat16(), torch.sin(fr).bfloat16()
    nbytes = 2.0 * 2 * B * S * H * D * 2  # q and k, read + write

    with torch.no_grad():
        for _ in range(max(3, args.warmup)):
            apply_rotary_emb_qkv_(qkv, cos, sin)
        with ClockSampler(R.local) as clk:
            # 268 MB of q, k per call: larger than L2
            per_step = timed_repeats(R, lambda: apply_rotary_emb_qkv_(qkv, cos, sin), args.steps, target_ms=500.0)
    ms = statistics.median(per_step)
    gbs = R.world * nbytes / (ms * 1e-3) / 1e9
    pk = peaks()
    if R.rank == 0:
        print(json.dumps({
            "metric": "rotary embedding GB/s (bf16, q and k of packed qkv, in place)", "value": gbs, "unit": "GB/s",
            "n_gpus": R.world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "rotary_qkv_b16_s2048_h16_d128", "batch_per_gpu": B, "seqlen": S, "heads": H, "head_dim": D,
                       "rotary_dim": D, "style": "neox", "l2": "268 MB of q and k per call, larger than L2",
                       "bytes_model": "2 (q, k) x 2 (read, write) x B S H D x 2 B"},
            "roofline": {"bound": "hbm", "kernel": "rotary_vec_kernel", "achieved": gbs / R.world, "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / R.world / pk["hbm_gbs"], "traffic": None, "peak_source": pk["source"]},
            "cpu_baseline": None, "e2e": None, "gpu_launches": args.steps, "clocks": clk.summary(),
            "device_status": _lib.lib().fa_device_status(),
        }))
    R.close()


# ------------------------------------------------------------------------------------------------ training shapes
def run_train(args, wl):
    import flash_attention_b200 as fa
    from flash_attention_b200 import _lib

    B, S, H, Hk, D, causal, dtype = WORKLOADS[wl]
    R = Ranks()
    dev, world = R.dev, R.world
    g = torch.Generator(device=dev).manual_seed(1 + R.rank)
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
    warm = max(3, args.warmup)
    for _ in range(warm):
        step(inputs, dout)
    # ---- timed region: K steps, device timed, max over ranks; repeated, median reported.  The GPU idles GAP_S before
    # every region: K steps of this workload are a burst of tens of milliseconds, and the denominator they are compared
    # with (the measured burst peak) was taken the same way.  The same regions back to back, where the 1 kW power cap
    # lowers the SM clock after ~0.1 s, are reported beside them as "sustained".
    GAP_S = 0.4
    with ClockSampler(R.local) as clk:
        per_step = timed_repeats(R, lambda: step(inputs, dout), args.steps, min_repeats=7, max_repeats=12, gap_s=GAP_S, clk=clk)
    ms_step = statistics.median(per_step)
    value = world * f_step / (ms_step * 1e-3) / 1e12
    clocks = clk.summary()
    with ClockSampler(R.local) as clk_s:
        ms_sustained = statistics.median(timed_repeats(R, lambda: step(inputs, dout), args.steps, target_ms=400.0, clk=clk_s))

    # ---- forward and backward timed separately (the kernels behind the roofline numbers)
    def forward_only():
        with torch.no_grad():
            forward(inputs)

    ms_fwd = statistics.median(timed_repeats(R, forward_only, args.steps, max_repeats=7, gap_s=GAP_S))
    out = forward(inputs)
    ms_bwd = statistics.median(timed_repeats(R, lambda: torch.autograd.grad(out, inputs, dout, retain_graph=True), args.steps,
                                             max_repeats=7, gap_s=GAP_S))
    del out
    pk = peaks()
    tf_fwd = f_fwd / (ms_fwd * 1e-3) / 1e12
    tf_bwd = 2.5 * f_fwd / (ms_bwd * 1e-3) / 1e12
    # The backward pass dominates a step.  FLOPs are the algorithmic 5 GEMMs; head dims up to 128 run a dK/dV kernel
    # and a dQ kernel that together execute 7 (S and dP twice), head dims above 128 one kernel as three passes
    # (dV, dK, dQ) that execute 8 (S three times, dP twice); a small bandwidth kernel (dot(dO, O)) precedes them.
    wide = D > 128
    bwd_kernels = ("backward (bwd_dot_do_o + bwd_wide_tc_kernel x3 [dV, dK, dQ passes])" if wide else
                   "backward (bwd_dot_do_o + bwd_tc_kernel [dK,dV] + bwd_dq_tc_kernel [dQ])")
    roofline = {"bound": "tensor", "kernel": bwd_kernels,
                "achieved": tf_bwd, "peak": pk["tflops_burst"], "unit": "TFLOP/s",
                "frac": tf_bwd / pk["tflops_burst"], "traffic": NCU_DRAM_BYTES_PER_BACKWARD.get(wl), "peak_source": pk["source"],
                "forward": {"kernel": "fwd_tc_kernel", "achieved": tf_fwd, "frac": tf_fwd / pk["tflops_burst"],
                            "frac_of_sustained": tf_fwd / pk["tflops_sustained"]},
                "step": {"achieved": value / world, "frac": value / world / pk["tflops_burst"]},
                "sustained": {"step_tflops": f_step / (ms_sustained * 1e-3) / 1e12, "ms_per_step": ms_sustained,
                              "peak": pk["tflops_sustained"],
                              "frac": f_step / (ms_sustained * 1e-3) / 1e12 / pk["tflops_sustained"],
                              "clocks": clk_s.summary(),
                              "note": "the same K-step regions back to back for >= 0.4 s, under the power cap; "
                                      "against the measured sustained peak"},
                "timing": "regions of K steps, GPU idle %.1f s before each, median of >= 7; against the measured burst peak" % GAP_S}

    # ---- end to end: every step copies its inputs from pinned host memory, computes, and copies its RESULT (out and
    # the gradient of every input) back to pinned host memory.  As a training loop would, the three stages run on
    # three streams with two buffers each, so a step costs max(h2d, compute, d2h), not their sum.
    host_in = [x.detach().cpu().pin_memory() for x in inputs]
    host_do = dout.cpu().pin_memory()
    dev_in = [[torch.empty_like(x).requires_grad_(True) for x in inputs] for _ in range(2)]
    dev_do = [torch.empty_like(dout) for _ in range(2)]
    h2d = sum(x.numel() * x.element_size() for x in host_in) + host_do.numel() * host_do.element_size()
    host_out = [torch.empty(dout.shape, dtype=dtype).pin_memory() for _ in range(2)]
    host_grads = [[torch.empty(x.shape, dtype=dtype).pin_memory() for x in inputs] for _ in range(2)]
    d2h = host_out[0].numel() * host_out[0].element_size() + sum(x.numel() * x.element_size() for x in host_grads[0])
    in_stream, out_stream = torch.cuda.Stream(), torch.cuda.Stream()
    main_stream = torch.cuda.current_stream()
    copied = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    computed = [torch.cuda.Event() for _ in range(2)]
    live = [None, None]  # results of a step stay referenced until their copy to the host has been queued behind them

    def e2e_steps(n):
        for buf in range(2):
            consumed[buf].record(main_stream)
        for i in range(n):
            buf = i & 1
            with torch.cuda.stream(in_stream):
                in_stream.wait_event(consumed[buf])  # the step that last used this buffer has finished
                for d_, h_ in zip(dev_in[buf], host_in):
                    d_.data.copy_(h_, non_blocking=True)
                dev_do[buf].copy_(host_do, non_blocking=True)
                copied[buf].record(in_stream)
            main_stream.wait_event(copied[buf])
            o, grads = step(tuple(dev_in[buf]), dev_do[buf])
            consumed[buf].record(main_stream)
            computed[buf].record(main_stream)
            with torch.cuda.stream(out_stream):
                out_stream.wait_event(computed[buf])
                host_out[buf].copy_(o.detach(), non_blocking=True)
                for h_, g_ in zip(host_grads[buf], grads):
                    h_.copy_(g_, non_blocking=True)
                    g_.record_stream(out_stream)
                o.record_stream(out_stream)
            live[buf] = (o, grads)
        main_stream.wait_stream(out_stream)

    e2e_steps(2)
    n_e2e = max(4, min(args.steps, 10))
    ms_e2e = statistics.median(timed_repeats(R, lambda: e2e_steps(n_e2e), 1, min_repeats=3, target_ms=300.0, max_repeats=5)) / n_e2e
    e2e_val = world * f_step / (ms_e2e * 1e-3) / 1e12
    live[0] = live[1] = None
    del host_in, host_do, host_out, host_grads, dev_in, dev_do
    torch.cuda.empty_cache()

    # ---- the other headline numbers, measured in this same run
    also = {"fwd": {"value": world * tf_fwd, "unit": "TFLOPS/s", "ms": ms_fwd, "kernel": "fwd_tc_kernel",
                    "frac_of_peak": tf_fwd / pk["tflops_burst"], "peak": pk["tflops_burst"], "peak_source": pk["source"]},
            "bwd": {"value": world * tf_bwd, "unit": "TFLOPS/s", "ms": ms_bwd, "frac_of_peak": tf_bwd / pk["tflops_burst"]}}
    launches = args.steps * (5 if wide else 4)
    if wl == DEFAULT and not args.no_also:
        for name, fn in (("decode", lambda: measure_decode(R, max(3, min(args.steps, 20)), 3)),
                         ("shapes", lambda: measure_other_shapes(R, max(2, min(args.steps, 10)))),
                         ("ring", lambda: measure_ring(R, max(2, min(args.steps, 5)), 2))):
            try:
                also[name] = fn()
            except Exception as e:  # a failure here must not cost the main line
                also[name] = {"error": "%s: %s" % (type(e).__name__, e)}
                R.barrier()
        if world > 1 and "error" not in also.get("ring", {}):
            try:
                also["ring"]["parity"] = ring_parity_small(R)
            except Exception as e:
                also["ring"]["parity"] = {"error": "%s: %s" % (type(e).__name__, e)}
    status = _lib.lib().fa_device_status()

    if R.rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            units = 16
            dt, kind = cpu_attention_sample(D, S, causal, heads=units, budget_s=12.0)
            what = "attention_ref of the reference's tests" if kind == "reference" else "fp32 attention_ref restatement"
            cpu = {"value": 3.5 * fwd_flops(1, S, units, D, causal) / dt / 1e12, "unit": "TFLOPS/s",
                   "cores": os.cpu_count() or 1, "kind": kind,
                   "sample": "%d of %d (batch x head) units at full seqlen %d per pass, %s, fwd+bwd, best of ~12 s of passes (%.2f s per pass)" % (units, B * H, S, what, dt)}
        mhz = clocks.get("sm_mhz")
        line = {
            "metric": METRIC,
            "value": value, "unit": "TFLOPS/s", "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16" if dtype == torch.bfloat16 else "fp16", "data": "synthetic",
            "config": {"workload": wl, "batch_per_gpu": B, "seqlen": S, "heads": H, "heads_k": Hk, "head_dim": D,
                       "causal": causal, "dropout_p": 0.0, "api": "flash_attn_qkvpacked_func" if packed else "flash_attn_func",
                       "l2": "inputs (%.0f MiB per step) larger than L2" % (h2d / 2**20),
                       "flop_model": "fwd 4*B*S^2*H*D%s, bwd 2.5x" % ("/2" if causal else ""),
                       "parallelism": "independent (batch x head) units per GPU, no communication"},
            "timing": {"repeats": len(per_step), "ms_per_step_min": min(per_step), "ms_per_step_max": max(per_step),
                       "ms_per_step_median": ms_step, "ms_times_sm_mhz": ms_step * mhz if mhz else None,
                       "idle_s_before_each_region": GAP_S, "ms_per_step_back_to_back": ms_sustained},
            "fwd_tflops": tf_fwd, "bwd_tflops": tf_bwd, "ms_fwd": ms_fwd, "ms_bwd": ms_bwd,
            "roofline": roofline, "cpu_baseline": cpu,
            "e2e": {"value": e2e_val, "unit": "TFLOPS/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": ms_e2e,
                    "pipeline": "inputs in (pinned host -> device), forward + backward, out and all input gradients back "
                                "(device -> pinned host); three streams, two buffers each: a step costs max(h2d, compute, d2h)"},
            "also": also,
            "gpu_launches": launches,
            "clocks": clocks, "device_status": status,
        }
        print(json.dumps(line))
    R.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-also", action="store_true", help="skip the decode and ring measurements of the default workload, and the caller-path part of the decode workload")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args, args.workload if args.workload in WORKLOADS else DEFAULT)
    if args.workload == "ring":
        return run_ring(args)
    if args.workload == "rotary":
        return run_rotary(args)
    if args.workload in ("decode", "decode_b8_cap8192"):
        return run_decode(args)
    return run_train(args, args.workload)


if __name__ == "__main__":
    main()
