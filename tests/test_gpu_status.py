"""The failure path of the bounded waits, exercised without faulting or hanging anything: a self-test
kernel waits ~1 ms for a barrier that nobody arrives at, gives up, and records its code exactly as a
stuck pipeline would.  The host must then see the failure (status 3 on the next call, RuntimeError
through the python module) until fa_device_status() has read and cleared it, and work normally after."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    import flash_attention_b200 as fa
    from flash_attention_b200 import _lib


def test_a_wait_that_runs_out_is_reported_and_cleared():
    lib = _lib.lib()
    q = torch.randn(2, 256, 4, 64, device="cuda", dtype=torch.float16)
    ref = fa.flash_attn_func(q, q, q, causal=True)  # also creates the host mirror of the status word
    torch.cuda.synchronize()
    assert lib.fa_device_status() == 0
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.fa_selftest_wait_timeout(2_000_000, stream) == 0  # ~1 ms of SM cycles
    torch.cuda.synchronize()
    # the next call is refused before any launch, with a message, not answered with unwritten tensors
    with pytest.raises(RuntimeError, match="gave up on a bounded wait"):
        fa.flash_attn_func(q, q, q, causal=True)
    assert lib.fa_device_status() == 99  # reads and clears
    assert lib.fa_device_status() == 0
    out = fa.flash_attn_func(q, q, q, causal=True)
    assert torch.equal(out, ref)


def test_second_device_gets_its_own_kernel_setup():
    # the shared-memory opt-in of a kernel is per device: a process that drives two GPUs must be
    # able to launch on the second one after the first
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    outs = []
    for dev in ("cuda:0", "cuda:1"):
        g = torch.Generator().manual_seed(0)
        q = torch.randn(1, 512, 16, 128, generator=g).bfloat16().to(dev).requires_grad_(True)
        o = fa.flash_attn_func(q, q, q, causal=True)
        (dq,) = torch.autograd.grad(o, q, torch.ones_like(o))
        outs.append((o.detach().cpu(), dq.cpu()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
