"""tcgen05 tile primitives: one-CTA matrix products in every operand-major combination; and the bounded barrier wait
running out the way it would on a protocol fault: status bit, RuntimeError on the host, context still usable."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode,n,k", [(0, 128, 64), (0, 128, 128), (0, 256, 128), (1, 64, 128), (1, 128, 128),
                                      (2, 64, 128), (2, 128, 128), (2, 128, 16), (3, 64, 128), (3, 128, 128), (3, 64, 64)])
def test_umma_selftest(mode, n, k):
    from moba_opt import _ext
    lib = _ext.lib()
    dev = "cuda"
    gen = torch.Generator(device=dev).manual_seed(mode * 1000 + n + k)
    if mode == 0:
        a, b = torch.randn(128, k, device=dev, generator=gen).bfloat16(), torch.randn(n, k, device=dev, generator=gen).bfloat16()
        ref = a.float() @ b.float().T
    elif mode in (1, 3):
        a, b = torch.randn(128, k, device=dev, generator=gen).bfloat16(), torch.randn(k, n, device=dev, generator=gen).bfloat16()
        ref = a.float() @ b.float()
    else:
        a, b = torch.randn(k, 128, device=dev, generator=gen).bfloat16(), torch.randn(k, n, device=dev, generator=gen).bfloat16()
        ref = a.float().T @ b.float()
    d = torch.full((128, n), float("nan"), device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = lib.moba_selftest_umma(mode, a.data_ptr(), b.data_ptr(), d.data_ptr(), n, k, status.data_ptr(), None)
    torch.cuda.synchronize()
    assert rc == 0 and int(status.item()) == 0
    assert (d - ref).abs().max().item() < 1e-3


def test_bounded_wait_runs_out_and_the_host_sees_it():
    """A barrier wait that nothing satisfies ends by itself after its limit (here 2e6 SM clocks, about a millisecond;
    the kernels use 2e9), the kernel returns, and the error surfaces as RuntimeError from check_status() - after
    which the same context runs the next kernel normally."""
    from moba_opt import _ext
    import moba_opt.grouped_attention as ga
    lib = _ext.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    ga.check_status()
    status = ga._status_word(dev)
    returned = torch.zeros(1, dtype=torch.int32, device=dev)
    assert lib.moba_selftest_wait(0, status.data_ptr(), returned.data_ptr(), None) == 1       # limit outside 1..2e9
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    assert lib.moba_selftest_wait(2_000_000, status.data_ptr(), returned.data_ptr(), None) == 0
    t1.record()
    torch.cuda.synchronize()
    assert int(returned.item()) == 2                     # the wait gave up, the kernel ran to its end
    assert 0.2 < t0.elapsed_time(t1) < 200.0             # and it did wait, for about the limit
    with pytest.raises(RuntimeError, match="status bits 0x1"):
        ga.check_status()
    ga.check_status()                                    # the word is cleared by the report
    test_umma_selftest(0, 128, 64)                       # the context is intact
