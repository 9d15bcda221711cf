"""tcgen05 tile primitives: one-CTA matrix products in every operand-major combination."""
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
