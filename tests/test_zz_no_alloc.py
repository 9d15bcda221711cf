"""Routing through the entry point that brings its own scratch memory.

`moba_prefill_route_static` serves hosts that cannot allocate on the device - a process whose GPU
memory was given to one pool at start-up, a request path where cudaMalloc is banned because it stalls
the whole device, a binding that only holds tensors handed to it.  It must produce exactly the route
state of `moba_prefill_route`, call after call, although every call reuses the same built-in array.
This file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _route_states(lens, hq, hkv, dim, chunk, topk, seed):
    from moba_opt import _ext
    import moba_opt.grouped_attention as ga
    lib = _ext.lib()
    dev = torch.device("cuda", 0)
    rng = torch.Generator().manual_seed(seed)
    total = sum(lens)
    q = torch.randn(total, hq, dim, generator=rng).bfloat16().to(dev)
    k = torch.randn(total, hkv, dim, generator=rng).bfloat16().to(dev)
    cu = [0] + list(np.cumsum(lens))
    plan = ga.get_plan(cu, chunk, dev)
    remote_k = min(topk - 1, plan.num_routable)
    with torch.cuda.device(dev):
        want = ga.route(q, k, plan, remote_k)                       # caller-allocated scratch
        d = plan.desc(q, k, k, remote_k)
        assert lib.moba_prefill_route_scratch_bytes(ctypes.byref(d)) <= lib.moba_prefill_route_static_capacity()
        got = torch.zeros_like(want)
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        rc = lib.moba_prefill_route_static(ctypes.byref(d), q.data_ptr(), k.data_ptr(), got.data_ptr(), stream)
        assert rc == 0, lib.moba_status_string(rc)
        torch.cuda.synchronize()
    used = total * hq * remote_k * 4                                 # sel table; the lists follow it
    return want, got, used, plan, remote_k, hq, hkv


def _compare(want, got, used, plan, remote_k, hq, hkv):
    # sel[T,Hq,R] is fully defined; of rowlist only the first M entries are, M = seg_base[-1]
    assert torch.equal(want[:used], got[:used])
    align = lambda x: (x + 255) // 256 * 256
    rows_bytes = align(used)
    seg_off = 2 * rows_bytes
    nseg = plan.num_chunks * hq + 1
    seg_w = want[seg_off:seg_off + nseg * 4].view(torch.int32)
    seg_g = got[seg_off:seg_off + nseg * 4].view(torch.int32)
    assert torch.equal(seg_w, seg_g)
    m = int(seg_w[-1].item())
    assert m > 0
    assert torch.equal(want[rows_bytes:rows_bytes + m * 4], got[rows_bytes:rows_bytes + m * 4])
    tile_off = seg_off + align(nseg * 4)
    ntile = plan.num_chunks * hkv + 1
    assert torch.equal(want[tile_off:tile_off + ntile * 4], got[tile_off:tile_off + ntile * 4])


def test_static_scratch_routing_matches_twice_in_a_row():
    # two different problems back to back: the second call finds the first call's leftovers in the array
    first = _route_states((700, 1300), 4, 2, 64, 256, 3, seed=11)
    _compare(*first)
    second = _route_states((333, 90), 6, 1, 128, 48, 4, seed=12)
    _compare(*second)
    again = _route_states((700, 1300), 4, 2, 64, 256, 3, seed=11)
    _compare(*again)
    assert torch.equal(first[1], again[1])


def test_static_scratch_call_allocates_nothing():
    """What the entry point is for: once the first call on the device has looked up the built-in array, a call
    changes neither the device's free memory (cudaMemGetInfo: it sees every allocation of the process, the caching
    allocator's included) nor torch's own count of allocated and reserved bytes."""
    from moba_opt import _ext
    import moba_opt.grouped_attention as ga
    lib = _ext.lib()
    dev = torch.device("cuda", 0)
    rng = torch.Generator().manual_seed(13)
    q = torch.randn(2048, 4, 64, generator=rng).bfloat16().to(dev)
    k = torch.randn(2048, 2, 64, generator=rng).bfloat16().to(dev)
    plan = ga.get_plan([0, 2048], 256, dev)
    with torch.cuda.device(dev):
        d = plan.desc(q, k, k, 2)
        state = torch.zeros(lib.moba_prefill_route_state_bytes(ctypes.byref(d)), dtype=torch.uint8, device=dev)
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        call = lambda: lib.moba_prefill_route_static(ctypes.byref(d), q.data_ptr(), k.data_ptr(), state.data_ptr(), stream)
        assert call() == 0                                 # first call on the device: address look-up
        torch.cuda.synchronize()
        before = (torch.cuda.mem_get_info(dev)[0], torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev))
        for _ in range(3):
            assert call() == 0
        torch.cuda.synchronize()
        after = (torch.cuda.mem_get_info(dev)[0], torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev))
    assert after == before


def test_static_scratch_rejects_oversized_problem():
    from moba_opt import _ext
    import moba_opt.grouped_attention as ga
    lib = _ext.lib()
    dev = torch.device("cuda", 0)
    # many tiny chunks: the per-(chunk, head, tile) count table alone outgrows the built-in array
    total, hq = 16384, 16
    plan = ga.get_plan([0, total], 16, dev)
    q = torch.zeros(total, hq, 8, dtype=torch.bfloat16, device=dev)
    k = torch.zeros(total, 1, 8, dtype=torch.bfloat16, device=dev)
    d = plan.desc(q, k, k, 2)
    assert lib.moba_prefill_route_scratch_bytes(ctypes.byref(d)) > lib.moba_prefill_route_static_capacity()
    state = torch.zeros(lib.moba_prefill_route_state_bytes(ctypes.byref(d)), dtype=torch.uint8, device=dev)
    rc = lib.moba_prefill_route_static(ctypes.byref(d), q.data_ptr(), k.data_ptr(), state.data_ptr(), None)
    assert rc == 3 and b"workspace" in lib.moba_status_string(rc)
