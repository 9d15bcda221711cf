"""PreparedDecode on the GPU: eager and CUDA-graph steps against the FP64 oracle, capture leaves the
visible cache state untouched, buffer addresses stay fixed, delta uploads happen only on new pages,
and lifecycle / validation errors are atomic (cases of tests/test_prepared_decode.py and
tests/test_decode_routing.py in the reference)."""
import numpy as np
import pytest
import torch

from helpers import torch_to_f64
from oracle import moba_oracle as mo

pytestmark = pytest.mark.gpu


def rand(shape, seed, dtype=torch.bfloat16):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)).to("cuda", dtype)


def reference(cache, result, q):
    import moba_opt.grouped_attention as ga
    ga.check_status()
    kv = [cache.materialize(i) for i in range(len(cache.lengths))]
    sel = None if result.selected_blocks is None else result.selected_blocks.cpu().numpy()
    out, lse = mo.decode_attend(torch_to_f64(q), [torch_to_f64(x[0]) for x in kv], [torch_to_f64(x[1]) for x in kv],
                                result.sequence_ids, result.positions, cache.chunk_size, sel)
    np.testing.assert_allclose(torch_to_f64(result.output), out, atol=0.02, rtol=0.02)
    np.testing.assert_allclose(torch_to_f64(result.lse), lse, atol=5e-4, rtol=2e-5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("graph", [False, True])
@pytest.mark.parametrize("page,chunk,dim,hq,hk", [(3, 4, 40, 15, 3), (7, 6, 64, 8, 1), (16, 8, 128, 8, 2), (48, 16, 128, 12, 2)])
def test_prepared_steps_match_oracle_and_payload(graph, page, chunk, dim, hq, hk, dtype):
    from moba_opt import PagedKVCache
    from functools import partial
    rand = partial(globals()["rand"], dtype=dtype)
    half = dtype == torch.float16
    cache = PagedKVCache(3, 40, hk, dim, page_size=page, chunk_size=chunk, dtype=dtype)
    k, v = rand((14, hk, dim), 501), rand((14, hk, dim), 502)
    cache.append(k, v, sequence_ids=[2, 0], cu_seqlens=[0, 5, 14])
    stored_k, stored_v = {2: k[:5], 0: k[5:]}, {2: v[:5], 0: v[5:]}
    lengths, table = cache.lengths, cache.page_table
    before = [cache.materialize(s) for s in (2, 0)]
    with cache.prepare_decode([2, 0], hq, topk=3) as plan:
        if graph:
            plan.capture("step").capture("attend")
            assert cache.lengths == lengths and cache.page_table == table
            for sid, (bk, bv) in zip((2, 0), before):
                ak, av = cache.materialize(sid)
                assert torch.equal(ak, bk) and torch.equal(av, bv)
        pointers = [t.data_ptr() for t in (cache._table, cache._lengths, plan.output, plan.scores, plan.selected)]
        for step in range(10):
            q = rand((2, hq, dim), 510 + step)
            kn, vn = rand((2, hk, dim), 530 + step), rand((2, hk, dim), 550 + step)
            result = plan.step(q, kn, vn, use_graph=graph)
            for i, sid in enumerate((2, 0)):
                stored_k[sid] = torch.cat((stored_k[sid], kn[i:i + 1]))
                stored_v[sid] = torch.cat((stored_v[sid], vn[i:i + 1]))
                actual = cache.materialize(sid)
                assert torch.equal(actual[0], stored_k[sid]) and torch.equal(actual[1], stored_v[sid])
            reference(cache, result, q)
            reference(cache, plan.attend(q, use_graph=graph), q)
            closed = cache.lengths[2] // chunk
            if closed:
                want = mo.chunk_means(torch_to_f64(stored_k[2]), chunk, rounding=mo.fp16_round if half else mo.bf16_round)
                np.testing.assert_allclose(torch_to_f64(cache._means[2, :closed]), want, atol=1e-5, rtol=0.002 if half else 0.01)
        assert pointers == [t.data_ptr() for t in (cache._table, cache._lengths, plan.output, plan.scores, plan.selected)]
        assert plan.delta_uploads <= 10
        with pytest.raises(ValueError, match="owns cache"):
            cache.reset()
    cache.reset([2])
    assert cache.lengths == (19, 0, 0)


def test_graph_and_eager_steps_are_bit_identical():
    from moba_opt import PagedKVCache
    outs = []
    for graph in (False, True):
        cache = PagedKVCache(2, 200, 2, 64, page_size=48, chunk_size=16)
        cache.append(rand((150, 2, 64), 701), rand((150, 2, 64), 702), sequence_ids=[0, 1], cu_seqlens=[0, 90, 150])
        with cache.prepare_decode([0, 1], 8, topk=4, check_finite=False) as p:
            if graph:
                p.capture("step")
            seq = []
            for step in range(20):
                r = p.step(rand((2, 8, 64), 710 + step), rand((2, 2, 64), 740 + step), rand((2, 2, 64), 770 + step), use_graph=graph)
                seq.append((r.output.clone(), r.lse.clone(), r.selected_blocks.clone()))
            outs.append(seq)
    for (o1, l1, s1), (o2, l2, s2) in zip(*outs):
        assert torch.equal(o1, o2) and torch.equal(l1, l2) and torch.equal(s1, s2)


@pytest.mark.parametrize("graph", [False, True])
@pytest.mark.parametrize("mode,topk", [("moba", 1), ("dense", 4), ("moba", 9)])
def test_prepared_empty_and_dense_fallback(graph, mode, topk):
    from moba_opt import PagedKVCache
    cache = PagedKVCache(1, 17, 1, 8, page_size=3, chunk_size=4)
    with cache.prepare_decode([0], 4, topk=topk, mode=mode) as p:
        if graph:
            p.capture("step")
        for step in range(9):
            q, kv = rand((1, 4, 8), 601 + step), rand((1, 1, 8), 621 + step)
            reference(cache, p.step(q, kv, kv, use_graph=graph), q)


def test_validation_lifecycle_capacity_and_metadata_delta():
    from moba_opt import PagedKVCache
    c = PagedKVCache(1, 7, 1, 8, page_size=3, chunk_size=4)
    q = torch.ones((1, 1, 8), device="cuda", dtype=c.dtype)
    with c.prepare_decode([0], 1) as p:
        before = c.lengths
        with pytest.raises(ValueError, match="NaN/Inf"):
            p.step(q * float("nan"), q, q)
        with pytest.raises(ValueError, match="capture"):
            p.step(q, q, q, use_graph=True)
        assert c.lengths == before
        for _ in range(7):
            p.step(q, q, q)
        assert p.delta_uploads == 3
        with pytest.raises(ValueError, match="max_seq_len"):
            p.step(q, q, q)
        assert c.lengths == (7,)
        with torch.cuda.stream(torch.cuda.Stream()):
            with pytest.raises(ValueError, match="cross-stream"):
                p.attend(q)
    with pytest.raises(ValueError, match="closed"):
        p.step(q, q, q)
    assert c.lengths == (7,)


def test_input_workspace_alias_and_output_reuse_contract():
    from moba_opt import PagedKVCache
    c = PagedKVCache(1, 8, 1, 8, page_size=3, chunk_size=4)
    q = torch.ones((1, 1, 8), device="cuda", dtype=c.dtype)
    with c.prepare_decode([0], 1, check_finite=False) as p:
        with pytest.raises(ValueError, match="aliases"):
            p.step(p.v, p.k, p.q)
        a = p.step(q, q, q)
        b = p.step(q, q, q)
        assert a.output.data_ptr() == b.output.data_ptr()


def test_capture_after_live_steps_and_graph_capacity_boundary():
    from moba_opt import PagedKVCache
    c = PagedKVCache(1, 4, 1, 8, page_size=1, chunk_size=2)
    q = torch.ones(1, 1, 8, device="cuda", dtype=c.dtype)
    with c.prepare_decode([0], 1) as p:
        for value in (1, 2, 3):
            p.step(q, q, q * value)
        before = c.materialize(0)
        p.capture("step").capture("attend")
        assert c.lengths == (3,)
        assert torch.equal(before[0], c.materialize(0)[0]) and torch.equal(before[1], c.materialize(0)[1])
        reference(c, p.step(q, q, q * 4, use_graph=True), q)
        with pytest.raises(ValueError, match="max_seq_len"):
            p.step(q, q, q, use_graph=True)
        assert c.lengths == (4,)


def test_graph_closes_large_chunk_at_maximum_head_dimension():
    from moba_opt import PagedKVCache
    c = PagedKVCache(1, 2050, 1, 256, page_size=48, chunk_size=2048)
    k, v = rand((2047, 1, 256), 801), rand((2047, 1, 256), 802)
    c.append(k, v, sequence_ids=[0], cu_seqlens=[0, 2047])
    q = rand((1, 4, 256), 803)
    kn, vn = k[:1].clone(), v[:1].clone()
    with c.prepare_decode([0], 4) as p:
        p.capture("step")
        reference(c, p.step(q, kn, vn, use_graph=True), q)
        expected = torch.cat((k, kn)).float().mean(0).to(c.dtype)
        torch.testing.assert_close(c._means[0, 0], expected, atol=1e-5, rtol=0.01)
        reference(c, p.step(q, kn, vn, use_graph=True), q)   # first query that can route to chunk 0


def test_bound_input_buffers_support_graph_without_staging_copies():
    from moba_opt import PagedKVCache
    c = PagedKVCache(1, 8, 1, 8, page_size=4, chunk_size=2)
    with c.prepare_decode([0], 1, check_finite=False) as p:
        p.q.fill_(1)
        p.k.fill_(1)
        p.v.fill_(2)
        p.capture("step")
        for _ in range(3):
            result = p.step(p.q, p.k, p.v, use_graph=True)
            assert torch.equal(result.output, torch.full_like(result.output, 2))
        assert p.delta_uploads == 1
        with pytest.raises(ValueError, match="owns cache"):
            c.prepare_decode([0], 1)


def test_no_history_preserves_padding():
    from moba_opt import PagedKVCache
    cache = PagedKVCache(2, 65, 1, 8, page_size=7, chunk_size=8)
    data = torch.ones(65, 1, 8, device="cuda", dtype=cache.dtype)
    cache.append(data, data, sequence_ids=[1], cu_seqlens=[0, 65])
    q = torch.ones(1, 4, 8, device="cuda", dtype=cache.dtype)
    result = cache.attend(q, sequence_ids=[1], positions=[0], topk=9)
    assert result.selected_blocks.shape == (1, 4, 9)
    assert (result.selected_blocks[:, :, 0] == 0).all()
    assert (result.selected_blocks[:, :, 1:] == -1).all()
    cache.reset()
    assert cache._candidate_count == 0


def test_device_metadata_mirrors_cpu_layout():
    from moba_opt import PagedKVCache
    cache = PagedKVCache(2, 16, 1, 8, page_size=3, chunk_size=4)
    q = torch.ones(3, 4, 8, device="cuda", dtype=cache.dtype)
    kv = torch.ones(3, 1, 8, device="cuda", dtype=cache.dtype)
    result = cache.append_and_attend(q, kv, kv, sequence_ids=[1, 0], cu_seqlens=[0, 2, 3])
    assert result.sequence_ids == (1, 1, 0) and result.positions == (0, 1, 0)
    again = cache.attend(q, sequence_ids=[1, 1, 0], positions=[0, 1, 0])
    assert torch.equal(result.output, again.output)
    assert torch.equal(cache._table.cpu(), torch.tensor(cache.page_table, dtype=torch.int32))
    assert torch.equal(cache._lengths.cpu(), torch.tensor(cache.lengths, dtype=torch.int32))


@pytest.mark.parametrize("bad_name", ["q", "k", "v"])
def test_combined_api_rejects_nonfinite_before_append(bad_name):
    from moba_opt import PagedKVCache
    cache = PagedKVCache(1, 8, 1, 8, page_size=3, chunk_size=4)
    tensors = {"q": torch.ones(1, 4, 8, device="cuda", dtype=cache.dtype), "k": torch.ones(1, 1, 8, device="cuda", dtype=cache.dtype),
               "v": torch.ones(1, 1, 8, device="cuda", dtype=cache.dtype)}
    tensors[bad_name][0, 0, 0] = float("nan")
    with pytest.raises(ValueError, match="NaN/Inf"):
        cache.append_and_attend(**tensors, sequence_ids=[0])
    assert cache.lengths == (0,)
