"""GPU parity of the KV cache and decode path against the FP64 oracle.  The cases follow the
reference's decode tests (tests/test_paged_decode.py): cache read-back bit-equal to what was
appended, chunk means, legality and ranking of routes, output/LSE under the kernel's own routes
(bf16: atol = rtol = 0.02, rel-L2 < 0.01, LSE atol 5e-4), page sizes that do not divide the chunk,
recycled pages, chunked (multi-token) appends, per-head routing known answers, error atomicity."""
import numpy as np
import pytest
import torch

from helpers import DECODE_GOLDENS, bits_to_torch, load, torch_to_f64
from oracle import moba_oracle as mo

pytestmark = pytest.mark.gpu


def rand(shape, seed, dtype=torch.bfloat16):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)).to("cuda", dtype)


def assert_payload(cache, sid, k, v):
    got_k, got_v = cache.materialize(sid)
    assert torch.equal(got_k, k) and torch.equal(got_v, v)


def check(cache, result, q):
    import moba_opt.grouped_attention as ga
    ga.check_status()
    C = cache.chunk_size
    keys, values = [], []
    for sid in range(len(cache.lengths)):
        k, v = cache.materialize(sid)
        keys.append(torch_to_f64(k))
        values.append(torch_to_f64(v))
        closed = cache.lengths[sid] // C
        if closed:
            half = cache.dtype == torch.float16
            want = mo.chunk_means(keys[-1], C, rounding=mo.fp16_round if half else mo.bf16_round)
            got = torch_to_f64(cache._means[sid, :closed])
            np.testing.assert_allclose(got, want, atol=1e-5, rtol=0.002 if half else 0.01)   # at most one ulp of the format apart
    qf = torch_to_f64(q)
    if result.selected_blocks is not None:
        route = result.selected_blocks.cpu().numpy()
        for row, (sid, pos) in enumerate(zip(result.sequence_ids, result.positions)):
            history = pos // C
            assert (route[row, :, 0] == history).all()
            means = torch_to_f64(cache._means[sid, :history]) if history else None
            for head in range(q.shape[1]):
                chosen = [int(c) for c in route[row, head, 1:] if c >= 0]
                assert len(chosen) == min(history, route.shape[-1] - 1)
                assert len(set(chosen)) == len(chosen) and all(c < history for c in chosen)
                if not chosen or len(chosen) == history:
                    continue
                kvh = head // (q.shape[1] // cache.num_kv_heads)
                scores = means[:, kvh] @ qf[row, head]
                rest = [i for i in range(history) if i not in chosen]
                bound = max(1e-6, float((np.abs(means[:, kvh]) @ np.abs(qf[row, head])).max())
                            * 4 * np.finfo(np.float32).eps * cache.head_dim)
                assert scores[chosen].min() + bound >= scores[rest].max()
    sel = None if result.selected_blocks is None else result.selected_blocks.cpu().numpy()
    want, lse = mo.decode_attend(qf, keys, values, result.sequence_ids, result.positions, C, sel)
    out = torch_to_f64(result.output)
    assert np.isfinite(out).all() and bool(torch.isfinite(result.lse).all())
    np.testing.assert_allclose(out, want, atol=0.02, rtol=0.02)
    assert np.linalg.norm(out - want) / max(np.linalg.norm(want), 1e-8) < 0.01
    np.testing.assert_allclose(torch_to_f64(result.lse), lse, atol=5e-4, rtol=2e-5)


@pytest.mark.parametrize("name", DECODE_GOLDENS)
def test_decode_matches_reference_golden(name):
    """Same inputs and hand-made routes as the fixtures produced by reference/decode_reference.py."""
    from moba_opt import PagedKVCache
    g = load(name)
    lengths, hq, hkv, dim, chunk = g["lengths"], int(g["hq"]), int(g["hkv"]), int(g["dim"]), int(g["chunk"])
    n = len(lengths)
    ks = [bits_to_torch(g[f"k{i}"], "cuda") for i in range(n)]
    vs = [bits_to_torch(g[f"v{i}"], "cuda") for i in range(n)]
    cache = PagedKVCache(n, int(max(lengths)) + 1, hkv, dim, page_size=5, chunk_size=chunk, dtype=ks[0].dtype)
    cache.append(torch.cat(ks), torch.cat(vs), sequence_ids=list(range(n)), cu_seqlens=[0] + [int(x) for x in np.cumsum(lengths)])
    q = bits_to_torch(g["q"], "cuda")
    dense = cache.attend(q, sequence_ids=list(range(n)), mode="dense")
    np.testing.assert_allclose(torch_to_f64(dense.output), g["out_dense"], atol=0.02, rtol=0.02)
    np.testing.assert_allclose(torch_to_f64(dense.lse), g["lse_dense"], atol=5e-4, rtol=2e-5)
    check(cache, dense, q)
    check(cache, cache.attend(q, sequence_ids=list(range(n)), topk=int(g["topk"])), q)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("kind", ["paged", "contiguous"])
@pytest.mark.parametrize("hq,hk", [(1, 1), (8, 1), (8, 2), (28, 4), (32, 8)])
def test_incremental_decode(kind, hq, hk, dtype):
    from moba_opt import ContiguousKVCache, PagedKVCache
    from functools import partial
    rand = partial(globals()["rand"], dtype=dtype)
    cache = (PagedKVCache(2, 32, hk, 64, chunk_size=4, page_size=3, dtype=dtype) if kind == "paged"
             else ContiguousKVCache(2, 32, hk, 64, chunk_size=4, dtype=dtype))
    k, v = rand((9, hk, 64), 101), rand((9, hk, 64), 102)
    cache.append(k, v, sequence_ids=[0, 1], cu_seqlens=[0, 4, 9])
    stored_k, stored_v = [k[:4], k[4:]], [v[:4], v[4:]]
    for sid in range(2):
        assert_payload(cache, sid, stored_k[sid], stored_v[sid])
    for step in range(3):
        q, k, v = rand((2, hq, 64), 103 + step), rand((2, hk, 64), 113 + step), rand((2, hk, 64), 123 + step)
        result = cache.append_and_attend(q, k, v, sequence_ids=[0, 1], topk=2)
        for sid in range(2):
            stored_k[sid] = torch.cat((stored_k[sid], k[sid:sid + 1]))
            stored_v[sid] = torch.cat((stored_v[sid], v[sid:sid + 1]))
            assert_payload(cache, sid, stored_k[sid], stored_v[sid])
        check(cache, result, q)
        check(cache, cache.attend(q, sequence_ids=[0, 1], mode="dense"), q)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("dim", [8, 16, 24, 40, 64, 80, 96, 128, 136, 192, 256])
def test_decode_head_dimensions(dim, dtype):
    from moba_opt import PagedKVCache
    from functools import partial
    rand = partial(globals()["rand"], dtype=dtype)
    cache = PagedKVCache(2, 64, 2, dim, page_size=7, chunk_size=12, dtype=dtype)
    k, v = rand((68, 2, dim), 131), rand((68, 2, dim), 132)
    cache.append(k, v, sequence_ids=[0, 1], cu_seqlens=[0, 27, 68])
    assert_payload(cache, 0, k[:27], v[:27])
    assert_payload(cache, 1, k[27:], v[27:])
    q = rand((3, 4, dim), 133)
    for mode in ("moba", "dense"):
        check(cache, cache.attend(q, sequence_ids=[0, 1, 1], positions=[26, 40, 5], topk=2, mode=mode), q)


@pytest.mark.parametrize("page", [1, 3, 7, 16, 31, 48, 64])
def test_pages_and_chunks_need_not_align(page):
    from moba_opt import PagedKVCache
    cache = PagedKVCache(1, 97, 2, 80, page_size=page, chunk_size=24)
    cache.k_cache.fill_(float("nan"))
    cache.v_cache.fill_(float("nan"))
    k, v = rand((79, 2, 80), 141), rand((79, 2, 80), 142)
    cache.append(k, v, sequence_ids=[0], cu_seqlens=[0, 79])
    assert_payload(cache, 0, k, v)
    q = rand((2, 8, 80), 143)
    for topk in (1, 2, 9):
        check(cache, cache.attend(q, sequence_ids=[0, 0], positions=[0, 78], topk=topk), q)


def test_recycled_pages_and_request_isolation():
    from moba_opt import PagedKVCache
    cache = PagedKVCache(3, 12, 1, 16, page_size=3, num_pages=4, chunk_size=4)
    cache.append(rand((9, 1, 16), 151), rand((9, 1, 16), 152), sequence_ids=[0, 1], cu_seqlens=[0, 6, 9])
    q = rand((1, 4, 16), 153)
    before = cache.attend(q, sequence_ids=[1], mode="dense").output.clone()
    cache.reset([0])
    cache.append(rand((6, 1, 16), 154), rand((6, 1, 16), 155), sequence_ids=[2], cu_seqlens=[0, 6])
    assert cache.page_table[2][:2] == (1, 0)
    assert torch.equal(cache.attend(q, sequence_ids=[1], mode="dense").output, before)
    check(cache, cache.attend(q, sequence_ids=[2], topk=2), q)
    with pytest.raises(ValueError, match="cached tokens"):
        cache.attend(q, sequence_ids=[0])


def test_chunked_append_is_causal():
    from moba_opt import PagedKVCache
    k, v = rand((19, 2, 32), 161), rand((19, 2, 32), 162)
    q = rand((7, 8, 32), 163)
    cache = PagedKVCache(2, 32, 2, 32, page_size=3, chunk_size=4)
    cache.append(torch.cat((k[:5], k[9:16])), torch.cat((v[:5], v[9:16])), sequence_ids=[0, 1], cu_seqlens=[0, 5, 12])
    result = cache.append_and_attend(q, torch.cat((k[5:9], k[16:])), torch.cat((v[5:9], v[16:])), sequence_ids=[0, 1],
                                     cu_seqlens=[0, 4, 7], topk=2)
    assert_payload(cache, 0, k[:9], v[:9])
    assert_payload(cache, 1, k[9:], v[9:])
    assert result.positions == (5, 6, 7, 8, 7, 8, 9)
    check(cache, result, q)
    other = PagedKVCache(2, 32, 2, 32, page_size=3, chunk_size=4)
    k2, v2 = k.clone(), v.clone()
    k2[6:9] = 100
    v2[6:9] = -100
    other.append(k2, v2, sequence_ids=[0, 1], cu_seqlens=[0, 9, 19])
    compare = other.attend(q[:1], sequence_ids=[0], positions=[5], topk=2)
    torch.testing.assert_close(compare.output, result.output[:1], atol=0.02, rtol=0.02)


def test_routing_is_per_query_head_and_uses_only_closed_history():
    from moba_opt import PagedKVCache
    cache = PagedKVCache(1, 16, 2, 8, page_size=3, chunk_size=4)
    k = torch.zeros(13, 2, 8, device="cuda", dtype=cache.dtype)
    for block in range(4):
        k[block * 4:min((block + 1) * 4, 13), 0, 0] = block + 1
        k[block * 4:min((block + 1) * 4, 13), 1, 0] = 4 - block
    cache.append(k, rand(k.shape, 171), sequence_ids=[0], cu_seqlens=[0, 13])
    q = torch.zeros(2, 4, 8, device="cuda", dtype=cache.dtype)
    q[:, :, 0] = 1
    result = cache.attend(q, sequence_ids=[0, 0], positions=[12, 7], topk=3)
    route = result.selected_blocks.cpu()
    assert route[0, 0].tolist() == [3, 2, 1]       # descending score order after the own chunk
    assert route[0, 2].tolist() == [3, 0, 1]
    assert route[1, 0].tolist() == [1, 0, -1]
    check(cache, result, q)


def test_exact_ties_choose_the_lowest_chunk():
    from moba_opt import PagedKVCache
    cache = PagedKVCache(1, 64, 1, 8, page_size=4, chunk_size=4)
    k = torch.ones(33, 1, 8, device="cuda", dtype=cache.dtype)      # every chunk mean identical
    cache.append(k, rand(k.shape, 172), sequence_ids=[0], cu_seqlens=[0, 33])
    q = torch.ones(1, 2, 8, device="cuda", dtype=cache.dtype)
    result = cache.attend(q, sequence_ids=[0], topk=4)
    assert result.selected_blocks[0, 0].tolist() == [8, 0, 1, 2]
    assert result.selected_blocks[0, 1].tolist() == [8, 0, 1, 2]


def test_append_partition_invariance():
    from moba_opt import PagedKVCache
    k, v = rand((25, 2, 24), 181), rand((25, 2, 24), 182)
    a = PagedKVCache(1, 32, 2, 24, page_size=7, chunk_size=6)
    b = PagedKVCache(1, 32, 2, 24, page_size=7, chunk_size=6)
    a.append(k, v, sequence_ids=[0], cu_seqlens=[0, 25])
    for lo, hi in [(0, 1), (1, 5), (5, 13), (13, 25)]:
        b.append(k[lo:hi], v[lo:hi], sequence_ids=[0], cu_seqlens=[0, hi - lo])
    assert torch.equal(a._means[:, :4], b._means[:, :4])
    q = rand((1, 8, 24), 183)
    x, y = a.attend(q, sequence_ids=[0], topk=3), b.attend(q, sequence_ids=[0], topk=3)
    assert torch.equal(x.output, y.output)


@pytest.mark.parametrize("hq,hk", [(8, 1), (8, 2), (28, 4)])
def test_decode_matches_last_prefill_row(hq, hk):
    from moba_opt import PagedKVCache
    from moba_opt.api import run_impl
    q, k, v = rand((97, hq, 64), 191), rand((97, hk, 64), 192), rand((97, hk, 64), 193)
    cu = torch.tensor([0, 97], device="cuda", dtype=torch.int32)
    ref = run_impl("opt_gqa_cuda", q, k, v, cu, 97, {"chunk_size": 16, "topk": 3})[-1:]
    cache = PagedKVCache(1, 128, hk, 64, page_size=7, chunk_size=16)
    cache.append(k, v, sequence_ids=[0], cu_seqlens=[0, 97])
    result = cache.attend(q[-1:], sequence_ids=[0], topk=3)
    torch.testing.assert_close(result.output, ref, atol=0.02, rtol=0.02)
    check(cache, result, q[-1:])


def test_errors_do_not_mutate_cache():
    from moba_opt import PagedKVCache
    cache = PagedKVCache(2, 8, 1, 16, page_size=3, num_pages=1, chunk_size=4)
    q = rand((1, 4, 16), 201)
    with pytest.raises(ValueError, match="cached tokens"):
        cache.attend(q, sequence_ids=[0])
    k, v = rand((3, 1, 16), 202), rand((3, 1, 16), 203)
    cache.append(k, v, sequence_ids=[0], cu_seqlens=[0, 3])
    before = cache.materialize(0)
    with pytest.raises(ValueError, match="pool exhausted"):
        cache.append(k[:1], v[:1], sequence_ids=[1])
    assert cache.lengths == (3, 0)
    for actual, expected in zip(cache.materialize(0), before):
        assert torch.equal(actual, expected)
    with pytest.raises(ValueError, match="inference-only"):
        cache.append_and_attend(q.clone().requires_grad_(True), k[:1], v[:1], sequence_ids=[0])
    with pytest.raises(ValueError, match="NaN/Inf"):
        cache.append(torch.full_like(k[:1], float("nan")), v[:1], sequence_ids=[1])
    assert cache.lengths == (3, 0)


def test_cross_stream_is_rejected():
    from moba_opt import PagedKVCache
    cache = PagedKVCache(1, 8, 1, 8, page_size=3, chunk_size=4)
    k, v = rand((3, 1, 8), 211), rand((3, 1, 8), 212)
    cache.append(k, v, sequence_ids=[0], cu_seqlens=[0, 3])
    q = rand((1, 1, 8), 213)
    with torch.cuda.stream(torch.cuda.Stream()):
        with pytest.raises(ValueError, match="cross-stream"):
            cache.attend(q, sequence_ids=[0])
    check(cache, cache.attend(q, sequence_ids=[0]), q)


def test_long_context_single_token_decode():
    from moba_opt import PagedKVCache
    cache = PagedKVCache(1, 8193, 8, 128, page_size=16, chunk_size=128)
    cache.append(rand((8192, 8, 128), 221), rand((8192, 8, 128), 222), sequence_ids=[0], cu_seqlens=[0, 8192])
    q, k, v = rand((1, 32, 128), 223), rand((1, 8, 128), 224), rand((1, 8, 128), 225)
    result = cache.append_and_attend(q, k, v, sequence_ids=[0], topk=4)
    assert cache.lengths == (8193,) and result.positions == (8192,)
    check(cache, result, q)


@pytest.mark.parametrize("chunk,dim,length,page", [(1, 8, 5, 3), (1024, 256, 1025, 3), (2048, 128, 4500, 48)])
def test_chunk_size_extremes(chunk, dim, length, page):
    from moba_opt import PagedKVCache
    cache = PagedKVCache(1, length + 1, 1, dim, page_size=page, chunk_size=chunk)
    cache.append(rand((length, 1, dim), 231), rand((length, 1, dim), 232), sequence_ids=[0], cu_seqlens=[0, length])
    q = rand((1, 4, dim), 233)
    check(cache, cache.attend(q, sequence_ids=[0], topk=2), q)
    check(cache, cache.attend(q, sequence_ids=[0], mode="dense"), q)


@pytest.mark.parametrize("hq,dim,chunk,length", [(32, 32, 4, 700), (8, 64, 1, 1100), (7, 64, 2, 300)])
def test_dense_merge_over_more_partials_than_fit_in_shared_memory(hq, dim, chunk, length):
    """The merge keeps the weights of a head's partials in shared memory up to a capacity that shrinks with the
    group size; the partials beyond it take the recomputing path.  (32 heads, dim 32: capacity 128 of 176
    partials; 8 heads, dim 64: 1024 of 1101; the last case stays inside the capacity.)"""
    from moba_opt import PagedKVCache
    cache = PagedKVCache(1, length + 1, 1, dim, page_size=16, chunk_size=chunk)
    cache.append(rand((length, 1, dim), 271), rand((length, 1, dim), 272), sequence_ids=[0], cu_seqlens=[0, length])
    q = rand((1, hq, dim), 273)
    check(cache, cache.attend(q, sequence_ids=[0], mode="dense"), q)


@pytest.mark.parametrize("page,chunk,dim,hk", [(16, 32, 64, 2), (7, 24, 40, 3), (48, 128, 128, 1), (3, 1, 8, 2), (16, 512, 64, 2)])
def test_prefill_hand_off_equals_append(page, chunk, dim, hk):
    """`append_prefill` (one launch: pages + means in one pass over K) leaves the cache exactly as `append` does:
    payload, lengths, page table and chunk means bit for bit, for ragged prompts, prompts that continue a sequence in
    the middle of a chunk, and prompts shorter than a chunk."""
    from moba_opt import PagedKVCache
    first = [chunk + 5, 3, 2 * chunk]
    second = [max(2, 3 * chunk - 7), chunk // 2 + 1, 1]
    caches = [PagedKVCache(3, sum(map(max, zip(first, second))) * 2 + 4 * chunk, hk, dim, page_size=page, chunk_size=chunk)
              for _ in range(2)]
    for round_, counts in enumerate((first, second)):
        total = sum(counts)
        k, v = rand((total, hk, dim), 281 + round_), rand((total, hk, dim), 291 + round_)
        cu = [0]
        for n in counts:
            cu.append(cu[-1] + n)
        order = [2, 0, 1] if round_ else [0, 1, 2]
        caches[0].append(k, v, sequence_ids=order, cu_seqlens=cu)
        lengths = caches[1].append_prefill(k, v, sequence_ids=order, cu_seqlens=cu)
        assert caches[0].lengths == caches[1].lengths and caches[0].page_table == caches[1].page_table
        assert lengths == tuple(caches[1].lengths[s] for s in order)
        for sid in range(3):
            a, b = caches[0].materialize(sid), caches[1].materialize(sid)
            assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
            closed = caches[0].lengths[sid] // chunk
            assert torch.equal(caches[0]._means[sid, :closed], caches[1]._means[sid, :closed])
    q = rand((3, 2 * hk, dim), 299)
    check(caches[1], caches[1].attend(q, sequence_ids=[0, 1, 2], topk=3), q)


def test_prefill_hand_off_errors_do_not_mutate_cache():
    from moba_opt import PagedKVCache
    cache = PagedKVCache(1, 64, 1, 8, page_size=4, chunk_size=8)
    k = rand((10, 1, 8), 301)
    cache.append_prefill(k, k.clone(), sequence_ids=[0], cu_seqlens=[0, 10])
    lengths, table = cache.lengths, cache.page_table
    with pytest.raises(ValueError):
        cache.append_prefill(rand((60, 1, 8), 302), rand((60, 1, 8), 303), sequence_ids=[0], cu_seqlens=[0, 60])   # over capacity
    with pytest.raises(ValueError):
        cache.append_prefill(k, k.clone(), sequence_ids=[0], cu_seqlens=[0, 9])                                    # bad cu_seqlens
    assert cache.lengths == lengths and cache.page_table == table
    got = cache.materialize(0)
    assert torch.equal(got[0], k)


def test_extreme_logits_use_stable_online_softmax():
    from moba_opt import PagedKVCache
    cache = PagedKVCache(1, 16, 1, 8, page_size=3, chunk_size=4)
    k = torch.full((13, 1, 8), 1000.0, device="cuda", dtype=cache.dtype)
    k[::2] = -1000
    cache.append(k, rand((13, 1, 8), 241), sequence_ids=[0], cu_seqlens=[0, 13])
    q = torch.full((1, 2, 8), 1000.0, device="cuda", dtype=cache.dtype)
    q[:, 1] = -1000
    check(cache, cache.attend(q, sequence_ids=[0], mode="dense"), q)


def test_maximum_topk_with_nonstandard_heads_and_ragged_queries():
    from moba_opt import PagedKVCache
    cache = PagedKVCache(3, 97, 3, 40, page_size=7, chunk_size=8)
    cache.append(rand((153, 3, 40), 261), rand((153, 3, 40), 262), sequence_ids=[0, 1, 2], cu_seqlens=[0, 81, 88, 153])
    q = rand((4, 15, 40), 263)
    result = cache.attend(q, sequence_ids=[2, 0, 1, 2], positions=[64, 80, 6, 23], topk=9)
    assert result.selected_blocks.shape == (4, 15, 9)
    assert (result.selected_blocks[2, :, 1:] == -1).all()
    check(cache, result, q)


@pytest.mark.parametrize("combined", [False, True])
def test_append_rejects_aliases_before_mutation(combined):
    from moba_opt import PagedKVCache
    cache = PagedKVCache(1, 8, 1, 8, page_size=3, chunk_size=4)
    cache.k_cache.zero_()
    cache.v_cache.zero_()
    alias = cache.k_cache.reshape(-1, 1, 8)[:1]
    external = rand((1, 1, 8), 271)
    with pytest.raises(ValueError, match="must not alias"):
        if combined:
            cache.append_and_attend(alias, external, external, sequence_ids=[0])
        else:
            cache.append(alias, external, sequence_ids=[0])
    assert cache.lengths == (0,)
    cache.append(external, external, sequence_ids=[0])
    assert cache.lengths == (1,)


@pytest.mark.parametrize("kwargs", [{"head_dim": 0}, {"head_dim": 264}, {"head_dim": 33}, {"num_kv_heads": 0}, {"page_size": 0},
                                    {"num_pages": 0}, {"chunk_size": 8193}, {"dtype": torch.float32}, {"dtype": torch.float64},
                                    {"device": "cpu"}])
def test_cache_contract_violations(kwargs):
    from moba_opt import PagedKVCache
    cfg = dict(batch_size=1, max_seq_len=16, num_kv_heads=2, head_dim=64)
    cfg.update(kwargs)
    with pytest.raises(ValueError):
        PagedKVCache(**cfg)
